from .adamw import AdamW, FusedAdamW, cosine_lr_schedule  # noqa: F401
