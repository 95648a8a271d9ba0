"""``llm_core.optimizer`` of the reference (llm-core/llm_core/optimizer.py)."""
from llm_systems_from_scratch_b200.optim.adamw import AdamW, cosine_lr_schedule  # noqa: F401
