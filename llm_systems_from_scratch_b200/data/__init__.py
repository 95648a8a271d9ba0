from .loader import BatchSampler, sample_batch  # noqa: F401
