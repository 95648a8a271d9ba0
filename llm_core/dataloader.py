"""``llm_core.dataloader`` of the reference (llm-core/llm_core/dataloader.py)."""
from llm_systems_from_scratch_b200.data.loader import BatchSampler, sample_batch  # noqa: F401
