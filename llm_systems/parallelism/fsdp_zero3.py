"""``llm_systems.parallelism.fsdp_zero3`` of the reference (llm-systems/llm_systems/parallelism/fsdp_zero3.py)."""
from llm_systems_from_scratch_b200.parallel.fsdp import FSDP, FSDPUnit  # noqa: F401
