"""``llm_systems.parallelism.ddp`` of the reference (llm-systems/llm_systems/parallelism/ddp.py)."""
from llm_systems_from_scratch_b200.parallel.ddp import DDP, GradBucket  # noqa: F401
