"""Name kept from the reference (kernels/triton_cross_entropy.py); backed by the sm_100a loss kernel."""
from llm_systems_from_scratch_b200.ops.modules import triton_cross_entropy  # noqa: F401
