"""Name kept from the reference (kernels/triton_rms_norm.py); backed by the sm_100a RMSNorm kernels."""
from llm_systems_from_scratch_b200.ops.modules import TritonRMSNorm  # noqa: F401
