"""Names kept from the reference (kernels/triton_swiglu.py); no Triton is involved."""
from llm_systems_from_scratch_b200.models.transformer import FusedSwiGLU  # noqa: F401
from llm_systems_from_scratch_b200.ops.modules import triton_silu_mul  # noqa: F401
