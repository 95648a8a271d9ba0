"""Name kept from the reference (kernels/triton_adamw.py); the optimizer runs a hand-written sm_100a kernel."""
from llm_systems_from_scratch_b200.optim.adamw import FusedAdamW  # noqa: F401
