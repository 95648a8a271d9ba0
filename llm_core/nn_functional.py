"""``llm_core.nn_functional`` of the reference (llm-core/llm_core/nn_functional.py)."""
from llm_systems_from_scratch_b200.ops.functional import clip_gradient, cross_entropy, log_softmax, softmax  # noqa: F401
