"""``llm_core.model`` of the reference (llm-core/llm_core/model.py) served by the native package."""
from llm_systems_from_scratch_b200.models.transformer import (  # noqa: F401
    CausalMultiHeadSelfAttention, Embedding, FusedSwiGLU, Linear, RMSNorm, RotaryEmbedding, SwiGLU, TransformerBlock,
    TransformerLM, scaled_dot_product_attention, silu)
from llm_systems_from_scratch_b200.ops.functional import softmax  # noqa: F401
