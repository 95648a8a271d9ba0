"""tcgen05 FlashAttention forward/backward against the fp32 PyTorch statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand_qkv(b, s, h, dh, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(b * s, 3 * h * dh, device="cuda", generator=g).bfloat16()


@pytest.mark.parametrize("b,s,h,dh", [(1, 128, 1, 128), (2, 256, 2, 64), (1, 384, 3, 128), (2, 200, 2, 64),
                                      (1, 1024, 4, 128), (3, 72, 2, 32), (1, 2048, 2, 128)])
def test_flash_fwd(b, s, h, dh):
    from llm_systems_from_scratch_b200.ops import attention, native, torch_impl
    qkv = _rand_qkv(b, s, h, dh)
    o, lse = attention.attention_fwd(qkv, b, s, h)
    native.check_status()
    ro, rl = torch_impl.attention_fwd(qkv.float(), b, s, h)
    assert (o.float() - ro).abs().max().item() < 2e-2
    assert (lse - rl).abs().max().item() < 2e-2


@pytest.mark.parametrize("b,s,h,dh", [(1, 128, 1, 128), (2, 256, 2, 64), (1, 384, 3, 128), (2, 200, 2, 64),
                                      (1, 1024, 2, 128), (3, 72, 2, 32)])
def test_flash_bwd(b, s, h, dh):
    from llm_systems_from_scratch_b200.ops import attention, native, torch_impl
    if not native.has("b200_flash_bwd"):
        pytest.skip("backward kernel not built")
    qkv = _rand_qkv(b, s, h, dh, seed=1)
    do = torch.randn(b * s, h * dh, device="cuda").bfloat16()
    o, lse = attention.attention_fwd(qkv, b, s, h)
    dqkv = attention.attention_bwd(do, qkv, o, lse, b, s, h)
    native.check_status()
    ro, rl = torch_impl.attention_fwd(qkv.float(), b, s, h)
    ref = torch_impl.attention_bwd(do.float(), qkv.float(), ro, rl, b, s, h)
    err = (dqkv.float() - ref).abs().max().item()
    assert err < 5e-2 * max(1.0, ref.abs().max().item() / 4), err


def test_flash_varlen_matches_per_sequence():
    from llm_systems_from_scratch_b200.ops import attention, native, torch_impl
    h, dh = 4, 128
    lens = [200, 37, 513, 128]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    qkv = _rand_qkv(1, sum(lens), h, dh, seed=2)
    o = attention.varlen_attention_fwd(qkv, cu, max(lens), h)
    native.check_status()
    ref = torch_impl.varlen_attention_fwd(qkv.float(), cu.cpu(), h)
    assert (o.float() - ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("b,s,h,dh", [(2, 1024, 4, 128), (4, 512, 4, 64)])
def test_rope_fused_into_qkv_gemm_and_attention_backward(b, s, h, dh):
    """QKV GEMM with RoPE in its epilogue, and attention backward that rotates dQ/dK back, against the separate kernels."""
    from llm_systems_from_scratch_b200.models.transformer import RotaryEmbedding
    from llm_systems_from_scratch_b200.ops import attention, native
    d = h * dh
    cache = RotaryEmbedding._build_cache(s + 7, dh, 10000.0).cuda().contiguous()
    x = torch.randn(b * s, d, device="cuda").bfloat16()
    w = (torch.randn(3 * d, d, device="cuda") / d ** 0.5).bfloat16()
    fused = native.gemm_qkv_rope(x, w, cache, s, h)
    assert fused is not None
    ref = native.gemm(x, w, "nt")
    native.rope_(ref, cache, None, h, False, s)
    native.check_status()
    # the fused epilogue rotates fp32 accumulators, the separate kernel rotates bf16-rounded values: <= 2 ulp apart
    assert bool(((fused.float() - ref.float()).abs() <= 2e-2 * ref.float().abs().clamp(min=1.0)).all())
    assert torch.equal(fused[:, 2 * d:], ref[:, 2 * d:])
    o, lse = attention.attention_fwd(ref, b, s, h)
    do = torch.randn_like(o)
    a = attention.attention_bwd(do, ref, o, lse, b, s, h, rope_cache=cache)
    plain = attention.attention_bwd(do, ref, o, lse, b, s, h)
    native.rope_(plain, cache, None, h, True, s)
    native.check_status()
    assert (a.float() - plain.float()).abs().max().item() < 3e-2 * max(1.0, plain.float().abs().max().item())
    assert torch.equal(a[:, 2 * d:], plain[:, 2 * d:])
