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
