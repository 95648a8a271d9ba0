"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory where they call it (code running
inside another framework's memory plan, a loop that must stay off the allocator).  For them the
library offers ``b200_rmsnorm_bwd_noalloc``: the per-block weight-gradient partials live in a fixed
array inside the library image, so the caller hands over inputs and outputs only.  This test drives
that symbol with ctypes exactly as such a caller would, twice in a row (the shared array keeps the
first call's contents), and compares with the ordinary entry point whose scratch the caller allocates.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from llm_systems_from_scratch_b200.ops import native
    lib = ctypes.CDLL(str(native.lib_path()))
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.b200_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, P]
    lib.b200_rmsnorm_bwd_noalloc.restype = I
    lib.b200_rmsnorm_bwd_noalloc_max_d.restype = I
    return lib


def _case(rows, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).bfloat16()
    dy = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    dres = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    return x, w, dy, dres


def test_noalloc_entry_matches_allocating_entry_twice_in_a_row():
    from llm_systems_from_scratch_b200.ops import native
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first call's partials in the array
    for rows, d, seed in [(1000, 2048, 0), (333, 768, 1)]:
        x, w, dy, dres = _case(rows, d, seed)
        _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
        ref_dx, ref_dw = native.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
        dx = torch.empty_like(x)
        dw = torch.empty(d, dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = lib.b200_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(),
                                          dx.data_ptr(), dw.data_ptr(), rows, d, 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert (dx.float() - ref_dx.float()).abs().max().item() <= 3e-2
        err = (dw - ref_dw).abs()
        assert bool((err <= 1e-2 * math.sqrt(rows) + 1e-2 * ref_dw.abs()).all()), err.max().item()
        # accumulate mode adds onto what dw already holds
        rc = lib.b200_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None,
                                          dx.data_ptr(), dw.data_ptr(), rows, d, 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        err = (dw - 2 * ref_dw).abs()
        assert bool((err <= 2e-2 * math.sqrt(rows) + 1e-2 * ref_dw.abs()).all()), err.max().item()


def test_noalloc_entry_rejects_widths_beyond_its_maximum():
    lib = _lib()
    max_d = lib.b200_rmsnorm_bwd_noalloc_max_d()
    assert max_d == 8192
    d = max_d + 8
    x = torch.zeros(2, d, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(d, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    dw = torch.full((d,), 7.0, device="cuda")
    rc = lib.b200_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, x.data_ptr(),
                                      dw.data_ptr(), 2, d, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -12                      # refused: nothing was launched, outputs untouched
    torch.cuda.synchronize()
    assert bool((dw == 7.0).all())
