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
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # different problems back to back: every later call finds an earlier call's partials in the array.  The shapes
    # cover one to four column groups per thread, the widest row the entry accepts, and fewer rows than blocks.
    for rows, d, seed in [(1000, 2048, 0), (333, 768, 1), (5, 8192, 2), (200, 4104, 3)]:
        x, w, dy, dres = _case(rows, d, seed)
        _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
        ref_dx, ref_dw = native.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
        dx = torch.empty_like(x)
        dw = torch.empty(d, dtype=torch.float32, device="cuda")
        # PyTorch's allocator must stay untouched by the call (a raw cudaMalloc inside the library would not show
        # here; that the entry point makes none is a property of its source, which calls no allocating routine)
        before = torch.cuda.memory_allocated()
        rc = lib.b200_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(),
                                          dx.data_ptr(), dw.data_ptr(), rows, d, 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert (dx.float() - ref_dx.float()).abs().max().item() <= 3e-2
        err = (dw - ref_dw).abs()
        assert bool((err <= 1e-2 * math.sqrt(rows) + 1e-2 * ref_dw.abs()).all()), err.max().item()
        # and against the fp32 PyTorch statement of the same op (the oracle of the other kernel tests)
        o_dx, o_dw = torch_impl.rmsnorm_bwd(dy.float(), x.float(), w.float(), rstd)
        assert (dx.float() - (o_dx + dres.float())).abs().max().item() <= 6e-2
        err = (dw - o_dw).abs()
        assert bool((err <= 2e-2 * math.sqrt(rows) + 2e-2 * o_dw.abs()).all()), err.max().item()
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


def test_noalloc_entry_with_no_rows_and_with_null_outputs():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    d = 512
    w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
    dw = torch.full((d,), 7.0, device="cuda")
    # no rows, accumulate: dw is left as it is; no rows, overwrite: dw becomes the (zero) gradient
    assert lib.b200_rmsnorm_bwd_noalloc(None, None, w.data_ptr(), None, None, None, dw.data_ptr(), 0, d, 1, stream) == 0
    torch.cuda.synchronize()
    assert bool((dw == 7.0).all())
    assert lib.b200_rmsnorm_bwd_noalloc(None, None, w.data_ptr(), None, None, None, dw.data_ptr(), 0, d, 0, stream) == 0
    torch.cuda.synchronize()
    assert bool((dw == 0.0).all())
    # a missing output or a missing rstd is refused before anything is launched
    x = torch.zeros(4, d, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    assert lib.b200_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, x.data_ptr(),
                                        None, 4, d, 0, stream) == -10
    assert lib.b200_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), None, None, x.data_ptr(),
                                        dw.data_ptr(), 4, d, 0, stream) == -10
