"""ctypes bindings to the sm_100a kernel library (``_b200_kernels.so``).

Every wrapper validates shapes, dtypes, contiguity and alignment on the host *before*
launching (the launchers re-check alignment and return a negative code rather than
faulting), allocates outputs with PyTorch's caching allocator, and launches on the
current CUDA stream.  On a machine with a GPU a missing library is an error, never a
silent fallback.

The kernels stand where the reference has its Triton kernels (llm-systems/llm_systems/kernels/triton_rms_norm.py:30-153,
triton_swiglu.py:27-91, triton_cross_entropy.py:22-145, triton_adamw.py:134-191) and the library calls behind
``Linear`` and attention (llm-core/llm_core/model.py:31-32, 381-385).
"""
from __future__ import annotations

import ctypes
import math
import os
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "_b200_kernels.so"
_STATUS: dict[int, torch.Tensor] = {}

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class KernelError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load(required: bool = True):
    """Load the kernel library once.  ``required`` raises if it is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        if os.environ.get("B200_AUTO_BUILD", "1") == "1":
            try:
                from ..build_ext import build
                build()
            except Exception as e:  # pragma: no cover - build machine specific
                if required:
                    raise KernelError(f"kernel library missing and build failed: {e}") from e
                return None
        if not _LIB_PATH.exists():
            if required:
                raise KernelError(f"kernel library not found at {_LIB_PATH}; run build_ext.build()")
            return None
    lib = ctypes.CDLL(str(_LIB_PATH))
    _declare(lib)
    _LIB = lib
    if os.environ.get("B200_PDL", "1") != "0":
        lib.b200_set_pdl(1)
    return lib


def available() -> bool:
    """True when CUDA is usable and the kernel library loads."""
    if not torch.cuda.is_available():
        return False
    return load(required=True) is not None


def _declare(lib):
    P, I, L, F = c_void_p, c_int, c_ll, c_float
    sigs = {
        "b200_gemm_bf16": [P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, I, P, P],
        "b200_gemm_bf16_pair": [P, P, P, P, I, I, I, L, L, L, L, I, I, I, P, P],
        "b200_gemm_bf16_pair_gather": [P, P, P, P, I, I, I, L, L, L, L, I, I, I, P, P, ctypes.c_ulonglong, I, I, P, P,
                                       P, ctypes.c_uint, P, P],
        "b200_gemm_bf16_splitk": [P, P, P, P, I, I, I, L, L, L, L, I, P, L, P, I, P, P],
        "b200_gemm_splitk_plan": [I, I, I, P, P],
        "b200_gemm_splitk_counters": [],
        "b200_rmsnorm_fwd": [P, P, P, P, I, I, F, P],
        "b200_rmsnorm_set_fwd_rows": [I],
        "b200_rmsnorm_set_bwd_rows": [I],
        "b200_set_pdl": [I],
        "b200_rmsnorm_bwd_parts": [I],
        "b200_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, P],
        "b200_silu_mul_fwd": [P, P, L, I, P],
        "b200_silu_mul_bwd": [P, P, P, L, I, P],
        "b200_rope": [P, P, P, L, I, I, I, I, I, P],
        "b200_embedding_fwd": [P, P, P, L, I, I, P],
        "b200_embedding_bwd": [P, P, P, L, I, I, P],
        "b200_embedding_bwd_sorted": [P, P, P, P, L, I, I, I, P],
        "b200_xent": [P, P, P, P, L, L, I, I, F, I, I, P, P],
        "b200_argmax": [P, L, L, I, P, P],
        "b200_sample_topk": [P, L, L, I, P, F, I, P, P],
        "b200_adamw": [P, P, I, P, P, P, L, P, F, F, F, F, F, F, P],
        "b200_sumsq": [P, I, L, P, P],
        "b200_sumsq_det": [P, I, L, P, P, P],
        "b200_sumsq_scratch": [],
        "b200_clip_coef": [P, F, P, P, P],
        "b200_scale": [P, I, L, P, P],
        "b200_cast_f32_bf16": [P, P, L, P],
        "b200_cast_bf16_f32": [P, P, L, P],
    }
    optional = {
        "b200_flash_fwd": [P, P, P, I, I, I, I, F, P, P],
        "b200_flash_bwd": [P, P, P, P, P, P, I, I, I, I, F, P, P],
        "b200_flash_varlen_fwd": [P, P, P, I, I, I, I, I, F, P, P],
        "b200_flash_bwd_rope": [P, P, P, P, P, P, I, I, I, I, F, P, I, P, P],
        "b200_gemm_bf16_pair_rope": [P, P, P, I, I, I, L, L, L, P, I, I, I, I, P, P],
        "b200_gemm_bf16_pair_swiglu": [P, P, P, P, I, I, I, L, L, L, L, P, P, ctypes.c_ulonglong, I, I, P, P],
        "b200_sample": [P, L, L, I, F, I, P, P, P, P],
    }
    for name, args in {**sigs, **optional}.items():
        fn = getattr(lib, name, None)
        if fn is None:
            if name in sigs:
                raise KernelError(f"symbol {name} missing from {_LIB_PATH}")
            continue
        fn.argtypes = args
        fn.restype = I


def set_pdl(on: bool) -> bool:
    """Launch the kernels of the decode path as programmatic dependents of the kernel before them (their set-up then
    overlaps that kernel's tail; each waits for it to complete before touching global memory).  Returns the previous
    setting."""
    return bool(load().b200_set_pdl(1 if on else 0))


def has(symbol: str) -> bool:
    lib = load(required=False)
    return lib is not None and hasattr(lib, symbol)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def status_word(device=None) -> torch.Tensor:
    """Per-device uint32 status word written by kernels whose bounded waits gave up."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev not in _STATUS:
        _STATUS[dev] = torch.zeros(4, dtype=torch.int32, device=f"cuda:{dev}")
    return _STATUS[dev]


def check_status(device=None):
    """Synchronise and raise if any kernel recorded a wait that ran out."""
    w = status_word(device)
    v = int(w[0].item())
    if v != 0:
        w.zero_()
        for _, counters in _SPLITK_SCRATCH.values():     # a kernel that gave up may have left its tile counters mid-count
            counters.zero_()
        raise KernelError(f"kernel reported error code {v & 0xff} from CTA {v >> 8}")


# Kernels launched per launcher call (a launcher may issue several).  Used to count this package's
# own launches inside a timed region.
_KERNELS_PER_CALL = {"rmsnorm_bwd": 2, "xent": 3, "flash_bwd": 3}
_LAUNCHES = 0


def reset_launch_count():
    global _LAUNCHES
    _LAUNCHES = 0


def launch_count() -> int:
    return _LAUNCHES


def _check(rc: int, name: str):
    global _LAUNCHES
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")
    _LAUNCHES += _KERNELS_PER_CALL.get(name, 1)


def _req(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


def _rowmajor(t: torch.Tensor, name: str):
    _req(t.dim() == 2 and t.stride(1) == 1, f"{name} must be 2-D with unit inner stride")


# ----------------------------------------------------------------------------- GEMM
EPI_BF16, EPI_F32, EPI_BF16_RES, EPI_F32_ACC, EPI_SWIGLU_BWD = 0, 1, 2, 3, 4
EPI_PAD_WRITABLE = 0x100
EPI_B_STABLE = 0x200


# Problems at least this large (rows of the output) run on CTA pairs (cta_group::2, 256 x 256 tiles).
PAIR_MIN_M = int(os.environ.get("B200_GEMM_PAIR_MIN_M", "1024"))
FUSE_ROPE = os.environ.get("B200_FUSE_ROPE", "1") == "1"                # RoPE in the QKV GEMM epilogue
FUSE_SWIGLU_FWD = os.environ.get("B200_FUSE_SWIGLU_FWD", "1") == "1"    # SiLU*mul in the gate|up GEMM epilogue
# The SiLU*mul backward can run in the epilogue of the W2 dgrad GEMM, but measured on the 1.3B step it is 1.3 %
# slower than GEMM + stand-alone kernel (the 128 epilogue threads of a CTA become the bottleneck), so it is opt-in.
FUSE_SWIGLU_BWD = os.environ.get("B200_FUSE_SWIGLU_BWD", "0") == "1"
USE_PAIR = os.environ.get("B200_GEMM_PAIR", "1") == "1"
# Tests of the GEMM-carried collectives run tiny models: this switch sends every GEMM whose default would be the
# single-CTA kernel to the CTA-pair kernel as well (it handles any shape; small ones just fill fewer SMs).
FORCE_PAIR = os.environ.get("B200_GEMM_FORCE_PAIR", "0") == "1"


def _pair_pays(m: int, n: int, sms: int = 148) -> bool:
    """Wave model of the two tensor-core kernels.  A 256x256 tile on a CTA pair is the unit of time; a 128x128
    tile on one SM is a quarter of the work on half the hardware at about 0.8 of the efficiency.  Small weight
    gradients (a few dozen pair tiles) fill the GPU better with the single-CTA kernel."""
    waves = lambda tiles, slots: -(-tiles // slots)
    cost_pair = waves(-(-m // 256) * -(-n // 256), sms // 2)
    cost_single = waves(-(-m // 128) * -(-n // 128), sms) * 0.625
    return cost_pair <= cost_single


def set_gemm_tma_store(on: bool) -> bool:
    """Switch the CTA-pair GEMM epilogue between TMA stores from shared memory (default) and direct register
    stores; returns the previous setting."""
    lib = load()
    lib.b200_gemm_set_tma_store.argtypes = [c_int]
    lib.b200_gemm_set_tma_store.restype = c_int
    return bool(lib.b200_gemm_set_tma_store(1 if on else 0))


def _task_descs(gather, reduce):
    """ctypes descriptions of the collectives a CTA-pair GEMM launch is about to carry (None where there is none)."""
    from ..parallel.peer import GatherDesc
    gdesc = None
    if gather is not None:
        table, dst, nbytes, world, rank = gather
        gdesc = GatherDesc()
        for r in range(world):
            gdesc.src[r] = table[r]
        gdesc.dst, gdesc.shard_bytes, gdesc.world, gdesc.rank = dst, nbytes, world, rank
    return gdesc, (reduce.desc if reduce is not None else None)


def _gemm_pair_tasks(lib, a, b, out, r, m, n, k, lda, ldb, ldc, ldr, a_mn, b_mn, epi, gargs, reduce):
    gdesc, rdesc = _task_descs(gargs, reduce)
    fn = lib.b200_gemm_bf16_pair_tasks
    if not getattr(fn, "_declared", False):
        P, I, L = c_void_p, c_int, c_ll
        fn.argtypes = [P, P, P, P, I, I, I, L, L, L, L, I, I, I, P, P, P, P]
        fn.restype = I
        fn._declared = True
    rc = fn(_ptr(a), _ptr(b), _ptr(out), _ptr(r), m, n, k, lda, ldb, ldc, ldr, a_mn, b_mn, epi,
            ctypes.byref(gdesc) if gdesc is not None else None, ctypes.byref(rdesc) if rdesc is not None else None,
            _ptr(status_word(a.device)), _stream())
    _check(rc, "b200_gemm_bf16_pair_tasks")


def gemm(a, b, layout: str, out=None, out_dtype=None, residual=None, accumulate=False, bn_hint=0, max_ctas=0,
         pair=None, gather=None, pad_writable=False, reduce=None, b_stable=False):
    """bf16 tensor-core GEMM (tcgen05).  layout 'nt' | 'nn' | 'tn' as in ``torch_impl.gemm``.

    ``pair`` forces (True) or forbids (False) the CTA-pair kernel; by default large problems use it.
    ``gather`` / ``reduce``: a pending all-gather / reduce-scatter (``parallel.comm.GatherTask`` /
    ``ReduceScatterTask``) that the CTA-pair kernel carries on its copy warps; a launch that cannot carry them
    performs them first as collectives of their own.
    ``b_stable``: ``b`` is not written by the kernel launched before this one on the stream (inference weights); the
    single-CTA kernel then requests its first weight tiles before it waits for that kernel (programmatic dependent
    launch), so the weights' DRAM latency overlaps the predecessor's tail.
    ``pad_writable``: ``out`` is a column slice of a wider buffer and the columns from N up to the next 16-byte
    boundary (inside the row pitch) may be overwritten with zeros; this lets a row count that is not a multiple of
    16 bytes (a vocabulary of 50,257) use the TMA-store epilogue."""
    lib = load()
    _req(a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm inputs must be bf16")
    _rowmajor(a, "a")
    _rowmajor(b, "b")
    if layout == "nt":
        m, k = a.shape
        n, kb = b.shape
        a_mn, b_mn = 0, 0
    elif layout == "nn":
        m, k = a.shape
        kb, n = b.shape
        a_mn, b_mn = 0, 1
    elif layout == "tn":
        k, m = a.shape
        kb, n = b.shape
        a_mn, b_mn = 1, 1
    else:
        raise ValueError(layout)
    _req(k == kb, f"contraction mismatch {k} vs {kb}")
    lda, ldb = a.stride(0), b.stride(0)
    _req(lda % 8 == 0 and ldb % 8 == 0, "leading dimensions must be multiples of 8 elements")
    _req(a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0, "operands must be 16-byte aligned")
    if out is None:
        dt = out_dtype or torch.bfloat16
        out = torch.empty((m, n), dtype=dt, device=a.device)
    else:
        _rowmajor(out, "out")
        _req(tuple(out.shape) == (m, n), f"out shape {tuple(out.shape)} != {(m, n)}")
    if out.dtype == torch.bfloat16:
        _req(not accumulate, "accumulate needs an fp32 output")
        epi = EPI_BF16_RES if residual is not None else EPI_BF16
    elif out.dtype == torch.float32:
        _req(residual is None, "residual needs a bf16 output")
        epi = EPI_F32_ACC if accumulate else EPI_F32
    else:
        raise ValueError("out must be bf16 or fp32")
    ldr = 0
    if residual is not None:
        _rowmajor(residual, "residual")
        _req(residual.dtype == torch.bfloat16 and tuple(residual.shape) == (m, n), "residual must be bf16 (M,N)")
        ldr = residual.stride(0)
    if pair is None:
        pair = USE_PAIR and bn_hint == 0 and max_ctas == 0 and (
            FORCE_PAIR or (m >= PAIR_MIN_M and n >= 256 and _pair_pays(m, n)))
    gargs = gather.native_args() if (gather is not None and not gather.done) else None
    if gather is not None and not gather.done and (gargs is None or not pair):
        gather.run()           # this launch cannot carry it: stand-alone collective
        gargs = None
    if reduce is not None and not reduce.done and (reduce.desc is None or not pair):
        reduce.run()
    if pair and pad_writable:
        per16 = 16 // out.element_size()
        if -(-n // per16) * per16 <= out.stride(0):
            epi |= EPI_PAD_WRITABLE
    carry_reduce = reduce if (reduce is not None and not reduce.done) else None
    if pair and (gargs is not None or carry_reduce is not None):
        _gemm_pair_tasks(lib, a, b, out, residual, m, n, k, lda, ldb, out.stride(0), ldr, a_mn, b_mn, epi, gargs,
                         carry_reduce)
        if gargs is not None:
            gather.mark_done(carried=True)
        if carry_reduce is not None:
            carry_reduce.mark_done()
        return out
    if pair:
        rc = lib.b200_gemm_bf16_pair(_ptr(a), _ptr(b), _ptr(out), _ptr(residual), m, n, k, lda, ldb, out.stride(0),
                                     ldr, a_mn, b_mn, epi, _ptr(status_word(a.device)), _stream())
        _check(rc, "b200_gemm_bf16_pair")
        return out
    if b_stable and layout == "nt":
        epi |= EPI_B_STABLE
    if USE_SPLITK and layout == "nt" and m <= SPLITK_MAX_M and k >= SPLITK_MIN_K and bn_hint == 0 and max_ctas == 0:
        scratch = _splitk_scratch(a.device)
        if scratch is not None:
            ws, counters = scratch
            rc = lib.b200_gemm_bf16_splitk(_ptr(a), _ptr(b), _ptr(out), _ptr(residual), m, n, k, lda, ldb, out.stride(0),
                                           ldr, epi, _ptr(ws), ws.numel(), _ptr(counters), counters.numel(),
                                           _ptr(status_word(a.device)), _stream())
            _check(rc, "b200_gemm_bf16_splitk")
            return out
    rc = lib.b200_gemm_bf16(_ptr(a), _ptr(b), _ptr(out), _ptr(residual), m, n, k, lda, ldb, out.stride(0), ldr,
                            a_mn, b_mn, epi, bn_hint, max_ctas, _ptr(status_word(a.device)), _stream())
    _check(rc, "b200_gemm_bf16")
    return out


# Split-K for GEMMs with at most two rows of tiles (decode).  One scratch (partial tiles, tile counters) per device,
# kept for the life of the process because captured CUDA graphs hold its address.  Launches that use it must be
# ordered with respect to each other: this package issues its GEMMs of a device on one stream at a time (the serving
# engine replays its graphs on the stream that also runs the prefills), so they are; a caller that runs small-M
# GEMMs on two streams at once must switch split-K off (B200_SPLITK=0).  The scratch is created outside CUDA-graph
# capture only (memory allocated during a capture belongs to that graph's pool): a capture that comes first falls
# back to the plain kernel.
USE_SPLITK = os.environ.get("B200_SPLITK", "1") != "0"
SPLITK_MAX_M = 256
SPLITK_MIN_K_DEFAULT = 4096      # measured: splitting pays for the long contractions (the down projection) only
SPLITK_MIN_K = SPLITK_MIN_K_DEFAULT
_SPLITK_SCRATCH: dict = {}


def _splitk_scratch(device):
    key = torch.device(device).index
    got = _SPLITK_SCRATCH.get(key)
    if got is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        lib = load()
        lib.b200_gemm_splitk_ws_floats.restype = c_ll
        ws = torch.empty(int(lib.b200_gemm_splitk_ws_floats()), dtype=torch.float32, device=device)
        counters = torch.zeros(int(lib.b200_gemm_splitk_counters()), dtype=torch.int32, device=device)
        got = _SPLITK_SCRATCH[key] = (ws, counters)
    return got


def splitk_plan(m: int, n: int, k: int) -> tuple[int, int]:
    """(tile width, K slices) the split-K launcher picks for an (m, n, k) problem; slices == 1 means the plain kernel."""
    bn, s = c_int(0), c_int(1)
    load().b200_gemm_splitk_plan(m, n, k, ctypes.byref(bn), ctypes.byref(s))
    return bn.value, s.value


def gemm_qkv_rope(x, wqkv, cos_sin, seq: int, n_heads: int):
    """qkv = x @ wqkv.T with the rotary embedding applied to the Q and K thirds in the GEMM epilogue.
    Returns None when the fused kernel does not apply (the caller then runs GEMM + rope separately)."""
    lib = load()
    m, k = x.shape
    n = wqkv.shape[0]
    d = n // 3
    dh = d // n_heads
    ok = (USE_PAIR and FUSE_ROPE and (m >= PAIR_MIN_M or FORCE_PAIR) and dh % 32 == 0 and m % seq == 0 and seq <= cos_sin.shape[1]
          and x.dtype == torch.bfloat16 and wqkv.dtype == torch.bfloat16 and x.stride(1) == 1 and wqkv.stride(1) == 1
          and x.stride(0) % 8 == 0 and wqkv.stride(0) % 8 == 0 and cos_sin.is_contiguous()
          and cos_sin.dtype == torch.float32 and cos_sin.shape[2] == dh // 2)
    if not ok:
        return None
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    rc = lib.b200_gemm_bf16_pair_rope(_ptr(x), _ptr(wqkv), _ptr(out), m, n, k, x.stride(0), wqkv.stride(0), n,
                                      _ptr(cos_sin), seq, d, dh, cos_sin.shape[1], _ptr(status_word(x.device)),
                                      _stream())
    _check(rc, "b200_gemm_bf16_pair_rope")
    return out


def gemm_swiglu(x, wgu, gather=None):
    """(gu, h) with gu = x @ wgu.T (gate columns then up columns) and h = silu(gate) * up, in one kernel.
    Returns None when the fused kernel does not apply.  A pending all-gather can ride on the launch."""
    lib = load()
    m, k = x.shape
    two_f = wgu.shape[0]
    f = two_f // 2
    ok = (USE_PAIR and FUSE_SWIGLU_FWD and (m >= PAIR_MIN_M or FORCE_PAIR) and f % 128 == 0 and x.dtype == torch.bfloat16 and wgu.dtype == torch.bfloat16
          and x.stride(1) == 1 and wgu.stride(1) == 1 and x.stride(0) % 8 == 0 and wgu.stride(0) % 8 == 0)
    if not ok:
        return None
    gu = torch.empty((m, two_f), dtype=torch.bfloat16, device=x.device)
    h = torch.empty((m, f), dtype=torch.bfloat16, device=x.device)
    gargs = gather.native_args() if (gather is not None and not gather.done) else None
    if gather is not None and not gather.done and gargs is None:
        gather.run()
    table, dst, nbytes, world, rank = gargs if gargs is not None else (None, None, 0, 0, 0)
    rc = lib.b200_gemm_bf16_pair_swiglu(_ptr(x), _ptr(wgu), _ptr(gu), _ptr(h), m, f, k, x.stride(0), wgu.stride(0),
                                        two_f, f, table, dst, nbytes, world, rank, _ptr(status_word(x.device)),
                                        _stream())
    _check(rc, "b200_gemm_bf16_pair_swiglu")
    if gargs is not None:
        gather.mark_done(carried=True)
    return gu, h


def gemm_swiglu_bwd(dy, wdown, gu, gather=None):
    """d(gate | up) of h = silu(gate) * up for dh = dy @ wdown, with the element-wise backward done in the
    GEMM epilogue (dh is never written).  dy (M, d), wdown (d, F), gu (M, 2F) -> (M, 2F), all bf16.
    Returns None when the fused kernel does not apply.  A pending all-gather can ride on the launch."""
    lib = load()
    m, k = dy.shape
    kb, f = wdown.shape
    ok = (USE_PAIR and FUSE_SWIGLU_BWD and (m >= PAIR_MIN_M or FORCE_PAIR) and f >= 256 and f % 8 == 0 and k == kb and tuple(gu.shape) == (m, 2 * f)
          and dy.dtype == torch.bfloat16 and wdown.dtype == torch.bfloat16 and gu.dtype == torch.bfloat16
          and dy.stride(1) == 1 and wdown.stride(1) == 1 and gu.stride(1) == 1 and dy.stride(0) % 8 == 0
          and wdown.stride(0) % 8 == 0 and gu.stride(0) % 8 == 0 and gu.data_ptr() % 16 == 0
          and dy.data_ptr() % 16 == 0 and wdown.data_ptr() % 16 == 0)
    if not ok:
        return None
    dgu = torch.empty((m, 2 * f), dtype=torch.bfloat16, device=dy.device)
    gargs = gather.native_args() if (gather is not None and not gather.done) else None
    if gather is not None and not gather.done and gargs is None:
        gather.run()
    if gargs is not None:
        _gemm_pair_tasks(lib, dy, wdown, dgu, gu, m, f, k, dy.stride(0), wdown.stride(0), 2 * f, gu.stride(0), 0, 1,
                         EPI_SWIGLU_BWD, gargs, None)
        gather.mark_done(carried=True)
    else:
        rc = lib.b200_gemm_bf16_pair(_ptr(dy), _ptr(wdown), _ptr(dgu), _ptr(gu), m, f, k, dy.stride(0), wdown.stride(0),
                                     2 * f, gu.stride(0), 0, 1, EPI_SWIGLU_BWD, _ptr(status_word(dy.device)), _stream())
        _check(rc, "b200_gemm_bf16_pair")
    return dgu


# -------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x, w, eps: float):
    lib = load()
    _req(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "rmsnorm inputs must be bf16")
    _req(x.is_contiguous() and w.is_contiguous(), "rmsnorm inputs must be contiguous")
    d = x.shape[-1]
    rows = x.numel() // d
    _req(w.numel() == d and d % 8 == 0, "bad rmsnorm width")
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(lib.b200_rmsnorm_fwd(_ptr(x), _ptr(w), _ptr(y), _ptr(rstd), rows, d, float(eps), _stream()), "rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy, x, w, rstd, dw_out=None, accumulate=False, dres=None):
    lib = load()
    _req(dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "bf16 expected")
    _req(dy.is_contiguous() and x.is_contiguous(), "contiguous expected")
    d = x.shape[-1]
    rows = x.numel() // d
    _req(d % 8 == 0 and d <= 8192, "rmsnorm_bwd supports widths that are multiples of 8 up to 8192")
    _req(rstd.numel() == rows and rstd.dtype == torch.float32, "bad rstd")
    dx = torch.empty_like(x)
    dw = dw_out if dw_out is not None else torch.empty(d, dtype=torch.float32, device=x.device)
    _req(dw.dtype == torch.float32 and dw.numel() == d and dw.is_contiguous(), "dw must be fp32 (d,)")
    if dres is not None:
        _req(dres.dtype == torch.bfloat16 and dres.is_contiguous() and dres.numel() == x.numel(), "bad dres")
    parts = lib.b200_rmsnorm_bwd_parts(rows)
    scratch = torch.empty(parts * d, dtype=torch.float32, device=x.device)
    _check(lib.b200_rmsnorm_bwd(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(dx), _ptr(dw), _ptr(scratch), rows, d,
                                1 if accumulate else 0, _stream()), "rmsnorm_bwd")
    return dx, dw


# --------------------------------------------------------------------------- SwiGLU
def silu_mul_fwd(gu):
    lib = load()
    _req(gu.dtype == torch.bfloat16 and gu.dim() == 2 and gu.is_contiguous(), "gu must be contiguous bf16 (M, 2F)")
    rows, two_f = gu.shape
    f = two_f // 2
    _req(two_f % 2 == 0 and f % 8 == 0, "F must be a multiple of 8")
    h = torch.empty((rows, f), dtype=gu.dtype, device=gu.device)
    _check(lib.b200_silu_mul_fwd(_ptr(gu), _ptr(h), rows, f, _stream()), "silu_mul_fwd")
    return h


def silu_mul_bwd(dh, gu):
    lib = load()
    rows, two_f = gu.shape
    f = two_f // 2
    _req(dh.dtype == torch.bfloat16 and dh.is_contiguous() and tuple(dh.shape) == (rows, f), "bad dh")
    _req(gu.dtype == torch.bfloat16 and gu.is_contiguous() and f % 8 == 0, "bad gu")
    dgu = torch.empty_like(gu)
    _check(lib.b200_silu_mul_bwd(_ptr(dh), _ptr(gu), _ptr(dgu), rows, f, _stream()), "silu_mul_bwd")
    return dgu


# ----------------------------------------------------------------------------- RoPE
def rope_(qkv, cos_sin, positions, n_heads: int, inverse: bool = False, seq: int | None = None):
    """positions: (M,) int32 tensor, or None with ``seq`` given (position = row % seq)."""
    lib = load()
    _req(qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.is_contiguous(), "qkv must be contiguous bf16")
    rows, three_d = qkv.shape
    d = three_d // 3
    dh = d // n_heads
    _req(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[0] == 2, "bad rope cache")
    ctx = cos_sin.shape[1]
    _req(cos_sin.shape[2] == dh // 2 and dh % 8 == 0, "head dim must be a multiple of 8 and match the cache")
    if positions is not None:
        _req(positions.dtype == torch.int32 and positions.numel() == rows and positions.is_contiguous(),
             "positions must be int32 (M,)")
        seq_arg = 1
    else:
        _req(seq is not None and seq <= ctx and rows % seq == 0, "seq must divide rows and fit the rope cache")
        seq_arg = seq
    _check(lib.b200_rope(_ptr(qkv), _ptr(cos_sin), _ptr(positions), rows, seq_arg, d, dh, ctx, 1 if inverse else 0,
                         _stream()), "rope")
    return qkv


# ------------------------------------------------------------------------ Embedding
def embedding_fwd(tokens, weight, out_dtype=None):
    lib = load()
    _req(tokens.dtype == torch.int64 and tokens.is_contiguous(), "tokens must be contiguous int64")
    _req(weight.dtype == torch.bfloat16 and weight.is_contiguous() and weight.dim() == 2, "table must be bf16 (V,d)")
    v, d = weight.shape
    rows = tokens.numel()
    out = torch.empty((rows, d), dtype=torch.bfloat16, device=weight.device)
    _check(lib.b200_embedding_fwd(_ptr(tokens), _ptr(weight), _ptr(out), rows, d, v, _stream()), "embedding_fwd")
    return out


def embedding_bwd(dx, tokens, grad_weight, accumulate=False, deterministic=True):
    """Scatter-add of dx rows into the fp32 gradient table.  The default sorts the token ids (stable device sort)
    and adds every run of equal ids in order inside one warp: no atomics, bitwise reproducible.
    ``deterministic=False`` uses 16-byte vector atomics instead (one launch, no sort)."""
    lib = load()
    _req(dx.dtype == torch.bfloat16 and dx.is_contiguous(), "dx must be contiguous bf16")
    _req(tokens.dtype == torch.int64 and tokens.is_contiguous(), "tokens must be contiguous int64")
    v, d = grad_weight.shape
    rows = tokens.numel()
    _req(dx.numel() == rows * d, "dx shape mismatch")
    if grad_weight.dtype == torch.bfloat16:
        # bf16 gradient staging (multi-GPU): each row is written once from the fp32 sum of its run
        _req(grad_weight.is_contiguous() and deterministic and not accumulate,
             "a bf16 gradient table is written by the deterministic kernel only, without accumulation")
        grad_weight.zero_()
        sorted_tokens, order = torch.sort(tokens.reshape(-1), stable=True)
        fn = lib.b200_embedding_bwd_sorted_bf16
        fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]
        fn.restype = c_int
        _check(fn(_ptr(sorted_tokens), _ptr(order), _ptr(dx), _ptr(grad_weight), rows, d, v, _stream()),
               "embedding_bwd_sorted")
        return grad_weight
    _req(grad_weight.dtype == torch.float32 and grad_weight.is_contiguous(), "grad table must be fp32")
    if not accumulate:
        grad_weight.zero_()
    if deterministic:
        flat = tokens.reshape(-1)
        sorted_tokens, order = torch.sort(flat, stable=True)
        _check(lib.b200_embedding_bwd_sorted(_ptr(sorted_tokens), _ptr(order), _ptr(dx), _ptr(grad_weight), rows, d, v,
                                             1 if accumulate else 0, _stream()), "embedding_bwd_sorted")
        return grad_weight
    _check(lib.b200_embedding_bwd(_ptr(tokens), _ptr(dx), _ptr(grad_weight), rows, d, v, _stream()), "embedding_bwd")
    return grad_weight


# -------------------------------------------------------------------- Cross entropy
def xent_fwd_bwd(logits, targets, grad_scale: float = 1.0, ignore_index: int = -100, valid_cols=None,
                 write_grad: bool = True, loss_out=None, accumulate_loss=False, n_valid=None):
    lib = load()
    _req(logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be bf16 2-D")
    rows, cols = logits.shape
    ld = logits.stride(0)
    v = valid_cols or cols
    _req(ld % 8 == 0 and v <= ld, "logits row stride must be a multiple of 8 elements")
    _req(targets.dtype == torch.int64 and targets.numel() == rows and targets.is_contiguous(), "bad targets")
    loss = loss_out if loss_out is not None else torch.empty((), dtype=torch.float32, device=logits.device)
    scratch = torch.empty(rows + 1, dtype=torch.float32, device=logits.device)
    _check(lib.b200_xent(_ptr(logits), _ptr(targets), _ptr(loss), _ptr(scratch), rows, ld, v, ignore_index,
                         float(grad_scale), 1 if write_grad else 0, 1 if accumulate_loss else 0, _ptr(n_valid),
                         _stream()), "xent")
    return loss


def xent_fwd(logits, targets, ignore_index: int = -100, valid_cols=None, loss_out=None, accumulate_loss=False,
             n_valid=None):
    return xent_fwd_bwd(logits, targets, 1.0, ignore_index, valid_cols, write_grad=False, loss_out=loss_out,
                        accumulate_loss=accumulate_loss, n_valid=n_valid)


def argmax_rows(logits, valid_cols=None):
    lib = load()
    _req(logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be bf16 2-D")
    rows, cols = logits.shape
    out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _check(lib.b200_argmax(_ptr(logits), rows, logits.stride(0), valid_cols or cols, _ptr(out), _stream()), "argmax")
    return out


# ---------------------------------------------------------------------------- AdamW
def sample_topk(logits, uniforms, temperature: float, top_k: int | None = None, valid_cols=None):
    """One token id per row: softmax(logits / temperature) restricted to the top-k logits (ties kept), drawn by
    inverse CDF with the caller's uniforms in [0, 1).  logits (rows, cols) bf16, uniforms (rows,) fp32 -> int64."""
    lib = load()
    _req(logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be bf16 2-D")
    rows, cols = logits.shape
    _req(uniforms.dtype == torch.float32 and uniforms.numel() == rows and uniforms.is_contiguous(), "bad uniforms")
    _req(temperature > 0, "temperature must be positive (use argmax_rows for greedy decoding)")
    out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _check(lib.b200_sample_topk(_ptr(logits), rows, logits.stride(0), valid_cols or cols, _ptr(uniforms),
                                float(temperature), int(top_k or 0), _ptr(out), _stream()), "sample_topk")
    return out


def adamw_step(master, grad, m, v, mirror, lr, beta1, beta2, eps, weight_decay, step: int, grad_scale=None):
    lib = load()
    n = master.numel()
    _req(master.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32, "state must be fp32")
    _req(master.is_contiguous() and grad.is_contiguous() and m.is_contiguous() and v.is_contiguous(), "contiguous")
    _req(grad.numel() == n and m.numel() == n and v.numel() == n, "size mismatch")
    _req(grad.dtype in (torch.float32, torch.bfloat16), "grad must be fp32 or bf16")
    if mirror is not None:
        _req(mirror.dtype == torch.bfloat16 and mirror.numel() == n and mirror.is_contiguous(), "bad mirror")
    if grad_scale is not None:
        _req(grad_scale.dtype == torch.float32 and grad_scale.numel() == 1, "grad_scale must be a device float")
    alpha_t = lr * math.sqrt(1 - beta2 ** step) / (1 - beta1 ** step)
    _check(lib.b200_adamw(_ptr(master), _ptr(grad), 1 if grad.dtype == torch.bfloat16 else 0, _ptr(m), _ptr(v),
                          _ptr(mirror), n, _ptr(grad_scale), float(lr), float(beta1), float(beta2), float(eps),
                          float(weight_decay), float(alpha_t), _stream()), "adamw")


def sumsq(x, out=None):
    lib = load()
    _req(x.is_contiguous() and x.dtype in (torch.float32, torch.bfloat16), "sumsq needs contiguous fp32/bf16")
    if out is None:
        out = torch.zeros((), dtype=torch.float32, device=x.device)
    # per-block partials added in index order: the gradient norm is bitwise reproducible
    scratch = torch.empty(lib.b200_sumsq_scratch(), dtype=torch.float32, device=x.device)
    _check(lib.b200_sumsq_det(_ptr(x), 1 if x.dtype == torch.bfloat16 else 0, x.numel(), _ptr(out), _ptr(scratch),
                              _stream()), "sumsq")
    return out


def clip_coef(sumsq_t, max_norm: float, coef_out=None, norm_out=None):
    lib = load()
    if coef_out is None:
        coef_out = torch.empty((), dtype=torch.float32, device=sumsq_t.device)
    _check(lib.b200_clip_coef(_ptr(sumsq_t), float(max_norm), _ptr(coef_out), _ptr(norm_out), _stream()), "clip_coef")
    return coef_out


def scale_(x, coef):
    lib = load()
    _req(x.is_contiguous() and x.dtype in (torch.float32, torch.bfloat16), "scale needs contiguous fp32/bf16")
    _req(torch.is_tensor(coef) and coef.dtype == torch.float32 and coef.numel() == 1, "coef must be a device float")
    _check(lib.b200_scale(_ptr(x), 1 if x.dtype == torch.bfloat16 else 0, x.numel(), _ptr(coef), _stream()), "scale")
    return x


def cast_copy(dst, src):
    lib = load()
    _req(dst.is_contiguous() and src.is_contiguous() and dst.numel() == src.numel(), "cast needs equal contiguous")
    if src.dtype == torch.float32 and dst.dtype == torch.bfloat16:
        _check(lib.b200_cast_f32_bf16(_ptr(src), _ptr(dst), src.numel(), _stream()), "cast")
    elif src.dtype == torch.bfloat16 and dst.dtype == torch.float32:
        _check(lib.b200_cast_bf16_f32(_ptr(src), _ptr(dst), src.numel(), _stream()), "cast")
    else:
        dst.copy_(src)
    return dst
