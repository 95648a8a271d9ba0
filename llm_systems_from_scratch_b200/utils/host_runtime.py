"""ctypes front end of the C++ host runtime (``csrc/host/host_runtime.cpp`` -> ``_b200_host.so``).

Used by ``data.loader.BatchSampler`` (window gather into the pinned staging buffer) and by
``serving.kv_cache.PageAllocator`` (free list, slot and block-table arithmetic).  Everything has a pure
Python fallback, so ``available()`` being false only costs speed.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import numpy as np
import torch

_PKG = Path(__file__).resolve().parent.parent
_PATH = _PKG / "_b200_host.so"
_LIB = None
_TRIED = False


def _load():
    global _LIB, _TRIED
    if _LIB is not None or _TRIED:
        return _LIB
    _TRIED = True
    if os.environ.get("B200_HOST_RUNTIME", "1") != "1":
        return None
    try:
        if not _PATH.exists():
            from ..build_ext import build_host
            build_host()
        lib = ctypes.CDLL(str(_PATH))
    except Exception:
        return None
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.b200h_gather_windows.argtypes = [P, L, P, I, I, P, I]
    lib.b200h_pages_create.argtypes = [I]
    lib.b200h_pages_create.restype = P
    lib.b200h_pages_destroy.argtypes = [P]
    lib.b200h_pages_destroy.restype = None
    lib.b200h_pages_free.argtypes = [P]
    lib.b200h_pages_take.argtypes = [P, I, P]
    lib.b200h_pages_give.argtypes = [P, P, I]
    lib.b200h_slots.argtypes = [P, I, I, I, I, P]
    lib.b200h_block_table.argtypes = [P, P, I, I, ctypes.c_int32, P]
    _LIB = lib
    return lib


def available() -> bool:
    return _load() is not None


def gather_windows(tokens: np.ndarray, starts: np.ndarray, width: int, out: torch.Tensor, threads: int = 4):
    """out[b, :] = tokens[starts[b] : starts[b] + width] widened to int64; ``out`` is a CPU (pinned) int64 tensor."""
    lib = _load()
    assert tokens.dtype == np.uint32 and starts.dtype == np.int64 and out.dtype == torch.int64 and out.is_contiguous()
    starts = np.ascontiguousarray(starts)
    rc = lib.b200h_gather_windows(tokens.ctypes.data, tokens.shape[0], starts.ctypes.data, starts.shape[0], width,
                                  out.data_ptr(), threads)
    if rc != 0:
        raise IndexError(f"window gather out of range ({rc})")


class NativePagePool:
    """LIFO page free list in native code (same order as the Python list it replaces)."""

    def __init__(self, num_pages: int):
        self._lib = _load()
        self._h = self._lib.b200h_pages_create(num_pages)
        self.num_pages = num_pages

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.b200h_pages_destroy(self._h)
            self._h = None

    @property
    def free(self) -> int:
        return self._lib.b200h_pages_free(self._h)

    def take(self, n: int) -> list[int]:
        buf = (ctypes.c_int32 * max(n, 1))()
        if self._lib.b200h_pages_take(self._h, n, buf) != 0:
            raise MemoryError(f"out of KV pages: want {n}, have {self.free}")
        return list(buf[:n])

    def give(self, pages: list[int]):
        n = len(pages)
        buf = (ctypes.c_int32 * max(n, 1))(*pages)
        if self._lib.b200h_pages_give(self._h, buf, n) != 0:
            raise ValueError("page id out of range")


def slots(pages: list[int], page_size: int, start: int, count: int) -> list[int]:
    lib = _load()
    pg = (ctypes.c_int32 * max(len(pages), 1))(*pages)
    out = (ctypes.c_int64 * max(count, 1))()
    if lib.b200h_slots(pg, len(pages), page_size, start, count, out) != 0:
        raise IndexError("token range outside the request's pages")
    return list(out[:count])


def block_table(page_lists: list[list[int]], width: int, pad: int = 0) -> torch.Tensor:
    """(rows, width) int32 tensor of page ids, padded with ``pad``."""
    lib = _load()
    flat = [p for pl in page_lists for p in pl]
    offs = [0]
    for pl in page_lists:
        offs.append(offs[-1] + len(pl))
    pg = (ctypes.c_int32 * max(len(flat), 1))(*flat)
    of = (ctypes.c_int32 * len(offs))(*offs)
    table = torch.empty((len(page_lists), width), dtype=torch.int32)
    if lib.b200h_block_table(pg, of, len(page_lists), width, pad, table.data_ptr()) != 0:
        raise ValueError("a request has more pages than the table is wide")
    return table


def block_table_into(page_lists: list[list[int]], table: torch.Tensor, pad: int = 0):
    """Fill the first ``len(page_lists)`` rows of a preallocated int32 CPU table in place; the other rows get ``pad``."""
    lib = _load()
    rows, width = table.shape
    lists = list(page_lists) + [[]] * (rows - len(page_lists))
    flat = [p for pl in lists for p in pl]
    offs = [0]
    for pl in lists:
        offs.append(offs[-1] + len(pl))
    pg = (ctypes.c_int32 * max(len(flat), 1))(*flat)
    of = (ctypes.c_int32 * len(offs))(*offs)
    if lib.b200h_block_table(pg, of, rows, width, pad, table.data_ptr()) != 0:
        raise ValueError("a request has more pages than the table is wide")
