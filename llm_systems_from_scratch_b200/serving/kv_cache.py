"""Paged KV cache: fixed-size pages (16 tokens by default), a free-list allocator and per-request
block tables.  The reference keeps no KV cache (its ``generate`` recomputes the whole context for
every token, llm-core/llm_core/model.py:210-233); everything here is new capability.

Memory: one K and one V tensor of shape (layers, num_pages, page_size, d_model) in bf16.  For the
1.3B model a page costs 2 * 24 * 16 * 2048 * 2 B = 3 MiB over all layers, so a 180 GB GPU holds tens
of thousands of pages next to the 2.8 GB of weights.
"""
from __future__ import annotations

import torch


class PageAllocator:
    """LIFO free list over page ids.  The list lives in the C++ host runtime when that library is available
    (``utils.host_runtime``), otherwise in a Python list; both hand pages out in the same order."""

    def __init__(self, num_pages: int, native: bool | None = None):
        self.num_pages = num_pages
        self._pool = None
        if native is not False:
            try:
                from ..utils import host_runtime
                if host_runtime.available():
                    self._pool = host_runtime.NativePagePool(num_pages)
            except Exception:
                self._pool = None
        if native is True and self._pool is None:
            raise RuntimeError("host runtime library is not available")
        self._free = list(range(num_pages - 1, -1, -1)) if self._pool is None else None

    @property
    def free(self) -> int:
        return self._pool.free if self._pool is not None else len(self._free)

    def take(self, n: int) -> list[int]:
        if self._pool is not None:
            return self._pool.take(n)
        if n > len(self._free):
            raise MemoryError(f"out of KV pages: want {n}, have {len(self._free)}")
        out = self._free[-n:][::-1] if n else []
        del self._free[len(self._free) - n:]
        return out

    def give(self, pages: list[int]):
        if self._pool is not None:
            return self._pool.give(pages)
        self._free.extend(reversed(pages))


class PagedKVCache:
    def __init__(self, n_layers: int, d_model: int, num_pages: int, page_size: int = 16, device="cuda",
                 dtype=torch.bfloat16):
        self.n_layers, self.d_model, self.page_size, self.num_pages = n_layers, d_model, page_size, num_pages
        self.k = torch.zeros((n_layers, num_pages, page_size, d_model), dtype=dtype, device=device)
        self.v = torch.zeros((n_layers, num_pages, page_size, d_model), dtype=dtype, device=device)
        self.allocator = PageAllocator(num_pages)

    @staticmethod
    def pages_for(tokens: int, page_size: int = 16) -> int:
        return -(-tokens // page_size)

    @staticmethod
    def bytes_per_page(n_layers: int, d_model: int, page_size: int = 16, itemsize: int = 2) -> int:
        return 2 * n_layers * page_size * d_model * itemsize

    def occupancy(self) -> float:
        return 1.0 - self.allocator.free / max(1, self.num_pages)

    def slots(self, pages: list[int], start: int, count: int) -> list[int]:
        """Flat cache slots (page * page_size + offset) of token positions [start, start + count)."""
        ps = self.page_size
        if self.allocator._pool is not None and count > 64:
            from ..utils import host_runtime
            return host_runtime.slots(pages, ps, start, count)
        return [pages[t // ps] * ps + t % ps for t in range(start, start + count)]
