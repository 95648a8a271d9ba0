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
    """LIFO free list over page ids with reservation accounting."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> list[int]:
        if n > len(self._free):
            raise MemoryError(f"out of KV pages: want {n}, have {len(self._free)}")
        out = self._free[-n:][::-1] if n else []
        del self._free[len(self._free) - n:]
        return out

    def give(self, pages: list[int]):
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
        return [pages[t // ps] * ps + t % ps for t in range(start, start + count)]
