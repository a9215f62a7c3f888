"""Device memory of the cache: pages of keys and values per layer, and slot-indexed state.

Layout of a layer's pages is the reference's: ``[num_pages, page_size, kv_heads, head_dim]``
for keys and the same for values, so one token's heads are contiguous and
``slot = page * page_size + offset`` indexes the flat view (src/paged_kv_cache.py:51-64).
Page ids are shared by all layers of a cache group: one id names a page in every layer's
tensors.  Pages are zero-filled at start; page 0 is never handed out and stays zero.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..parts.base import CacheNeeds


@dataclass
class LayerCache:
    """What the mixer of one schedule entry gets."""

    group: Optional[int] = None          # index of the cache group whose tables address k / v
    k: Optional[torch.Tensor] = None     # [num_pages, page_size, kv_heads, head_dim]
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None  # [max_num_seqs + 1, *shape]; last row is for padding
    read_only: bool = False              # the cache belongs to another schedule entry

    def num_bytes(self) -> int:
        total = 0
        for t in (self.k, self.v, self.state):
            if t is not None:
                total += t.numel() * t.element_size()
        return total


def allocate_layer_cache(
    needs: CacheNeeds,
    group: Optional[int],
    num_pages: int,
    page_size: int,
    max_num_seqs: int,
    dtype: torch.dtype,
    device: torch.device,
) -> LayerCache:
    cache = LayerCache(group=group)
    if needs.paged is not None:
        shape = (num_pages, page_size, needs.paged.num_kv_heads, needs.paged.head_dim)
        cache.k = torch.zeros(shape, dtype=dtype, device=device)
        cache.v = torch.zeros(shape, dtype=dtype, device=device)
    if needs.state is not None:
        cache.state = torch.zeros(
            (max_num_seqs + 1,) + tuple(needs.state.shape), dtype=needs.state.dtype, device=device
        )
    return cache


def bytes_per_page(needs_list: List[CacheNeeds], page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id costs across every layer that caches keys and values."""
    element = torch.tensor([], dtype=dtype).element_size()
    total = 0
    for needs in needs_list:
        if needs.paged is not None:
            total += 2 * page_size * needs.paged.num_kv_heads * needs.paged.head_dim * element
    return total


def compute_num_pages(
    needs_list: List[CacheNeeds],
    page_size: int,
    dtype: torch.dtype,
    device: torch.device,
    gpu_memory_utilization: float = 0.90,
    reserve_bytes: int = 512 * 1024 * 1024,
) -> int:
    """Pages that fit in the free GPU memory, by the reference's rule
    (src/paged_kv_cache.py:159-194): ``(free * utilization - reserve) // bytes_per_page``
    where free counts memory the torch allocator holds but does not use."""
    per_page = bytes_per_page(needs_list, page_size, dtype)
    if per_page == 0:
        return 2
    free_bytes, _ = torch.cuda.mem_get_info(device)
    free_bytes += torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    budget = int(free_bytes * gpu_memory_utilization) - reserve_bytes
    if budget <= 0:
        raise RuntimeError("not enough free GPU memory for a KV cache")
    pages = budget // per_page
    if pages < 2:
        raise RuntimeError("free GPU memory is too small to hold even one KV cache page")
    return int(pages)
