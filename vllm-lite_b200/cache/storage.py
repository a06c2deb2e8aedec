"""Device tensors behind the cache manager's bookkeeping.

A paged group with c entries of the running order is one tensor
[c, 2, pages, kv_heads, page_size, head_dim] (keys at [:, 0], values at [:, 1]):
a (kv head, page) tile of page_size x head_dim is contiguous, which is what the
attention kernels read.  A fixed-state group is [c, slots, *shape].  Pages are
never cleared when they change hands: attention reads only what the block table
and the positions name.  State slots are zeroed when they are handed out.
"""
from __future__ import annotations

import torch

from ..parts.base import CallCache
from .manager import CacheLayout

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CacheStorage:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages, max_requests: int, dtype, device):
        self.layout = layout
        counts = [int(num_pages)] * len(layout.paged_groups) if isinstance(num_pages, int) else list(num_pages)
        self.paged = [torch.zeros((len(members), 2, n, need.num_kv_heads, page_size, need.head_dim),
                                  dtype=dtype, device=device)
                      for need, members, n in zip(layout.paged_groups, layout.paged_members, counts)]
        self.state = [torch.zeros((len(members), max_requests) + tuple(need.shape),
                                  dtype=_STATE_DTYPES[need.dtype], device=device)
                      for need, members in zip(layout.state_groups, layout.state_members)]
        self.call_caches = []
        for place in layout.call_place:
            if place is None:
                self.call_caches.append(CallCache())
                continue
            kind, g, idx, owns = place
            if kind == "paged":
                self.call_caches.append(CallCache(group=g, k=self.paged[g][idx, 0], v=self.paged[g][idx, 1], writes=owns))
            else:
                self.call_caches.append(CallCache(group=g, state=self.state[g][idx], writes=owns))

    def zero_slots(self, slots):
        if not slots:
            return
        for t in self.state:
            t[:, slots] = 0

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.paged + self.state)
