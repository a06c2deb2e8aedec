"""What a mixer keeps for each request, as plain data.

`PagedKV`: keys and values that grow by one row per token, stored in pages.
`window`, when set, means that only the last `window` tokens are ever read, so
pages that lie wholly before the window may be given back.
`FixedState`: a tensor of fixed shape per request, stored in a slot.
Calls of the running order whose needs are equal share one group: one pool of
pages (or slots) and one block table per request.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKV:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def bytes_per_token(self, itemsize: int) -> int:
        return 2 * self.num_kv_heads * self.head_dim * itemsize


@dataclass(frozen=True)
class FixedState:
    shape: Tuple[int, ...]
    dtype: str = "float32"
