"""What parts are given at build time and at every step, and what each family must offer.

Interfaces (duck-typed; a part is any class registered under its kind):

  every part     declare(spec) -> {relative tensor name: TensorDecl}     static
                 __init__(spec, weights, ctx)   weights: {relative name: device tensor}
  norm           __call__(x, delta, step, rows=None) -> h
                     x float32 [T, H] residual stream; delta (activation dtype) or None is
                     added into x first (not stored when `rows` picks rows); h is new
  position       fused_rotary() -> (inv_freq, rotary_dim), or None for an encoding of its own, which then
                 offers apply(qkv, positions, num_heads, num_kv_heads, head_dim, step): it changes the
                 q and k parts of qkv [T, (nq + 2 nkv) hd] in place, before the head norm
  mixer          cache_need(spec) -> PagedKV | FixedState | None                  static
                 __call__(h, step, cache) -> [T, hidden] in the activation dtype
  feed-forward   __call__(h, step) -> [T, hidden]
  block          __call__(residual, step, cache) -> None   (updates residual.x / residual.pending)
  mixers and feed-forwards may set `graph_safe = True` when their forward only launches
  stream-ordered kernels on static buffers (no host reads, no Python over the entries);
  decode steps of a model whose parts all say so are replayed from CUDA graphs

No part learns which model it is in: it sees its own description, its own
tensors, the step's batch and the cache of its own call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class BuildContext:
    device: torch.device
    dtype: torch.dtype            # activation / model dtype: torch.bfloat16 or torch.float32


class Workspace:
    """Scratch buffers that live across steps, so that a step allocates nothing
    once its shapes have been seen (and can be captured in a CUDA graph)."""

    def __init__(self, device):
        self.device = device
        self._buffers = {}

    def get(self, tag: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (tag, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:n].view(*shape)

    def zeros(self, tag: str, n: int, dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out and that its users leave zero (counters that
        the kernels reset themselves); it only grows."""
        key = (tag, dtype, "zeros")
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class GroupView:
    """One cache group as a step sees it."""
    page_size: int
    block_table: torch.Tensor       # int32 [B, max_blocks], -1 where no page is held
    slots: torch.Tensor             # int32 [T]: page * page_size + offset of every token of the step
    max_context: int = 0            # host copy: the longest context among the entries


@dataclass
class Entry:
    """Host-side description of one request's share of a step."""
    request: object
    start: int                      # tokens of the request that are already in the cache
    count: int                      # tokens it brings in this step
    state_slot: int = -1


# most consecutive tokens of one request in an entry of StepBatch.query_tiles (what the tiled
# attention kernels take as one tile of query rows)
QUERY_TILE = 128


@dataclass
class StepBatch:
    tokens: torch.Tensor            # int32 [T]
    positions: torch.Tensor         # int32 [T] absolute position of each token in its request
    req_index: torch.Tensor         # int32 [T] row of the block tables
    cu_seqlens: torch.Tensor        # int32 [B + 1]
    state_slots: torch.Tensor       # int32 [B] per-request state slot
    logit_rows: torch.Tensor        # int32 [R] token indices whose logits are wanted
    groups: List[GroupView]
    entries: List[Entry]
    err: torch.Tensor               # device error word (uint32 as int32 [1])
    workspace: Workspace
    num_tokens: int = 0
    num_entries: int = 0
    max_query_len: int = 0
    tag: str = ""                   # namespace for workspace buffers
    graph_bucket: int = 0           # padded batch size when the step is replayed from a CUDA graph
    query_tiles: Optional[torch.Tensor] = None   # int32 [n, 4]: (table row, first token, tokens <= QUERY_TILE, first position)
    single_tokens: Optional[torch.Tensor] = None  # int32: tokens of one-token requests, when the step also holds portions
    single_context: int = 0                      # bound on position + 1 of those tokens


@dataclass
class CallCache:
    """The cache of one entry of the running order.

    Paged: `k`, `v` are [pages, kv_heads, page_size, head_dim]; `group` indexes
    StepBatch.groups; `writes` is False for a call that reads an earlier call's
    cache.  Fixed state: `state` is [slots, *shape], indexed by StepBatch.state_slots.
    """
    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    writes: bool = True
    state: Optional[torch.Tensor] = None


@dataclass
class Residual:
    x: torch.Tensor                           # float32 [T, H]
    pending: Optional[torch.Tensor] = None    # not yet added into x
    normed: Optional["ScaledRows"] = None     # output of the norm `normed_for` on x, in factored form
    normed_for: object = None


@dataclass
class ScaledRows:
    """The output of an RMS norm in factored form, as input of a linear layer: row m of the matrix is
    rows[m] * scale[m] with scale[m] = 1 / sqrt(sum_b partial[b, m] / size + eps).  `rows` already
    carries the norm's weight; the partial sums of squares of the stream were left by the kernel
    that last wrote the stream, one vector per block, and the product kernel that reads `rows`
    applies the scales to its result.  It saves the norm's own kernel in steps of few rows."""
    rows: torch.Tensor                        # [M, size], activation dtype
    partial: torch.Tensor                     # float32 [capacity, 16]
    count: int
    eps: float
    size: int


@dataclass
class StreamSink:
    """Offer to a part whose last step is a linear layer: add your result into the float32 stream `x`
    yourself and return the next norm's output (weight `weight`) as ScaledRows."""
    x: torch.Tensor
    weight: torch.Tensor                      # float32 [size]
    eps: float
    size: int


def sub_weights(weights: dict, prefix: str) -> dict:
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def prefixed(decls: dict, prefix: str) -> dict:
    return {prefix + k: v for k, v in decls.items()}
