"""How many pages the cache gets when nobody says: what is left of the GPU after the weights.

The reference takes `--kv-blocks` with a default of 1,024 (crates/server/src/cli/args.rs:161-162); on
a GPU with 180 GB that is 16,384 tokens of cache beside a hundred and more GB unused.  Here an explicit
count still wins; without one the pools are sized from the free device memory: a fraction of what is
free once the weights are resident, less a reserve for the step's activations, shared out among the
paged groups by the bytes a page of each costs.  Plain arithmetic on numbers: nothing here touches
a device, the caller brings the free bytes.
"""
from __future__ import annotations

from typing import List, Optional

from .manager import CacheLayout

MIN_RESERVE = 512 << 20


def page_bytes(layout: CacheLayout, page_size: int, itemsize: int) -> List[int]:
    """Bytes of one page in every paged group: keys and values of every call of the group."""
    return [len(members) * page_size * need.bytes_per_token(itemsize)
            for need, members in zip(layout.paged_groups, layout.paged_members)]


def state_bytes(layout: CacheLayout, max_requests: int) -> int:
    sizes = {"float32": 4, "bfloat16": 2, "int32": 4}
    total = 0
    for need, members in zip(layout.state_groups, layout.state_members):
        n = sizes[need.dtype]
        for s in need.shape:
            n *= int(s)
        total += n * len(members) * max_requests
    return total


def activation_reserve(plan, max_step_tokens: int, max_requests: int, max_context: int, itemsize: int) -> int:
    """A bound on what steps allocate beside weights and cache: the buffers of the longest step (the
    float32 stream, a layer's widest intermediates) and, for every decode graph that may be recorded
    (batch buckets up to max_requests, context bounds from 1,024 up), its own logits."""
    H, V = plan.hidden_size, plan.vocab_size
    widest = 0
    for block in plan.layers:
        w = 0
        mixer, ffn = getattr(block, "mixer", None), getattr(block, "ffn", None)
        if hasattr(mixer, "num_heads"):
            w += (2 * mixer.num_heads + 2 * mixer.num_kv_heads) * mixer.head_dim
        if hasattr(ffn, "intermediate_size"):
            w += 3 * ffn.intermediate_size
        widest = max(widest, w)
    per_token = 4 * H + itemsize * (widest + 4 * H)
    bounds, b = 1, 1024
    while b < max_context:
        b, bounds = b * 2, bounds + 1
    graph_logits = 2 * max_requests * V * 4 * bounds          # buckets 1, 2, 4, ... sum to under twice the largest
    return int(1.25 * per_token * max_step_tokens) + graph_logits + MIN_RESERVE


def pages_from_memory(layout: CacheLayout, page_size: int, itemsize: int, free_bytes: int, fraction: float,
                      reserve_bytes: int, max_requests: int, max_context: int,
                      max_step_tokens: Optional[int] = None) -> List[int]:
    """Pages for every paged group.  budget = free_bytes * fraction - reserve_bytes - state slots; every
    group gets the same count, except that no group gets more pages than its requests could ever hold
    at once (max_requests at max_context; a windowed group: the window plus the longest step), and
    what such a group leaves goes to the others.  Raises ValueError when not even one request of
    max_context fits."""
    if not 0.0 < fraction <= 1.0:
        raise ValueError(f"the memory fraction must lie in (0, 1], got {fraction}")
    costs = page_bytes(layout, page_size, itemsize)
    if not costs:
        return []
    budget = int(free_bytes * fraction) - int(reserve_bytes) - state_bytes(layout, max_requests)
    per_request = -(-max_context // page_size)
    caps, least = [], []
    for need in layout.paged_groups:
        most = per_request
        if need.window is not None:
            most = min(most, -(-(need.window + (max_step_tokens or max_context)) // page_size) + 1)
        least.append(most)                                    # what one request alone may come to hold
        caps.append(max_requests * most + 1)
    counts: List[Optional[int]] = [None] * len(costs)
    while True:
        open_groups = [g for g, c in enumerate(counts) if c is None]
        if not open_groups:
            break
        left = budget - sum(costs[g] * c for g, c in enumerate(counts) if c is not None)
        share = left // sum(costs[g] for g in open_groups)
        capped = [g for g in open_groups if caps[g] <= share]
        if not capped:
            for g in open_groups:
                counts[g] = int(share)
            break
        for g in capped:
            counts[g] = caps[g]
    if any(c < l for c, l in zip(counts, least)):
        raise ValueError(f"{free_bytes / 2**30:.1f} GiB free x {fraction} less {reserve_bytes / 2**30:.1f} GiB of reserve "
                         f"holds {counts} pages; one request of {max_context} tokens needs {least}")
    return counts
