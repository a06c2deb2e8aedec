"""The step function: one batch of (request, its next tokens) through the model.

`ModelRunner.step(entries)` takes any mix of prompt portions and single decoded
tokens, cut anywhere.  It takes the pages the new tokens need, lays the batch out
flat (tokens, positions, block tables, cache slots), uploads that in one copy,
runs only the given tokens from the cache that earlier steps left, and returns
float32 logits at the wanted places.  The reference's seam has the same inputs
(crates/traits/src/model.rs:67-75: tokens, positions, block ids, computed counts)
but runs the entries one by one and returns logits for every position
(crates/model/src/causal_lm/model/mod.rs:143-164); here the entries are one batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import make_cache_manager
from ..cache.manager import CacheLayout, OutOfPages
from ..cache.storage import CacheStorage
from ..parts.base import QUERY_TILE, BuildContext, Entry, GroupView, StepBatch, Workspace
from ..parts.model import CausalLM, cache_needs


class StepError(RuntimeError):
    pass


@dataclass
class StepEntry:
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()        # places among `tokens` whose logits are asked for


_DEVICE_ERRORS = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
                  4: "a block table entry that names no page", 8: "a wait inside a kernel ran out",
                  0x10: "a position beyond the context that the attention launch was sized for",
                  # which kernel waited in vain (csrc/common.cuh) ...
                  0x100: "in the float32 decode attention", 0x200: "in the weight-streaming product",
                  0x400: "in the tcgen05 product", 0x800: "in the paired tcgen05 product",
                  0x1000: "in the tcgen05 attention", 0x2000: "in the streaming decode attention",
                  # ... and, in the tcgen05 products, for what
                  0x10000: "for a free stage", 0x20000: "for a free accumulator", 0x40000: "for a filled stage",
                  0x80000: "for a complete accumulator"}


# Steps of up to this many tokens launch their kernels with programmatic dependent launch (each kernel's
# start-up overlaps the end of the one before: what a step of few tokens spends between kernels); longer
# steps, whose kernels run for tens of microseconds and more, are launched the plain way (csrc/common.cuh).
PDL_MAX_TOKENS = 64


def _align4(n: int) -> int:
    return (n + 3) & ~3


def _pow2_at_least(n: int, floor: int = 1) -> int:
    p = floor
    while p < n:
        p *= 2
    return p


class ModelRunner:
    def __init__(self, plan, weights: dict, *, dtype=torch.bfloat16, device="cuda:0", page_size: int = 64,
                 num_pages=1024, max_requests: int = 256, decode_graphs: bool = True,
                 max_context: Optional[int] = None, native_host: bool = True, memory_fraction: float = 0.9,
                 max_step_tokens: int = 4096, own_weights: bool = False, free_memory_bytes: Optional[int] = None):
        """`num_pages`: pages of every paged group (an int, or one count per group), or None: the pools are
        then sized from the device memory that is free once the model is built (`memory_fraction` of it,
        less a reserve for the activations of steps of up to `max_step_tokens` tokens; cache/sizing.py).
        `own_weights`: the dict is emptied once the model holds its tensors, so that what the model stacked
        into new matrices (q/k/v, gate/up) is freed before memory is measured.  `free_memory_bytes` stands
        in for the measurement (tests)."""
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise StepError("the engine runs on a CUDA device only; there is no CPU path")
        if dtype not in (torch.bfloat16, torch.float32):
            raise StepError(f"dtype must be bfloat16 or float32, got {dtype}")
        self.plan = plan
        self.dtype = dtype
        self.page_size = int(page_size)
        torch.cuda.set_device(self.device)
        self.model = CausalLM(plan, weights, BuildContext(self.device, dtype))
        self.layout = CacheLayout.from_needs(cache_needs(plan), [c.cache_of for c in plan.order])
        self.max_context = int(max_context or plan.max_position_embeddings)
        if own_weights:
            weights.clear()
        self.sized_from_memory = None
        if num_pages is None:
            from ..cache.sizing import activation_reserve, pages_from_memory
            itemsize = 2 if dtype == torch.bfloat16 else 4
            if free_memory_bytes is None:
                torch.cuda.empty_cache()
                free_memory_bytes = torch.cuda.mem_get_info(self.device)[0]
            reserve = activation_reserve(plan, max_step_tokens, max_requests, self.max_context, itemsize)
            num_pages = pages_from_memory(self.layout, self.page_size, itemsize, free_memory_bytes, memory_fraction,
                                          reserve, max_requests, self.max_context, max_step_tokens)
            self.sized_from_memory = dict(free_bytes=int(free_memory_bytes), fraction=memory_fraction,
                                          reserve_bytes=reserve, pages=list(num_pages))
        # bookkeeping and batch packing in C++ (csrc/host/cache_core.cpp); the Python manager is the reference
        self.native_host = bool(native_host)
        self.cache = make_cache_manager(self.layout, self.page_size, num_pages, max_requests, native=self.native_host)
        self.storage = CacheStorage(self.layout, self.page_size, num_pages, max_requests, dtype, self.device)
        self.workspace = Workspace(self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._meta_dev = None
        self._meta_pin = [None, None]
        self._meta_evt = [None, None]
        self._flip = 0
        self.steps = 0
        # Decode-only steps (one token per request) are replayed from CUDA graphs, one per
        # batch-size bucket, when every part of the model launches only stream-ordered kernels.
        self.decode_graphs = bool(decode_graphs) and getattr(self.model, "graph_safe", False)
        self._graphs = {}
        self._graph_meta = {}
        self.graph_replays = 0
        self._graph_launches = {}
        self.uploaded_bytes = 0

    # ---- requests ---------------------------------------------------------
    def has_request(self, request_id) -> bool:
        return request_id in self.cache.requests

    def cached_tokens(self, request_id) -> int:
        return self.cache.requests[request_id].num_tokens

    def release(self, request_id):
        """Give back what a finished (or pre-empted) request holds."""
        if request_id in self.cache.requests:
            self.cache.free(request_id)

    # ---- the step ---------------------------------------------------------
    def fits(self, entries: List[StepEntry]) -> bool:
        need = [0] * len(self.cache.pools)
        new_requests = 0
        for e in entries:
            if e.request_id in self.cache.requests:
                pn = self.cache.pages_needed(e.request_id, len(e.tokens))
            else:
                new_requests += 1
                pn = [-(-len(e.tokens) // self.page_size)] * len(self.cache.pools)
            need = [a + b for a, b in zip(need, pn)]
        return all(n <= p.free_count for n, p in zip(need, self.cache.pools)) and \
            new_requests <= self.cache.slots.free_count

    def step(self, entries: List[StepEntry]) -> torch.Tensor:
        """Logits float32 [sum of len(want), vocab] on the device, in the order of
        the entries and of their `want`.  The tensor is a view of a buffer that the
        next step writes again: copy what must outlive it.  Raises OutOfPages, with
        nothing changed, when the pool cannot hold the new tokens."""
        fast = self._decode_step_native(entries)
        if fast is not None:
            return fast
        batch = self.prepare(entries)
        if batch.graph_bucket:
            logits = self._forward_graph(batch)[:sum(len(e.want) for e in entries)]
        else:
            from ..csrc import ops
            ops.set_pdl(batch.num_tokens <= PDL_MAX_TOKENS)
            logits = self.model.forward(batch, self.storage.call_caches)
        self.finish(batch)
        return logits

    def _decode_step_native(self, entries):
        """The common step of serving: every request brings one token and wants its logits, and a graph
        is there to run it.  One call of the C++ core checks, appends and packs; then upload and
        replay.  None when the step is of another kind (the general path takes it)."""
        if not (self.native_host and self.decode_graphs):
            return None
        cache = self.cache
        ids = []
        for e in entries:
            if len(e.tokens) != 1 or len(e.want) != 1 or e.want[0] != 0 or e.request_id not in cache.requests:
                return None
            ids.append(e.request_id)
        B = len(ids)
        if B == 0 or len(set(ids)) != B:
            return None
        bucket = _pow2_at_least(B)
        fixed = -(-self.max_context // self.page_size)
        G = len(cache.pools)
        words = 64 + 8 * bucket + G * (bucket + bucket * fixed + 8)
        while True:
            i, pin = self._pinned_slot(words)
            got = cache.decode_step(ids, [e.tokens[0] for e in entries], bucket, fixed, self.max_context, pin.numpy())
            if got is None:                           # a request at the end of its context: no graph for that
                self._flip ^= 1
                return None
            used, off, sizes, starts = got
            if used >= 0:
                break
            self._flip ^= 1
            words = -used
        dev = self._to_device(i, used, bucket)
        bound = self._context_bound(int(starts.max()) + 1)
        self.steps += 1
        entry = self._graphs.get((bucket, bound))
        if entry is not None:
            entry[0].replay()
            from ..csrc import ops
            ops.launch_count += self._graph_launches[(bucket, bound)]
            self.graph_replays += 1
            return entry[1][:B]
        host_entries = [Entry(r, int(s), 1, cache.requests[r].state_slot) for r, s in zip(ids, starts)]
        batch = self._batch_from_packed(dev, off, sizes, [fixed] * G, host_entries, bucket)
        return self._forward_graph(batch)[:B]         # records the graph

    def step_ahead(self, request_ids, token_source: torch.Tensor, longest: int):
        """A decode step launched before the host knows its tokens: request i's token is
        token_source[i] (int32 on the device, written by work already queued on the stream), every
        request wants its logits, and `longest` bounds position + 1 of the new tokens.  Returns the
        logits, or None with nothing changed when this cannot be done (no graph recorded for the
        shape yet, pages or context exhausted): the caller then steps the ordinary way."""
        if not (self.native_host and self.decode_graphs):
            return None
        B = len(request_ids)
        bucket, bound = _pow2_at_least(B), self._context_bound(longest)
        entry = self._graphs.get((bucket, bound))
        if entry is None or longest > self.max_context or any(r not in self.cache.requests for r in request_ids):
            return None
        fixed = -(-self.max_context // self.page_size)
        G = len(self.cache.pools)
        i, pin = self._pinned_slot(64 + 8 * bucket + G * (bucket + bucket * fixed + 8))
        try:
            # the caller's bound is the core's limit on a request's length: a request that would pass it
            # makes the call return before anything is appended or released
            got = self.cache.decode_step(request_ids, [0] * B, bucket, fixed, min(int(longest), self.max_context),
                                         pin.numpy())
        except OutOfPages:
            got = None
        if got is None or got[0] < 0:
            self._flip ^= 1
            return None
        used, off, sizes, starts = got
        dev = self._to_device(i, used, bucket)
        dev[int(off[0]):int(off[0]) + B].copy_(token_source[:B])
        self.steps += 1
        entry[0].replay()
        from ..csrc import ops
        ops.launch_count += self._graph_launches[(bucket, bound)]
        self.graph_replays += 1
        return entry[1][:B]

    def _forward_graph(self, batch: StepBatch) -> torch.Tensor:
        """Rows of padded requests come after the real ones, so the caller slices them off."""
        key = (batch.graph_bucket, batch.groups[0].max_context if batch.groups else 0)
        entry = self._graphs.get(key)
        if entry is None:
            # first sight of this bucket: run it as it is (also sizes the workspace), then record
            from ..csrc import ops
            ops.set_pdl(True)                          # a decode step: one token a request
            logits = self.model.forward(batch, self.storage.call_caches)
            torch.cuda.current_stream().synchronize()
            before = ops.launch_count
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = self.model.forward(batch, self.storage.call_caches)
            self._graph_launches[key] = ops.launch_count - before
            ops.launch_count = before                  # recording launches nothing
            self._graphs[key] = (graph, static_logits)
            return logits
        graph, static_logits = entry
        graph.replay()
        from ..csrc import ops
        ops.launch_count += self._graph_launches[key]
        self.graph_replays += 1
        return static_logits

    def prepare(self, entries: List[StepEntry]) -> StepBatch:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id!r} brings no token")
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.request_id!r} wants place {w} of {len(e.tokens)} tokens")
        if not self.fits(entries):
            raise OutOfPages(f"the step needs more pages or slots than are free {self.cache.free_pages()}")
        host_entries = []
        for e in entries:
            if e.request_id not in self.cache.requests:
                self.cache.admit(e.request_id)
            start = self.cache.append(e.request_id, len(e.tokens))
            host_entries.append(Entry(e.request_id, start, len(e.tokens),
                                      self.cache.requests[e.request_id].state_slot))
        self.storage.zero_slots(self.cache.take_fresh_slots())
        return self._layout_batch(entries, host_entries, self._graph_bucket(entries, host_entries))

    def _graph_bucket(self, entries, host_entries) -> int:
        """Padded batch size of a decode-only step that can be replayed from a graph, else 0."""
        if not self.decode_graphs or any(h.count != 1 for h in host_entries):
            return 0
        if any(len(e.want) != 1 for e in entries) or any(h.start + 1 > self.max_context for h in host_entries):
            return 0
        return _pow2_at_least(len(entries))

    def _context_bound(self, longest: int) -> int:
        """A graph is recorded for a bound on the context, not for its value: the next power of two
        from 1,024 on, at most the longest context the runner takes."""
        return min(_pow2_at_least(longest, 1024), self.max_context)

    def _layout_batch(self, entries, host_entries, bucket: int = 0) -> StepBatch:
        if self.native_host:
            return self._layout_native(entries, host_entries, bucket)
        return self._layout_python(entries, host_entries, bucket)

    def _pinned_slot(self, words: int):
        """A pinned host buffer of at least `words` int32 whose last upload has completed."""
        i = self._flip
        self._flip ^= 1
        if self._meta_evt[i] is not None:
            self._meta_evt[i].synchronize()
        if self._meta_pin[i] is None or self._meta_pin[i].numel() < words:
            self._meta_pin[i] = torch.empty(max(words, 4096) * 2, dtype=torch.int32).pin_memory()
        return i, self._meta_pin[i]

    def _to_device(self, i: int, n: int, bucket: int) -> torch.Tensor:
        pin = self._meta_pin[i]
        if bucket:                                  # a graph reads its batch from a buffer of its own
            dev = self._graph_meta.get(bucket)
            if dev is None or dev.numel() < n:
                # graphs recorded for this bucket read the old buffer: they are recorded again
                for key in [k for k in self._graphs if k[0] == bucket]:
                    del self._graphs[key]
                dev = self._graph_meta[bucket] = torch.empty(n, dtype=torch.int32, device=self.device)
        else:
            if self._meta_dev is None or self._meta_dev.numel() < n:
                self._meta_dev = torch.empty(max(n, 4096) * 2, dtype=torch.int32, device=self.device)
            dev = self._meta_dev
        dev[:n].copy_(pin[:n], non_blocking=True)
        self.uploaded_bytes += 4 * n
        if self._meta_evt[i] is None:
            self._meta_evt[i] = torch.cuda.Event()
        self._meta_evt[i].record()
        return dev[:n]

    def _layout_native(self, entries, host_entries, bucket: int) -> StepBatch:
        """The C++ core packs the batch straight into pinned memory."""
        B = len(entries)
        counts = [h.count for h in host_entries]
        starts = [h.start for h in host_entries]
        if all(c == 1 for c in counts):
            tokens = [e.tokens[0] for e in entries]
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]).astype(np.int32)
        want_offsets, wants = [0], []
        for e in entries:
            wants.extend(e.want)
            want_offsets.append(len(wants))
        ids = [e.request_id for e in entries]
        fixed = -(-self.max_context // self.page_size) if bucket else 0
        guess = 4096
        while True:
            i, pin = self._pinned_slot(guess)
            used, off, sizes, max_blocks = self.cache.pack_step(ids, counts, starts, tokens, want_offsets, wants,
                                                                bucket, 0 if bucket else QUERY_TILE, fixed, pin.numpy())
            if used >= 0:
                break
            self._flip ^= 1                          # the slot was not used; take it again, larger
            guess = -used
        dev = self._to_device(i, used, bucket)
        return self._batch_from_packed(dev, off, sizes, max_blocks, host_entries, bucket)

    def _batch_from_packed(self, dev, off, sizes, max_blocks, host_entries, bucket: int) -> StepBatch:
        """Views of the uploaded buffer that the C++ core packed (sections: csrc/host/cache_core.cpp)."""
        sec = lambda k: dev[int(off[k]):int(off[k]) + int(sizes[k])]
        counts = [h.count for h in host_entries]
        Bp = bucket or len(host_entries)
        longest = max(h.start + h.count for h in host_entries)
        if bucket:
            longest = self._context_bound(longest)
        groups = [GroupView(page_size=self.page_size, block_table=sec(9 + 2 * g).view(Bp, int(max_blocks[g])),
                            slots=sec(8 + 2 * g), max_context=longest) for g in range(len(self.cache.pools))]
        tiles, single = sec(6), sec(7)
        single_context = max([h.start + 1 for h in host_entries if h.count == 1], default=0)
        return StepBatch(tokens=sec(0), positions=sec(1), req_index=sec(2), cu_seqlens=sec(3), state_slots=sec(4),
                         logit_rows=sec(5), groups=groups, entries=host_entries, err=self.err, workspace=self.workspace,
                         num_tokens=bucket or sum(counts), num_entries=Bp, max_query_len=max(counts),
                         tag=f"g{bucket}.{longest}." if bucket else "", graph_bucket=bucket,
                         query_tiles=tiles.view(-1, 4) if tiles.numel() else None,
                         single_tokens=single if single.numel() else None, single_context=single_context)

    def _layout_python(self, entries, host_entries, bucket: int = 0) -> StepBatch:
        real_B = len(entries)
        real_T = sum(h.count for h in host_entries)
        real_R = sum(len(e.want) for e in entries)
        # a graph step is padded to its bucket with tokens at position -1: they read no key,
        # write no cache slot, and their rows are cut off by the caller
        B, T, R = (bucket, bucket, bucket) if bucket else (real_B, real_T, real_R)
        G = len(self.cache.pools)
        ps = self.page_size
        tables = [[self.cache.requests[e.request_id].block_tables[g] for e in entries] for g in range(G)]
        if bucket:
            max_blocks = [-(-self.max_context // ps)] * G
        else:
            max_blocks = [max(1, max(len(t) for t in tables[g])) for g in range(G)]
        # section offsets (int32 words), each aligned to 16 bytes
        off, cursor = {}, 0
        def section(name, n):
            nonlocal cursor
            off[name] = (cursor, n)
            cursor += _align4(max(n, 1))
        # tiles of up to QUERY_TILE consecutive tokens of one request, for the tensor-core prefill kernels
        # ... and, when the step also holds requests that bring one token, the indices of those tokens
        tile_list, single_list = [], []
        if not bucket:
            t0 = 0
            for b, h in enumerate(host_entries):
                if h.count > 1:
                    for lo in range(0, h.count, QUERY_TILE):
                        tile_list.append((b, t0 + lo, min(QUERY_TILE, h.count - lo), h.start + lo))
                else:
                    single_list.append(t0)
                t0 += h.count
            if not tile_list:
                single_list = []
        for name, n in (("tokens", T), ("positions", T), ("req_index", T), ("cu_seqlens", B + 1),
                        ("state_slots", B), ("logit_rows", R), ("tiles", 4 * len(tile_list)),
                        ("single", len(single_list))):
            section(name, n)
        for g in range(G):
            section(f"slots{g}", T)
            section(f"table{g}", B * max_blocks[g])
        meta = np.full(cursor, -1, dtype=np.int32)
        def view(name):
            o, n = off[name]
            return meta[o:o + n]
        tok, pos, req, cu = view("tokens"), view("positions"), view("req_index"), view("cu_seqlens")
        rows = view("logit_rows")
        if bucket:
            tok[:], req[:], cu[:] = 0, 0, real_T
            rows[:] = np.arange(bucket)
            view("state_slots")[:] = 0
        cu[0] = 0
        t = r = 0
        for b, (e, h) in enumerate(zip(entries, host_entries)):
            tok[t:t + h.count] = np.asarray(e.tokens, dtype=np.int64).astype(np.int32)
            pos[t:t + h.count] = np.arange(h.start, h.start + h.count, dtype=np.int32)
            req[t:t + h.count] = b
            for w in e.want:
                rows[r] = t + w
                r += 1
            t += h.count
            cu[b + 1] = t
        view("state_slots")[:real_B] = [h.state_slot for h in host_entries]
        if tile_list:
            view("tiles")[:] = np.asarray(tile_list, dtype=np.int32).reshape(-1)
        if single_list:
            view("single")[:] = single_list
        for g in range(G):
            tb = view(f"table{g}").reshape(B, max_blocks[g])
            sl = view(f"slots{g}")
            t = 0
            for b, h in enumerate(host_entries):
                tab = np.asarray(tables[g][b], dtype=np.int32)
                tb[b, :len(tab)] = tab
                p = np.arange(h.start, h.start + h.count)
                pages = tab[p // ps]
                if (pages < 0).any():
                    raise StepError(f"request {h.request!r} writes into a page that was given back")
                sl[t:t + h.count] = pages * ps + (p % ps)
                t += h.count
        dev = self._upload(meta, bucket)
        def dview(name):
            o, n = off[name]
            return dev[o:o + n]
        groups = []
        longest = max(h.start + h.count for h in host_entries)
        if bucket:
            longest = self._context_bound(longest)
        for g in range(G):
            groups.append(GroupView(page_size=ps, block_table=dview(f"table{g}").view(B, max_blocks[g]),
                                    slots=dview(f"slots{g}"), max_context=longest))
        return StepBatch(tokens=dview("tokens"), positions=dview("positions"), req_index=dview("req_index"),
                         cu_seqlens=dview("cu_seqlens"), state_slots=dview("state_slots"),
                         logit_rows=dview("logit_rows"), groups=groups, entries=host_entries, err=self.err,
                         workspace=self.workspace, num_tokens=T, num_entries=B,
                         max_query_len=max(h.count for h in host_entries),
                         tag=f"g{bucket}.{longest}." if bucket else "", graph_bucket=bucket,
                         query_tiles=dview("tiles").view(-1, 4) if tile_list else None,
                         single_tokens=dview("single") if single_list else None,
                         single_context=max([h.start + 1 for h in host_entries if h.count == 1], default=0))

    def _upload(self, meta: np.ndarray, bucket: int = 0) -> torch.Tensor:
        n = meta.shape[0]
        i = self._flip
        self._flip ^= 1
        if self._meta_evt[i] is not None:
            self._meta_evt[i].synchronize()
        if self._meta_pin[i] is None or self._meta_pin[i].numel() < n:
            self._meta_pin[i] = torch.empty(max(n, 4096) * 2, dtype=torch.int32).pin_memory()
        if self._meta_dev is None or self._meta_dev.numel() < n:
            self._meta_dev = torch.empty(max(n, 4096) * 2, dtype=torch.int32, device=self.device)
        pin = self._meta_pin[i]
        pin[:n].numpy()[:] = meta
        if bucket:                                  # a graph reads its batch from a buffer of its own
            dev = self._graph_meta.get(bucket)
            if dev is None:
                dev = self._graph_meta[bucket] = torch.empty(n, dtype=torch.int32, device=self.device)
        else:
            dev = self._meta_dev
        dev[:n].copy_(pin[:n], non_blocking=True)
        self.uploaded_bytes += 4 * n
        if self._meta_evt[i] is None:
            self._meta_evt[i] = torch.cuda.Event()
        self._meta_evt[i].record()
        return dev[:n]

    def finish(self, batch: StepBatch):
        """Bookkeeping after the step's kernels are queued: windows move on."""
        for h in batch.entries:
            self.cache.release_behind_window(h.request)
        self.steps += 1

    def check_device_errors(self):
        """Read the device error word (synchronises); raise if a kernel refused an access."""
        word = int(self.err.item())
        if word:
            self.err.zero_()
            what = [msg for bit, msg in _DEVICE_ERRORS.items() if word & bit]
            raise StepError("a kernel skipped an access: " + "; ".join(what))
