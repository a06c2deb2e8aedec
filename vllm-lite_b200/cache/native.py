"""The cache manager with its bookkeeping in C++ (csrc/host/cache_core.cpp).

Same interface and same rules as `cache.manager.CacheManager`, which stays as the
reference implementation; both run the same tests.  Besides the bookkeeping the
native core packs a step's batch (tokens, positions, block tables, cache slots,
wanted rows, query tiles) straight into the pinned upload buffer.
Requests are named by any hashable id; the core knows them by a 64-bit key.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_longlong, c_void_p
from typing import List

import numpy as np

from .manager import CacheLayout, OutOfPages
from .pool import PoolError

_ERR = {-1: "not enough free pages or slots", -2: "no such request or group", -3: "the request already holds a cache",
        -4: "a unit is freed twice or was never handed out", -5: "bad argument", -6: "a position lies in a page that was given back",
        -7: "the books do not balance"}
_lib = None


def _core():
    global _lib
    if _lib is None:
        from ..csrc import build
        lib = build.load_host("cache_core")
        I, L, P, V = c_int, c_longlong, POINTER(c_int), c_void_p
        sig = {
            "vc_create": (V, [I, I, P, P, I]), "vc_destroy": (None, [V]), "vc_admit": (I, [V, L, P]),
            "vc_free": (I, [V, L]), "vc_has": (I, [V, L]), "vc_pages_needed": (I, [V, L, L, P]),
            "vc_append": (I, [V, L, L, POINTER(L)]), "vc_release_behind_window": (I, [V, L, P]),
            "vc_request_info": (I, [V, L, POINTER(L), P]), "vc_block_table": (I, [V, L, I, P, I]),
            "vc_slot_of": (I, [V, L, I, L, POINTER(L)]), "vc_pool_counts": (I, [V, I, P, P]),
            "vc_is_held": (I, [V, I, I]), "vc_take_fresh_slots": (I, [V, P, I]), "vc_num_requests": (I, [V]),
            "vc_check": (I, [V]),
            "vc_pack_step": (L, [V, I, V, V, V, V, V, V, I, I, V, V, L, V, V]),
            "vc_decode_step": (L, [V, I, V, V, I, I, L, V, L, V, V, V]),
            "vs_schedule": (I, [V, I, L, L, I, I, V, V, V, V, V, V, V, V, V, V, V]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class _PoolView:
    def __init__(self, mgr, group, what):
        self._m, self._g, self.what = mgr, group, what

    def _counts(self):
        size, free = c_int(), c_int()
        self._m._call("vc_pool_counts", self._g, ctypes.byref(size), ctypes.byref(free))
        return size.value, free.value

    @property
    def size(self):
        return self._counts()[0]

    @property
    def free_count(self):
        return self._counts()[1]

    @property
    def held_count(self):
        size, free = self._counts()
        return size - free

    def is_held(self, unit):
        return _core().vc_is_held(self._m._h, self._g, int(unit)) == 1


class _RequestView:
    def __init__(self, mgr, request_id, key, state_slot):
        self._m, self.request_id, self._key = mgr, request_id, key
        self.state_slot = state_slot           # fixed for the request's life

    def _info(self):
        n, s = c_longlong(), c_int()
        self._m._call("vc_request_info", self._key, ctypes.byref(n), ctypes.byref(s))
        return n.value, s.value

    @property
    def num_tokens(self):
        return self._info()[0]

    @property
    def block_tables(self) -> List[List[int]]:
        out = []
        for g in range(self._m.num_groups):
            n = _core().vc_block_table(self._m._h, self._key, g, None, 0)
            buf = (c_int * max(n, 1))()
            _core().vc_block_table(self._m._h, self._key, g, buf, n)
            out.append(list(buf[:n]))
        return out


class NativeCacheManager:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages, max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.layout = layout
        self.page_size = int(page_size)
        self.num_groups = len(layout.paged_groups)
        counts = [int(num_pages)] * self.num_groups if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(counts) != self.num_groups:
            raise ValueError(f"{self.num_groups} paged groups need {self.num_groups} page counts, got {len(counts)}")
        if any(n < 0 for n in counts):
            raise ValueError("a pool cannot have a negative size")
        windows = [int(g.window or 0) for g in layout.paged_groups]
        arr = lambda v: (c_int * max(len(v), 1))(*v)
        self._h = _core().vc_create(self.page_size, self.num_groups, arr(counts), arr(windows), int(max_requests))
        if not self._h:
            raise ValueError("the native cache core refused its sizes")
        self.pools = [_PoolView(self, g, "page") for g in range(self.num_groups)]
        self.slots = _PoolView(self, -1, "state slot")
        self.requests = {}                  # request id -> view
        self._keys = {}                     # request id -> 64-bit key
        self._next_key = 1
        self._need = (c_int * max(self.num_groups, 1))()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.vc_destroy(h)

    def _call(self, name, *args):
        rc = getattr(_core(), name)(self._h, *args)
        if rc == 0:
            return
        if rc == -1:
            raise OutOfPages(_ERR[-1])
        if rc in (-2, -3):
            raise KeyError(_ERR[rc])
        if rc == -5:
            raise ValueError(_ERR[rc])
        raise PoolError(_ERR.get(rc, f"native cache core error {rc}"))

    # ---- admission and release -------------------------------------------
    def admit(self, request_id):
        if request_id in self._keys:
            raise KeyError(f"request {request_id!r} already holds a cache")
        key = self._next_key
        slot = c_int()
        rc = _core().vc_admit(self._h, key, ctypes.byref(slot))
        if rc == -1:
            raise OutOfPages("no state slot is free")
        if rc:
            self._call("vc_admit", key, ctypes.byref(slot))
        self._next_key += 1
        self._keys[request_id] = key
        view = _RequestView(self, request_id, key, slot.value)
        self.requests[request_id] = view
        return view

    def free(self, request_id):
        key = self._keys.pop(request_id)       # KeyError for an unknown request, as the reference raises
        del self.requests[request_id]
        self._call("vc_free", key)

    # ---- growth -------------------------------------------------------------
    def pages_needed(self, request_id, count: int) -> List[int]:
        self._call("vc_pages_needed", self._keys[request_id], int(count), self._need)
        return list(self._need[:self.num_groups])

    def can_append(self, request_id, count: int) -> bool:
        return all(n <= p.free_count for n, p in zip(self.pages_needed(request_id, count), self.pools))

    def append(self, request_id, count: int) -> int:
        if count <= 0:
            raise ValueError("a step brings at least one token per request")
        start = c_longlong()
        rc = _core().vc_append(self._h, self._keys[request_id], int(count), ctypes.byref(start))
        if rc == -1:
            raise OutOfPages(f"request {request_id!r} needs {self.pages_needed(request_id, count)} pages, "
                             f"free: {self.free_pages()}")
        if rc:
            self._call("vc_append", self._keys[request_id], int(count), ctypes.byref(start))
        return start.value

    def slot_of(self, request_id, group: int, position: int) -> int:
        slot = c_longlong()
        self._call("vc_slot_of", self._keys[request_id], int(group), int(position), ctypes.byref(slot))
        return slot.value

    def release_behind_window(self, request_id) -> int:
        freed = c_int()
        self._call("vc_release_behind_window", self._keys[request_id], ctypes.byref(freed))
        return freed.value

    def take_fresh_slots(self) -> List[int]:
        buf = (c_int * 4096)()
        n = _core().vc_take_fresh_slots(self._h, buf, 4096)
        return list(buf[:n])

    # ---- figures and checks -------------------------------------------------
    def free_pages(self) -> List[int]:
        return [p.free_count for p in self.pools]

    def check_invariants(self):
        self._call("vc_check")
        if len(self.requests) != _core().vc_num_requests(self._h):
            raise PoolError("the host's and the core's lists of requests differ")

    def schedule(self, max_num_seqs, max_num_batched_tokens, prefill_chunk_size, n_run, remaining, computed,
                 request_ids, arrival):
        """The scheduler's decision in the C++ core (csrc/host/cache_core.cpp, vs_schedule): sequences
        0 .. n_run - 1 run (in order of arrival), the rest wait (from the head of the queue);
        request_ids[i] is None for a sequence that holds nothing in the cache.  Returns
        (entries [(sequence, tokens)], victims, admitted); raises OutOfPages when a sequence that runs
        alone cannot get its pages."""
        n = len(remaining)
        rem = np.ascontiguousarray(remaining, dtype=np.int64)
        comp = np.ascontiguousarray(computed, dtype=np.int64)
        keys = np.fromiter((self._keys[r] if r is not None else 0 for r in request_ids), dtype=np.int64, count=n)
        arr = np.ascontiguousarray(arrival, dtype=np.int64)
        e_seq, e_cnt = np.zeros(max(n, 1), dtype=np.int32), np.zeros(max(n, 1), dtype=np.int64)
        victims, admitted = np.zeros(max(n, 1), dtype=np.int32), np.zeros(max(n, 1), dtype=np.int32)
        ne, nv, na = c_int(), c_int(), c_int()
        ptr = lambda a: a.ctypes.data
        rc = _core().vs_schedule(self._h, int(max_num_seqs), int(max_num_batched_tokens), int(prefill_chunk_size),
                                 int(n_run), n - int(n_run), ptr(rem), ptr(comp), ptr(keys), ptr(arr), ptr(e_seq),
                                 ptr(e_cnt), ctypes.addressof(ne), ptr(victims), ctypes.addressof(nv), ptr(admitted),
                                 ctypes.addressof(na))
        if rc == -1:
            raise OutOfPages("a sequence cannot get its pages although it runs alone")
        if rc < 0:
            raise PoolError(_ERR.get(rc, f"native cache core error {rc}"))
        return (list(zip(e_seq[:ne.value].tolist(), e_cnt[:ne.value].tolist())), victims[:nv.value].tolist(),
                admitted[:na.value].tolist())

    def decode_step(self, request_ids, tokens, pad_to: int, fixed_blocks: int, max_tokens: int, out: np.ndarray):
        """One token for each of the requests, in one call of the core: the check that the pools can
        take them (OutOfPages, nothing changed, if not), the appends, the packed batch (as `pack_step`
        with pad_to) written into `out`, and the release of pages behind windows.  Returns (words
        used, offsets, sizes, positions of the tokens); a negative first value is the size `out`
        must have, and None is returned when a request would grow beyond max_tokens (nothing was
        changed in either case)."""
        B = len(request_ids)
        G = self.num_groups
        keys = np.fromiter((self._keys[r] for r in request_ids), dtype=np.int64, count=B)
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        offsets = np.zeros(8 + 2 * G, dtype=np.int32)
        sizes = np.zeros(8 + 2 * G, dtype=np.int32)
        starts = np.zeros(B, dtype=np.int64)
        ptr = lambda a: a.ctypes.data
        used = _core().vc_decode_step(self._h, B, ptr(keys), ptr(tokens), int(pad_to), int(fixed_blocks),
                                      int(max_tokens), ptr(out), out.shape[0], ptr(offsets), ptr(sizes), ptr(starts))
        if used == -8:
            return None
        if used == -1:
            raise OutOfPages(f"the step needs more pages than are free {self.free_pages()}")
        if used < 0:
            if used == -2:
                raise KeyError(_ERR[-2])
            raise PoolError(_ERR.get(int(used), f"native cache core error {used}"))
        if used > out.shape[0]:
            return -int(used), offsets, sizes, starts
        return int(used), offsets, sizes, starts

    # ---- packing a step (used by the step function) ---------------------------
    def pack_step(self, request_ids, counts, starts, tokens, want_offsets, wants, pad_to, tile_rows, fixed_blocks,
                  out: np.ndarray):
        """Writes the packed batch into `out` (int32).  Returns (words used, offsets, sizes, max_blocks)
        or raises; when `out` is too small returns the words needed as a negative number."""
        B = len(request_ids)
        G = self.num_groups
        keys = np.fromiter((self._keys[r] for r in request_ids), dtype=np.int64, count=B)
        counts = np.ascontiguousarray(counts, dtype=np.int32)
        starts = np.ascontiguousarray(starts, dtype=np.int64)
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        want_offsets = np.ascontiguousarray(want_offsets, dtype=np.int32)
        wants = np.ascontiguousarray(wants if len(wants) else [0], dtype=np.int32)
        max_blocks = np.full(max(G, 1), int(fixed_blocks), dtype=np.int32)
        offsets = np.zeros(8 + 2 * G, dtype=np.int32)
        sizes = np.zeros(8 + 2 * G, dtype=np.int32)
        ptr = lambda a: a.ctypes.data
        used = _core().vc_pack_step(self._h, B, ptr(keys), ptr(counts), ptr(starts), ptr(tokens), ptr(want_offsets),
                                    ptr(wants), int(pad_to), int(tile_rows), ptr(max_blocks), ptr(out),
                                    out.shape[0], ptr(offsets), ptr(sizes))
        if used < 0:
            self._call("vc_check") if used == -7 else None
            if used == -6:
                raise PoolError(_ERR[-6])
            raise ValueError(_ERR.get(int(used), f"native cache core error {used}"))
        if used > out.shape[0]:
            return -int(used), None, None, None
        return int(used), offsets, sizes, max_blocks[:G]
