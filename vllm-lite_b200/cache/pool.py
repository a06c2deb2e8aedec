"""Pools of numbered units (pages, state slots) with a free list.

`allocate(n)` is all-or-nothing and hands out the most recently freed units
first (the reference's allocator is a LIFO free list too,
crates/core/src/scheduler/memory/allocator.rs:51-110), so a replayed trace gets
the same ids.  Unlike the reference, which logs and ignores a double free, a
unit that is freed twice or that was never handed out raises: such a call means
the accounting above is wrong.
"""
from __future__ import annotations


class PoolError(RuntimeError):
    pass


class Pool:
    def __init__(self, size: int, what: str = "page"):
        if size < 0:
            raise ValueError("a pool cannot have a negative size")
        self.size = int(size)
        self.what = what
        self._free = list(range(self.size - 1, -1, -1))   # pop() hands out 0 first
        self._held = [False] * self.size

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.size - len(self._free)

    def allocate(self, n: int):
        """n unit ids, or None (and nothing taken) when fewer than n are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of units")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for u in out:
            self._held[u] = True
        return out

    def release(self, units):
        units = list(units)
        for u in units:
            if not 0 <= u < self.size:
                raise PoolError(f"{self.what} {u} does not exist (pool of {self.size})")
            if not self._held[u]:
                raise PoolError(f"{self.what} {u} is freed twice or was never handed out")
            self._held[u] = False
        self._free.extend(reversed(units))

    def is_held(self, u: int) -> bool:
        return self._held[u]

    def check(self):
        """Every unit is either free exactly once or held."""
        if len(set(self._free)) != len(self._free):
            raise PoolError(f"a {self.what} is on the free list twice")
        for u in self._free:
            if self._held[u]:
                raise PoolError(f"{self.what} {u} is both free and held")
        if sum(self._held) + len(self._free) != self.size:
            raise PoolError(f"a {self.what} is lost: {sum(self._held)} held + {len(self._free)} free != {self.size}")
