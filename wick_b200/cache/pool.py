"""Index pools: which slots and which pages are held, and by whom.

Pure host bookkeeping (no tensors), so that it can be tested exhaustively on a
CPU: an index is handed out at most once until it is given back, giving back an
index that is not held is an error, and every index is either free or held.
"""
from __future__ import annotations

from typing import Iterable, List, Set


class PoolError(RuntimeError):
    pass


class PoolExhausted(PoolError):
    pass


class IndexPool:
    """Indices ``0..n-1`` minus ``reserved``; lowest free index first, so that
    freed indices are used again soon (which makes stale contents show up)."""

    def __init__(self, n: int, reserved: Iterable[int] = (), what: str = "index"):
        self.n = n
        self.what = what
        self.reserved: Set[int] = set(reserved)
        if any(not 0 <= r < n for r in self.reserved):
            raise PoolError(f"reserved {what} outside 0..{n - 1}")
        self._free: List[int] = sorted((i for i in range(n) if i not in self.reserved), reverse=True)
        self._held: Set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    @property
    def capacity(self) -> int:
        return self.n - len(self.reserved)

    def held(self) -> Set[int]:
        return set(self._held)

    def is_held(self, i: int) -> bool:
        return i in self._held

    def alloc(self) -> int:
        if not self._free:
            raise PoolExhausted(f"no free {self.what} (all {self.capacity} are held)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def alloc_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise PoolExhausted(f"{k} {self.what}s wanted, {len(self._free)} free of {self.capacity}")
        return [self.alloc() for _ in range(k)]

    def free(self, i: int) -> None:
        if i not in self._held:
            if 0 <= i < self.n and i not in self.reserved:
                raise PoolError(f"{self.what} {i} is given back but is not held (freed twice?)")
            raise PoolError(f"{self.what} {i} does not belong to this pool")
        self._held.remove(i)
        # keep the free list sorted descending so that pop() yields the lowest
        lo, hi = 0, len(self._free)
        while lo < hi:
            mid = (lo + hi) // 2
            if self._free[mid] > i:
                lo = mid + 1
            else:
                hi = mid
        self._free.insert(lo, i)

    def check(self) -> None:
        """Every index is free or held, never both, never lost."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PoolError(f"a {self.what} is in the free list twice")
        if free & self._held:
            raise PoolError(f"a {self.what} is free and held at once")
        if len(free) + len(self._held) != self.capacity:
            raise PoolError(f"a {self.what} was lost: {len(free)} free + {len(self._held)} held != {self.capacity}")
