"""Free lists with their invariants: the cache's slots and pages are handed out and
taken back through these, and they refuse what would corrupt the cache (taking
from an empty pool, giving back what is not held, giving back twice)."""
from __future__ import annotations

from typing import List, Set

from ..errors import CacheError


class IdPool:
    """Ids 0..n-1, each either free or held.  The lowest free id is handed out first,
    so that a freed id is used again at once (tests rely on reuse happening)."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))    # pop() takes the lowest
        self._held: Set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def held(self) -> Set[int]:
        return set(self._held)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"the cache has no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def give_back(self, i: int) -> None:
        if i not in self._held:
            if 0 <= i < self.n:
                raise CacheError(f"{self.what} {i} is given back but is not held (freed twice?)")
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        self._held.remove(i)
        # keep the free list sorted descending so that pop() stays the lowest id
        lo, hi = 0, len(self._free)
        while lo < hi:
            mid = (lo + hi) // 2
            if self._free[mid] > i:
                lo = mid + 1
            else:
                hi = mid
        self._free.insert(lo, i)

    def check(self) -> None:
        """Every id is free or held, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError(f"a {self.what} is in the free list twice")
        if free & self._held:
            raise CacheError(f"a {self.what} is both free and held")
        if len(free) + len(self._held) != self.n:
            raise CacheError(f"a {self.what} was lost: {len(free)} free + {len(self._held)} held != {self.n}")
