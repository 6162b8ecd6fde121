"""Fixed pool of ids handed out and taken back in O(1), last freed first.

The block allocator of davidjoyme/flashdecode-cuda (engine/paged_cache.py:85-119)
is a LIFO list whose ``free`` builds a set of the whole free list to catch a
double free; here a per-id flag does that check in O(1).  The same class hands
out cache blocks and sequence slots.
"""

from __future__ import annotations

from typing import Iterable, List


class PoolExhausted(MemoryError):
    """More ids were asked for than the pool has free."""


class IdAllocator:
    def __init__(self, count: int, what: str = "block"):
        if count < 0:
            raise ValueError(f"{what} pool size must be >= 0, got {count}")
        self.count = count
        self.what = what
        # reversed so the first ids handed out are 0, 1, 2, ...
        self._free: List[int] = list(range(count - 1, -1, -1))
        self._in_use = bytearray(count)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.count - len(self._free)

    def in_use(self, i: int) -> bool:
        return 0 <= i < self.count and bool(self._in_use[i])

    def allocate(self, n: int = 1) -> List[int]:
        if n < 0:
            raise ValueError(f"cannot allocate {n} {self.what}s")
        if n > len(self._free):
            raise PoolExhausted(f"{self.what} pool exhausted: asked for {n}, {len(self._free)} free of {self.count}")
        out = [self._free.pop() for _ in range(n)]
        for i in out:
            self._in_use[i] = 1
        return out

    def free(self, ids: Iterable[int]) -> None:
        ids = list(ids)
        seen = set()
        for i in ids:        # check everything before changing anything
            if not (0 <= i < self.count):
                raise ValueError(f"{self.what} {i} is outside the pool of {self.count}")
            if not self._in_use[i] or i in seen:
                raise ValueError(f"double free of {self.what} {i}")
            seen.add(i)
        for i in ids:
            self._in_use[i] = 0
            self._free.append(i)
