"""Host-side bookkeeping of the cache: slots and pages.

A *slot* belongs to one sequence from its first step until the sequence ends;
a *page* holds the keys and values of ``page_size`` consecutive positions of
one sequence for every layer of one cache group.  Both are plain free lists
with checks: nothing is handed out twice, nothing is given back twice, and a
request that cannot be met changes nothing.

NNIS gives each sequence a whole session with a cache of its own
(crates/nnis-model/src/session_batch.rs:30-41) and resets lengths to reuse it
(crates/nnis-rt/src/kv_cache.rs:170-172); one shared store with slots is the
batched form of that.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """No slot or not enough pages; the cache is unchanged."""


class SlotError(RuntimeError):
    """A slot or page was used that is not held, or freed twice."""


class FreeList:
    """Hands out the integers 0..n-1; lowest free first, so reuse is prompt."""

    def __init__(self, count: int, what: str):
        if count <= 0:
            raise ValueError(f"a pool of {what}s needs a positive count; got {count}")
        self.count = count
        self.what = what
        self._free: List[int] = list(range(count - 1, -1, -1))
        self._held = [False] * count

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.count - len(self._free)

    def is_held(self, index: int) -> bool:
        return 0 <= index < self.count and self._held[index]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.count} are held)")
        index = self._free.pop()
        self._held[index] = True
        return index

    def take_many(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} {self.what}s wanted, {len(self._free)} of {self.count} free")
        return [self.take() for _ in range(n)]

    def give(self, index: int) -> None:
        if not 0 <= index < self.count:
            raise SlotError(f"{self.what} {index} does not exist (0..{self.count - 1})")
        if not self._held[index]:
            raise SlotError(f"{self.what} {index} is not held (freed twice?)")
        self._held[index] = False
        self._free.append(index)
        # keep "lowest first": the list is popped from its end
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every index is either free once or held, never both."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise SlotError(f"a {self.what} is free twice")
        for i in range(self.count):
            if self._held[i] == (i in set(free)):
                raise SlotError(f"{self.what} {i} is lost or held and free at once")
