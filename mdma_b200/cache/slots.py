"""Bookkeeping of sequence slots and cache pages: plain free lists that refuse
to hand out what is held and to take back what is free."""
from __future__ import annotations


class CacheFull(RuntimeError):
    """No slot or not enough pages are free."""


class FreeList:
    """`n` numbered items; each is either free or held."""

    def __init__(self, n: int, what: str):
        self.what = what
        self.n = n
        self._free = list(range(n - 1, -1, -1))     # pop() hands out the lowest number first
        self._held: set[int] = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held(self) -> frozenset:
        return frozenset(self._held)

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        item = self._free.pop()
        self._held.add(item)
        return item

    def acquire_many(self, count: int) -> list[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.acquire() for _ in range(count)]

    def release(self, item: int) -> None:
        if item not in self._held:
            raise ValueError(f"{self.what} {item} is not held (freed twice, or never given out)")
        self._held.remove(item)
        self._free.append(item)

    def check(self) -> None:
        """Every item is free or held, exactly once."""
        assert len(self._free) == len(set(self._free)), f"a {self.what} is on the free list twice"
        assert not (set(self._free) & self._held), f"a {self.what} is both free and held"
        assert len(self._free) + len(self._held) == self.n, f"a {self.what} was lost"
