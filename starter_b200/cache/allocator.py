"""Hands out numbered resources (sequence slots, cache pages) and takes them back.

Pure host logic.  A number is held by at most one owner; handing back a number
that is not held, or asking for more than are free, is an error and changes
nothing.
"""

from __future__ import annotations


class CacheFull(RuntimeError):
    """More slots or pages were asked for than are free."""


class IndexAllocator:
    def __init__(self, count: int, what: str = "index"):
        if count < 0:
            raise ValueError(f"cannot manage {count} {what}s")
        self.count = count
        self.what = what
        # lowest numbers are handed out first, so a small workload stays in a small part of memory
        self._free = list(range(count - 1, -1, -1))
        self._held = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return len(self._held)

    def is_held(self, index: int) -> bool:
        return index in self._held

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.count} {self.what}s are in use")
        index = self._free.pop()
        self._held.add(index)
        return index

    def take_many(self, n: int) -> list:
        if n > len(self._free):
            raise CacheFull(f"{n} {self.what}s wanted, {len(self._free)} of {self.count} free")
        return [self.take() for _ in range(n)]

    def give_back(self, index: int) -> None:
        if index not in self._held:
            raise ValueError(f"{self.what} {index} is not held, so it cannot be given back")
        self._held.remove(index)
        self._free.append(index)

    def check(self) -> None:
        """Every number is either free or held, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        if free & self._held:
            raise AssertionError(f"a {self.what} is both free and held")
        if len(free) + len(self._held) != self.count:
            raise AssertionError(f"a {self.what} was lost")
