"""Host-side bookkeeping of the cache: which slots and which pages are held.

A slot stands for one live sequence; a page holds the keys and values of PAGE
consecutive positions of one sequence. Both allocators refuse to hand out what
is held, to take back what is not, and to take back anything twice.
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot or not enough free pages; the message names the slot."""


class _Pool:
    what = "item"

    def __init__(self, count: int, first: int = 0):
        if count < 0:
            raise CacheError(f"cannot make a pool of {count} {self.what}s")
        self._first = first
        self._count = count
        # LIFO: what was given back last is handed out first, so a stale entry
        # left behind by a finished sequence is met by the very next one.
        self._free: List[int] = list(range(first + count - 1, first - 1, -1))
        self._held = set()

    @property
    def capacity(self) -> int:
        return self._count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held(self):
        return frozenset(self._held)

    def take(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"asked for {n} {self.what}(s), {len(self._free)} free "
                            f"of {self._count}")
        got = [self._free.pop() for _ in range(n)]
        self._held.update(got)
        return got

    def give_back(self, items) -> None:
        items = list(items)
        for i in items:
            if i not in self._held:
                inside = self._first <= i < self._first + self._count
                raise CacheError(f"{self.what} {i} " + ("is not held (freed twice?)" if inside
                                                        else "does not exist"))
        if len(set(items)) != len(items):
            raise CacheError(f"the same {self.what} is given back twice in one call")
        for i in items:
            self._held.remove(i)
            self._free.append(i)

    def check(self) -> None:
        """Nothing lost, nothing held twice."""
        if len(self._free) != len(set(self._free)):
            raise CacheError(f"a free {self.what} is listed twice")
        if self._held & set(self._free):
            raise CacheError(f"a {self.what} is both held and free")
        if len(self._free) + len(self._held) != self._count:
            raise CacheError(f"{self._count - len(self._free) - len(self._held)} {self.what}(s) lost")


class SlotAllocator(_Pool):
    what = "slot"

    def alloc(self) -> int:
        return self.take(1)[0]

    def free(self, slot: int) -> None:
        self.give_back([slot])


class PagePool(_Pool):
    """Pages 0 .. reserved-1 are never handed out (page 0 takes the writes of
    padding rows)."""
    what = "page"

    def __init__(self, count: int, reserved: int = 1):
        super().__init__(count, first=reserved)
        self.reserved = reserved
