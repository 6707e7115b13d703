"""Host-side bookkeeping of pages and slots.

A page holds the keys and values of `page_size` consecutive positions of one request (the
reference's "block" of 16 tokens, src/main.zig:604, src/paged_attention/block.zig:3-33).  The
reference's allocator is a free-list stack with reference counts (`BlockAllocator`,
src/paged_attention/allocator.zig:72-97) and its block table a growable list of physical ids
(src/paged_attention/block_table.zig:4-45); the same here, with every misuse (freeing a page that
is not held, holding one twice) raised as an error instead of corrupting the list.  The device
memory is authoritative; the host keeps only these ids.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """Not enough free pages (or slots) for what was asked; nothing was taken."""


class IdPool:
    """Ids first..first+count-1 with a free-list stack and reference counts."""

    def __init__(self, count: int, first: int = 0, what: str = "page"):
        if count < 0:
            raise ValueError(f"a pool cannot hold {count} {what}s")
        self.count, self.first, self.what = int(count), int(first), what
        self._free: List[int] = list(range(first + count - 1, first - 1, -1))   # pop() gives the lowest id first
        self._refs = {}
        self.high_water = 0
        self.total_allocs = 0

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_used(self) -> int:
        return self.count - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages(f"no free {self.what}")
        i = self._free.pop()
        if i in self._refs:
            raise AssertionError(f"{self.what} {i} was on the free list while held")
        self._refs[i] = 1
        self.total_allocs += 1
        self.high_water = max(self.high_water, self.n_used)
        return i

    def share(self, i: int) -> None:
        if i not in self._refs:
            raise ValueError(f"{self.what} {i} is not held and cannot be shared")
        self._refs[i] += 1

    def free(self, i: int) -> None:
        if i not in self._refs:
            raise ValueError(f"{self.what} {i} is freed but not held")
        self._refs[i] -= 1
        if self._refs[i] == 0:
            del self._refs[i]
            self._free.append(i)

    def held(self, i: int) -> bool:
        return i in self._refs

    def check(self) -> None:
        """Every id is either free once or held, never both, never lost."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        if free & set(self._refs):
            raise AssertionError(f"a {self.what} is both free and held")
        if free | set(self._refs) != set(range(self.first, self.first + self.count)):
            raise AssertionError(f"a {self.what} was lost")
