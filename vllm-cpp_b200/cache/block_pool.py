"""Free list of page ids with reference counts.

Same shape as the reference's BlockManager (src/core/block_manager.cpp:20-53):
a LIFO list of free ids, ``acquire`` sets the count to one, ``release`` frees at
zero.  LIFO means a page just given back is the next one handed out, which makes
stale contents show up in tests.  Unlike the reference, releasing a page that is
not held is an error instead of a silent second entry in the free list.
"""
from __future__ import annotations

from typing import List, Optional


class PageError(RuntimeError):
    """A page was released twice, or an id is out of range."""


class BlockPool:
    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_blocks = num_blocks
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))   # page 0 is handed out first
        self._refs: List[int] = [0] * num_blocks

    @property
    def num_free(self) -> int:
        return len(self._free)

    def can_allocate(self, n: int) -> bool:
        return len(self._free) >= n

    def acquire(self) -> Optional[int]:
        if not self._free:
            return None
        b = self._free.pop()
        self._refs[b] = 1
        return b

    def inc_ref(self, block: int) -> None:
        self._check(block)
        if self._refs[block] <= 0:
            raise PageError(f"page {block} is not held; its count cannot be raised")
        self._refs[block] += 1

    def release(self, block: int) -> bool:
        """Drop one reference; True if the page went back to the free list."""
        self._check(block)
        if self._refs[block] <= 0:
            raise PageError(f"page {block} released while not held (freed twice?)")
        self._refs[block] -= 1
        if self._refs[block] == 0:
            self._free.append(block)
            return True
        return False

    def ref_count(self, block: int) -> int:
        self._check(block)
        return self._refs[block]

    def _check(self, block: int) -> None:
        if not 0 <= block < self.num_blocks:
            raise PageError(f"page id {block} outside 0..{self.num_blocks - 1}")
