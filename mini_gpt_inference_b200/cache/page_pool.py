"""Fixed pools of page ids and of state slots.

Free pages are handed out last-freed-first, like the reference's list used as a stack
(src/minigpt_infer/cache/paged.py:38, 63, 76, 80), so a page that was just given back
is the next one used again.  Unlike the reference, a page freed twice or a page that is
not out is an error here, not a silent corruption of the free list.
"""

from __future__ import annotations


class PoolError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        # pop() takes from the end: start so that page 0 goes out first.
        self._free = list(range(num_pages - 1, -1, -1))
        self._out = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            raise PoolError(f"asked for {count} pages, {len(self._free)} free")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            self._out[p] = 1
        return pages

    def give_back(self, pages) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise PoolError(f"page {p} is not of this pool")
            if not self._out[p]:
                raise PoolError(f"page {p} given back twice (or never taken)")
            self._out[p] = 0
            self._free.append(p)

    def check(self) -> None:
        """No page lost, none listed free twice, none both free and out."""
        if len(set(self._free)) != len(self._free):
            raise PoolError("a page is listed free twice")
        for p in self._free:
            if self._out[p]:
                raise PoolError(f"page {p} is both free and out")
        if len(self._free) + sum(self._out) != self.num_pages:
            raise PoolError("a page is lost")


class SlotPool(PagePool):
    """Slots for per-request state of fixed size: one per running request."""

    def take_one(self) -> int:
        return self.take(1)[0]
