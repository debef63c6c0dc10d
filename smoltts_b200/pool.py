"""Host-side allocators of the engines' device pools: key/value pages and per-sequence state slots.

Both pools are index allocators over memory the engine owns; the device side sees only the indices (block tables,
slot arrays).  ``IndexPool`` hands out the lowest-numbered free index last (LIFO): an index freed by a finished
sequence is the first one reused, which keeps the working set of pages small and makes reuse bugs show early.
"""
from __future__ import annotations

from typing import Iterable, List

from ._errors import SMOL_ERR_CAPACITY, SmolError


class IndexPool:
    def __init__(self, n: int, what: str = "page"):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n - 1, -1, -1))
        self._is_free = bytearray([1]) * self.n

    def __len__(self) -> int:
        """Indices currently free."""
        return len(self._free)

    def allocate(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise SmolError(SMOL_ERR_CAPACITY, f"{self.what} pool exhausted: need {n}, {len(self._free)} of {self.n} free")
        got = [self._free.pop() for _ in range(n)]
        for i in got:
            self._is_free[i] = 0
        return got

    def free(self, items: Iterable[int]) -> None:
        items = list(items)
        for i in items:
            if not 0 <= i < self.n or self._is_free[i]:
                raise ValueError(f"{self.what} {i} is not an allocated index of this pool")
            self._is_free[i] = 1
        self._free.extend(reversed(items))


class PagePool(IndexPool):
    """Pages of ``page_size`` cached positions each."""

    def __init__(self, n_pages: int, page_size: int):
        super().__init__(n_pages, "KV page")
        self.page_size = int(page_size)

    def pages_for(self, positions: int) -> int:
        return (positions + self.page_size - 1) // self.page_size


class SlotPool(IndexPool):
    """Slots of per-sequence recurrent state."""

    def __init__(self, n_slots: int):
        super().__init__(n_slots, "state slot")
