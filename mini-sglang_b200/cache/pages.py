"""Page pool: ids 1..n handed out first-in first-out; page 0 is never handed out (it is the
dump target of padded rows and of block-table entries whose page was given back).

The reference keeps the free ids in a device tensor (mini_sglang/mem_cache/token2kv.py:154-212);
here the list lives on the host, so allocation never waits for the device, and every page's
state is tracked so that a page lost, held twice or freed twice is an error at the moment it
happens."""

from __future__ import annotations

from collections import deque
from typing import Iterable, List


class OutOfPages(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = deque(range(1, num_pages + 1))
        self._held = bytearray(num_pages + 1)      # 1 while a page is out

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        out = [self._free.popleft() for _ in range(n)]
        for p in out:
            self._held[p] = 1
        return out

    def free(self, pages: Iterable[int]) -> None:
        for p in pages:
            if p <= 0 or p > self.num_pages:
                raise ValueError(f"page {p} does not belong to this pool")
            if not self._held[p]:
                raise ValueError(f"page {p} freed twice")
            self._held[p] = 0
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return bool(self._held[page])

    def reset(self) -> None:
        self._free = deque(range(1, self.num_pages + 1))
        self._held = bytearray(self.num_pages + 1)
