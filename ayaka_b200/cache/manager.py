"""The cache manager: who holds which page. Host bookkeeping only; no tensor lives here.

Keys and values are kept in pages of ``page_size`` tokens. Layers whose mixers have the
same need (geometry and window) form a *group*; every group has its own pool of page ids
and its own block table, because a group that keeps all keys and one that keeps a window
of them hold different pages at different times. A request gets one table row for life
(also the index of its slot in every per-request state tensor); ``table[group][row, i]`` is
the page that holds tokens ``i * page_size ..`` of that request, or 0 for "no page" (page 0
is padding and is never handed out).

The three calls follow the reference's manager (``python/ayaka/kvcache/manager.py:248-340,
407-419``): ``allocate(id, n)`` makes room for ``n`` more tokens beyond the committed ones,
in all groups or in none, and returns ``False`` instead of raising or evicting when pages,
a row or the table's width run out; ``commit(id, n)`` records that the step wrote them;
``free(id)`` gives everything back. Added here: a windowed group gives a page back as soon
as a commit has moved the window past it, and freed pages are reused first (LIFO).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ayaka_b200.errors import CapacityError, EngineError
from ayaka_b200.parts.base import CacheNeed

__all__ = ["CacheManager", "PagePool"]


class PagePool:
    """Page ids ``1 .. num_pages - 1`` of one group: a LIFO free stack and reference counts."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 2:
            raise CapacityError(f"a pool needs at least 2 pages (page 0 is padding), got "
                                f"{num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, 0, -1))  # pop() hands out 1, 2, 3, ...
        self._refs = np.zeros(num_pages, dtype=np.int32)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_usable(self) -> int:
        return self.num_pages - 1

    def take(self) -> int | None:
        if not self._free:
            return None
        page = self._free.pop()
        self._refs[page] = 1
        return page

    def give(self, page: int) -> None:
        if not 0 < page < self.num_pages:
            raise EngineError(f"page {page} does not exist")
        if self._refs[page] <= 0:
            raise EngineError(f"page {page} is given back twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refs(self, page: int) -> int:
        return int(self._refs[page])

    def free_pages(self) -> list[int]:
        return list(self._free)


@dataclass(slots=True)
class _Held:
    row: int
    committed: int = 0
    reserved: int = 0  # tokens beyond `committed` that pages exist for
    pages_hi: int = 0  # every live table entry below this index holds a page


class CacheManager:
    """Pages and table rows of every live request, for all groups.

    Args:
        needs: one :class:`CacheNeed` per group.
        num_pages: pages per group's pool, page 0 included.
        page_size: tokens per page, shared by all groups.
        max_requests: rows of every block table.
        max_pages_per_request: width of every block table.
    """

    def __init__(self, needs: list[CacheNeed], num_pages: list[int], page_size: int,
                 max_requests: int, max_pages_per_request: int) -> None:
        if len(needs) != len(num_pages):
            raise ValueError("one page count per group")
        if page_size < 1 or max_requests < 1 or max_pages_per_request < 1:
            raise ValueError("page_size, max_requests and max_pages_per_request must be >= 1")
        self.needs = list(needs)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_pages_per_request = max_pages_per_request
        self.pools = [PagePool(count) for count in num_pages]
        self.tables = [np.zeros((max_requests, max_pages_per_request), dtype=np.int32)
                       for _ in needs]
        self._free_rows = list(range(max_requests - 1, -1, -1))  # pop() hands out 0, 1, 2, ...
        self._held: dict[str, _Held] = {}
        self._fresh_rows: list[int] = []

    # ---- limits -------------------------------------------------------------------------
    @property
    def max_tokens_per_request(self) -> int:
        return self.max_pages_per_request * self.page_size

    @property
    def max_context_tokens(self) -> int:
        """Longest sequence one request can ever hold (a windowed group never limits it
        below its window plus a page)."""
        limit = self.max_tokens_per_request
        for need, pool in zip(self.needs, self.pools):
            if need.window == 0:
                limit = min(limit, pool.num_usable * self.page_size)
        return limit

    def pages_needed(self, group: int, committed: int, total: int) -> int:
        """Pages group ``group`` must hold for a request with ``committed`` tokens stored
        that is about to hold ``total``."""
        first = self._first_live_page(group, committed)
        return max(0, -(-total // self.page_size) - first)

    def _first_live_page(self, group: int, committed: int) -> int:
        window = self.needs[group].window
        if window == 0:
            return 0
        # the next row sits at position `committed` and sees keys committed - window + 1 ..
        oldest = max(0, committed - window + 1)
        return oldest // self.page_size

    # ---- queries ------------------------------------------------------------------------
    def __contains__(self, request_id: str) -> bool:
        return request_id in self._held

    def row(self, request_id: str) -> int:
        return self._held[request_id].row

    def held(self, request_id: str) -> _Held:
        """Row and token counts of a live request (read only)."""
        return self._held[request_id]

    def committed(self, request_id: str) -> int:
        held = self._held.get(request_id)
        return 0 if held is None else held.committed

    def live_requests(self) -> list[str]:
        return list(self._held)

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def take_fresh_rows(self) -> list[int]:
        """Rows handed to new requests since the last call; their state slots must be zeroed."""
        fresh, self._fresh_rows = self._fresh_rows, []
        return fresh

    # ---- the three calls ----------------------------------------------------------------
    def allocate(self, request_id: str, num_tokens: int) -> bool:
        """Make room for ``num_tokens`` tokens beyond the committed ones. Idempotent until
        the next commit (asking again for the same or fewer tokens changes nothing)."""
        if num_tokens < 0:
            raise ValueError("num_tokens must not be negative")
        held = self._held.get(request_id)
        new_request = held is None
        if held is None:
            if not self._free_rows:
                return False
            held = _Held(row=self._free_rows[-1])
        total = held.committed + num_tokens
        if total > self.max_tokens_per_request:
            return False
        page_hi = -(-total // self.page_size)
        if not new_request and page_hi <= held.pages_hi:  # the usual decode step: the last page still has room
            if num_tokens > held.reserved:
                held.reserved = num_tokens
            return True
        plan: list[list[int]] = []
        for group, pool in enumerate(self.pools):
            table = self.tables[group][held.row]
            first = self._first_live_page(group, held.committed)
            lacking = [index for index in range(first, page_hi) if table[index] == 0]
            if len(lacking) > pool.num_free:
                return False
            plan.append(lacking)
        if new_request:
            self._free_rows.pop()
            self._held[request_id] = held
            self._fresh_rows.append(held.row)
        for group, lacking in enumerate(plan):
            table = self.tables[group][held.row]
            for index in lacking:
                page = self.pools[group].take()
                assert page is not None
                table[index] = page
        held.reserved = max(held.reserved, num_tokens)
        held.pages_hi = max(held.pages_hi, page_hi)
        return True

    def commit(self, request_id: str, num_tokens: int) -> None:
        """Record that ``num_tokens`` more tokens were written; a windowed group gives back
        the pages the window has left behind."""
        held = self._held.get(request_id)
        if held is None:
            raise EngineError(f"commit for the unknown request {request_id!r}")
        if num_tokens < 0 or num_tokens > held.reserved:
            raise EngineError(
                f"request {request_id!r} commits {num_tokens} tokens but {held.reserved} "
                "were allocated")
        before = held.committed
        held.committed += num_tokens
        held.reserved -= num_tokens
        for group, need in enumerate(self.needs):
            if need.window == 0:
                continue
            table = self.tables[group][held.row]
            for index in range(self._first_live_page(group, before),
                               self._first_live_page(group, held.committed)):
                if table[index]:
                    self.pools[group].give(int(table[index]))
                    table[index] = 0

    def free(self, request_id: str) -> None:
        """Give back every page and the row of a request; an unknown id is ignored."""
        held = self._held.pop(request_id, None)
        if held is None:
            return
        for group, pool in enumerate(self.pools):
            table = self.tables[group][held.row]
            # last page first, so the next request takes them in ascending order again
            for index in range(self.max_pages_per_request - 1, -1, -1):
                if table[index]:
                    pool.give(int(table[index]))
                    table[index] = 0
        self._free_rows.append(held.row)
        if held.row in self._fresh_rows:
            self._fresh_rows.remove(held.row)

    # ---- self check ---------------------------------------------------------------------
    def check_integrity(self) -> None:
        """Raise :class:`EngineError` if a page is lost, held twice or both free and held,
        if a row is shared, or if a table holds pages its request should not have."""
        rows = [held.row for held in self._held.values()]
        if len(set(rows)) != len(rows):
            raise EngineError("two requests share a table row")
        if set(rows) & set(self._free_rows) or \
                len(rows) + len(self._free_rows) != self.max_requests:
            raise EngineError("table rows are lost or both free and held")
        for group, pool in enumerate(self.pools):
            table = self.tables[group]
            free = pool.free_pages()
            if len(set(free)) != len(free):
                raise EngineError(f"group {group}: a page is in the free list twice")
            held_pages: list[int] = []
            live = np.zeros(self.max_requests, dtype=bool)
            for request_id, held in self._held.items():
                live[held.row] = True
                row = table[held.row]
                first = self._first_live_page(group, held.committed)
                last = -(-(held.committed + held.reserved) // self.page_size)
                if held.pages_hi > last:
                    raise EngineError(
                        f"request {request_id!r} counts {held.pages_hi} table entries as "
                        f"filled but its tokens end in page {last}")
                for index in range(self.max_pages_per_request):
                    page = int(row[index])
                    if page and not first <= index < max(last, first):
                        raise EngineError(
                            f"group {group}: request {request_id!r} holds page {page} at "
                            f"index {index}, outside its live range [{first}, {last})")
                    if not page and first <= index < last:
                        raise EngineError(
                            f"group {group}: request {request_id!r} lacks a page at index "
                            f"{index}")
                    if page:
                        held_pages.append(page)
            if np.any(table[~live] != 0):
                raise EngineError(f"group {group}: a free table row holds pages")
            if len(set(held_pages)) != len(held_pages):
                raise EngineError(f"group {group}: a page is held twice")
            if set(held_pages) & set(free):
                raise EngineError(f"group {group}: a page is both free and held")
            if len(held_pages) + len(free) != pool.num_usable:
                raise EngineError(
                    f"group {group}: {pool.num_usable - len(held_pages) - len(free)} pages "
                    "are lost")
            for page in held_pages:
                if pool.refs(page) != 1:
                    raise EngineError(f"group {group}: page {page} has reference count "
                                      f"{pool.refs(page)}")
            for page in free:
                if pool.refs(page) != 0:
                    raise EngineError(f"group {group}: free page {page} has references")
