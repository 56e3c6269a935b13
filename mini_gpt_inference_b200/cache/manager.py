"""Host-side cache manager: page tables per request and per layer group, state slots.

It owns no tensors.  Layers with equal needs (``PagedKVSpec``) form a group; each group
has a page pool and a page size of its own (the manager's defaults unless its spec says
otherwise) and every request has one block table per group, shared by
the group's layers — the same page id indexes every layer's storage, as in the
reference (src/minigpt_infer/cache/paged.py:122-123, 154-155).  Pages are given back
when a request is released (src/minigpt_infer/cache/paged.py:79-81) or, in a group with
a window, as soon as no later query can read them.  A request also holds one slot of
the state pool from admission to release, whether or not any layer keeps state.

Growth is asked for in two halves so that a caller can back out: ``reserve`` takes the
pages a request needs to reach a length (all groups or none), ``advance`` records that
the tokens are now in the cache.
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass, field

from .page_pool import PagePool, PoolError, SlotPool
from .spec import FixedStateSpec, PagedKVSpec

NO_PAGE = -1


class CacheFullError(RuntimeError):
    """Not enough free pages (or slots) for what was asked."""


@dataclass
class CacheGroup:
    spec: PagedKVSpec
    layers: list[int]
    pool: PagePool
    page_tokens: int

    @property
    def num_pages(self) -> int:
        return self.pool.num_pages

    def pages_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_tokens - 1) // self.page_tokens


@dataclass
class RequestCache:
    request_id: str
    state_slot: int
    length: int = 0                                   # tokens in the cache
    tables: list[list[int]] = field(default_factory=list)   # per group: page id per page index
    # (serial, version) names one state of the tables: serial is unique per admission, version
    # counts their changes, so a copy of the tables kept elsewhere knows when it is stale
    serial: int = 0
    version: int = 0
    capacity: int = 0                                 # tokens its pages have room for (every group)


class CacheManager:
    def __init__(self, layer_specs, page_tokens: int, num_pages: int, max_requests: int,
                 window_slack_tokens: int | None = None) -> None:
        """``page_tokens`` and ``num_pages``: the geometry of every group whose spec names none.
        ``window_slack_tokens``: the most tokens a request writes in one step (a windowed group
        sizes its pool for ``window + slack`` tokens per request slot); None: no such bound is
        known, and a windowed group gets the default pool."""
        if page_tokens <= 0:
            raise ValueError("page_tokens must be positive")
        self.page_tokens = page_tokens
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.window_slack_tokens = window_slack_tokens
        self.groups: list[CacheGroup] = []
        self.group_of_layer: dict[int, int] = {}
        self.state_layers: dict[int, FixedStateSpec] = {}
        for layer, spec in enumerate(layer_specs):
            if spec is None:
                continue
            if isinstance(spec, FixedStateSpec):
                self.state_layers[layer] = spec
            elif isinstance(spec, PagedKVSpec):
                for g, group in enumerate(self.groups):
                    if group.spec == spec:
                        group.layers.append(layer)
                        self.group_of_layer[layer] = g
                        break
                else:
                    self.group_of_layer[layer] = len(self.groups)
                    pt, pages = self._geometry(spec)
                    self.groups.append(CacheGroup(spec, [layer], PagePool(pages), pt))
            else:
                raise TypeError(f"layer {layer}: unknown cache spec {spec!r}")
        self.slots = SlotPool(max_requests)
        self.requests: dict[str, RequestCache] = {}
        self._serial = 0                      # admissions so far
        self._none_needed = (0,) * len(self.groups)
        self._any_window = any(g.spec.window is not None for g in self.groups)

    # ---- sizes -------------------------------------------------------------------
    def _geometry(self, spec: PagedKVSpec) -> tuple[int, int]:
        pt = spec.page_tokens or self.page_tokens
        if spec.num_pages is not None:
            return pt, spec.num_pages
        # the default pool holds num_pages * page_tokens tokens, whatever the group's page size
        pages = max(1, self.num_pages * self.page_tokens // pt)
        if spec.window is not None and self.window_slack_tokens is not None:
            # pages a request can hold at once: the window, the tokens of one step, and the two
            # pages that the window's and the portion's ends share with their neighbours
            per_request = (spec.window + self.window_slack_tokens + pt - 1) // pt + 2
            pages = min(pages, self.max_requests * per_request)
        return pt, pages

    def pages_for(self, num_tokens: int, group: int = 0) -> int:
        pt = self.groups[group].page_tokens if self.groups else self.page_tokens
        return (num_tokens + pt - 1) // pt

    def max_pages_per_request(self, max_tokens: int, group: int = 0) -> int:
        """Width of a block table of ``group``: page indices are absolute positions / page size,
        also in a group with a window (pages it gave back stay in the table as NO_PAGE)."""
        return max(1, self.pages_for(max_tokens, group))

    def can_ever_hold(self, num_tokens: int) -> bool:
        """Whether a request of ``num_tokens`` tokens fits the pools when it is alone (a group
        with a window counts the pages it holds at once, see ``_geometry``)."""
        for group in self.groups:
            need = group.pages_for(num_tokens)
            if group.spec.window is not None:
                slack = self.window_slack_tokens if self.window_slack_tokens is not None else num_tokens
                need = min(need, (group.spec.window + slack + group.page_tokens - 1) // group.page_tokens + 2)
            if need > group.num_pages:
                return False
        return True

    def _first_live_page(self, group: CacheGroup, length: int) -> int:
        """Index of the first page that a query at position >= length may still read."""
        if group.spec.window is None:
            return 0
        first_key = max(0, length - group.spec.window + 1)
        return first_key // group.page_tokens

    def _missing(self, req: RequestCache, new_length: int) -> list[int]:
        """Pages each group still needs so that positions < new_length have a page."""
        need = []
        for g, group in enumerate(self.groups):
            have = len(req.tables[g])
            need.append(max(0, group.pages_for(new_length) - have))
        return need

    # ---- life of a request ----------------------------------------------------------
    def admit(self, request_id: str) -> RequestCache:
        if request_id in self.requests:
            raise PoolError(f"request {request_id!r} is already admitted")
        if self.slots.num_free == 0:
            raise CacheFullError("no state slot free")
        self._serial += 1
        req = RequestCache(request_id, self.slots.take_one(), 0, [[] for _ in self.groups], self._serial,
                           capacity=0 if self.groups else 1 << 30)
        self.requests[request_id] = req
        return req

    def has(self, request_id: str) -> bool:
        return request_id in self.requests

    def get(self, request_id: str) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise PoolError(f"request {request_id!r} is not admitted") from None

    def pages_needed(self, request_id: str | None, new_length: int) -> Sequence[int]:
        """Per group, pages that would have to be taken to reach ``new_length``."""
        if request_id is None or request_id not in self.requests:
            return [group.pages_for(new_length) for group in self.groups]
        req = self.requests[request_id]
        if new_length <= req.capacity:
            return self._none_needed
        return self._missing(req, new_length)

    def can_reserve(self, request_id: str | None, new_length: int) -> bool:
        need = self.pages_needed(request_id, new_length)
        return all(n <= group.pool.num_free for n, group in zip(need, self.groups))

    def tokens_that_fit(self, request_id: str, length: int | None = None) -> int:
        """How many tokens beyond ``length`` (default: what the cache holds) the request could
        store using its pages and all free ones."""
        req = self.get(request_id)
        length = req.length if length is None else length
        room = None
        for g, group in enumerate(self.groups):
            cap = (len(req.tables[g]) + group.pool.num_free) * group.page_tokens - length
            room = cap if room is None else min(room, cap)
        return max(0, room) if room is not None else 1 << 30

    def reserve(self, request_id: str, new_length: int) -> bool:
        """Take the pages needed to hold ``new_length`` tokens.  All groups or none:
        returns False and changes nothing if any group is short."""
        req = self.get(request_id)
        if new_length <= req.capacity:
            return True
        need = self._missing(req, new_length)
        if any(n > group.pool.num_free for n, group in zip(need, self.groups)):
            return False
        for g, (n, group) in enumerate(zip(need, self.groups)):
            if n:
                req.tables[g].extend(group.pool.take(n))
                req.version += 1
        req.capacity = (min(len(t) * group.page_tokens for t, group in zip(req.tables, self.groups))
                        if req.tables else 1 << 30)
        return True

    def advance(self, request_id: str, new_length: int) -> None:
        """Tokens up to ``new_length`` are written.  Gives back pages a window has passed."""
        req = self.get(request_id)
        if new_length < req.length:
            raise PoolError("a request's cache cannot shrink; release and recompute instead")
        if new_length > req.capacity:
            raise PoolError(f"request {request_id!r} advanced past its reserved pages")
        req.length = new_length
        if not self._any_window:
            return
        for g, group in enumerate(self.groups):
            first = self._first_live_page(group, new_length)
            table = req.tables[g]
            passed = [p for p in table[:first] if p != NO_PAGE]
            if passed:
                group.pool.give_back(passed)
                for i in range(min(first, len(table))):
                    table[i] = NO_PAGE
                req.version += 1

    def release(self, request_id: str) -> None:
        req = self.get(request_id)
        for g, group in enumerate(self.groups):
            group.pool.give_back([p for p in req.tables[g] if p != NO_PAGE])
            req.tables[g] = []
        self.slots.give_back([req.state_slot])
        del self.requests[request_id]

    # ---- what a step needs ------------------------------------------------------------
    def block_table(self, request_id: str, group: int) -> list[int]:
        return self.get(request_id).tables[group]

    def slot_of(self, request_id: str, group: int, position: int) -> int:
        """Flat index of a position's row in the group's storage."""
        pt = self.groups[group].page_tokens
        page = self.get(request_id).tables[group][position // pt]
        if page == NO_PAGE:
            raise PoolError(f"position {position} of {request_id!r} was given back already")
        return page * pt + position % pt

    # ---- accounting ---------------------------------------------------------------------
    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free if self.groups else 0

    def stats(self) -> dict[str, int]:
        """As src/minigpt_infer/cache/paged.py:83-94, summed over groups."""
        held_tokens = used_tokens = 0
        for r in self.requests.values():
            for g, group in enumerate(self.groups):
                held_tokens += sum(1 for p in r.tables[g] if p != NO_PAGE) * group.page_tokens
                first = self._first_live_page(group, r.length) * group.page_tokens
                used_tokens += max(0, r.length - first)
        return {
            "free_blocks": sum(g.pool.num_free for g in self.groups),
            "allocated_blocks": sum(g.pool.num_used for g in self.groups),
            "internal_fragmentation_slots": held_tokens - used_tokens,
            "free_state_slots": self.slots.num_free,
            "live_requests": len(self.requests),
        }

    def check(self) -> None:
        """Every page is either free or in exactly one table; the same for slots."""
        for g, group in enumerate(self.groups):
            group.pool.check()
            seen: set[int] = set()
            for r in self.requests.values():
                for p in r.tables[g]:
                    if p == NO_PAGE:
                        continue
                    if p in seen:
                        raise PoolError(f"page {p} of group {g} is held twice")
                    seen.add(p)
            if len(seen) != group.pool.num_used:
                raise PoolError(
                    f"group {g}: {group.pool.num_used} pages out, {len(seen)} in tables")
        self.slots.check()
        slots = [r.state_slot for r in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slots.num_used:
            raise PoolError("state slots and requests disagree")
