"""The cache manager: pages, block tables, state slots.  Host-side bookkeeping only, no device code.

* A **group** is a set of cache-writing schedule positions with the same need (the mixer's
  ``CacheSpec``: its streams and what it retains).  Each group has its own pool of page ids and one block table per request: page ``i`` of a
  request holds its positions ``[i*page_size, (i+1)*page_size)`` for every layer of the group.
  (The reference allocates per layer, src/quanta/paged/paged_kv_cache.py:229-238; layers with equal
  needs always move together, so here they share one table.)
* Pages are reserved before a step for the positions it will write, given back when a request ends
  and as soon as the group's retention rule (``Retention.needed_ranges``: everything, a window, or a
  rule of the mixer's own) says that no future query reads any position of the page.  Freed pages are reused first-in first-out (src/quanta/paged/block_pool.py:67-106).
* A **state slot** is a row index into per-request state of fixed size (a mixer's own state, the
  sampler's counters).  Every live request holds exactly one.
* Running out is an exception (``OutOfPages`` / ``OutOfSlots``) raised before anything is changed; it
  is the scheduler's job to decide what happens then.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

from ..parts.base import CacheSpec, Retention


class OutOfPages(RuntimeError):
    pass


class OutOfSlots(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        self.num_pages = int(num_pages)
        self._free = deque(range(self.num_pages))
        self._held = [False] * self.num_pages
        self.high_water = 0
        self.allocations = 0

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> list[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} page(s) wanted, {len(self._free)} free of {self.num_pages}")
        out = [self._free.popleft() for _ in range(n)]
        for p in out:
            assert not self._held[p], f"page {p} handed out twice"
            self._held[p] = True
        self.allocations += n
        self.high_water = max(self.high_water, self.used_count)
        return out

    def give_back(self, pages) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages) or not self._held[p]:
                raise RuntimeError(f"page {p} freed but not held")
            self._held[p] = False
            self._free.append(p)


class SlotPool:
    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free = deque(range(self.num_slots))
        self._held = [False] * self.num_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} state slots are held")
        s = self._free.popleft()
        self._held[s] = True
        return s

    def give_back(self, s: int) -> None:
        if not self._held[s]:
            raise RuntimeError(f"slot {s} freed but not held")
        self._held[s] = False
        self._free.append(s)


@dataclass
class CacheGroup:
    spec: CacheSpec
    positions: list[int]                 # schedule positions whose streams live in this group's pages
    pool: PagePool
    tables: dict = field(default_factory=dict)     # request id -> list of page ids (-1: given back)
    arrays: dict = field(default_factory=dict)     # request id -> int32 array with the same entries (for packing a step)
    # retention: request id -> [first page index not yet passed by the open range, held page indices below it]
    passed: dict = field(default_factory=dict)

    @property
    def window(self):
        return self.spec.window

    @property
    def keeps_all(self) -> bool:
        return type(self.spec.retention).needed_ranges is Retention.needed_ranges


@dataclass
class RequestRecord:
    slot: int
    length: int = 0            # tokens whose K/V are in the cache
    reserved: int = 0          # positions [0, reserved) have pages (where the window still needs them)


class CacheManager:
    def __init__(self, needs: list[CacheSpec | None], page_size: int, num_pages: int, max_requests: int):
        """``needs[pos]``: what schedule position ``pos`` keeps (None: nothing).  Every group gets
        ``num_pages`` pages of ``page_size`` tokens."""
        if page_size <= 0 or num_pages <= 0 or max_requests <= 0:
            raise ValueError("page_size, num_pages and max_requests must be positive")
        self.page_size = int(page_size)
        self.groups: list[CacheGroup] = []
        self.group_of: dict[int, int] = {}
        by_spec: dict[CacheSpec, int] = {}
        for pos, spec in enumerate(needs):
            if spec is None:
                continue
            if spec not in by_spec:
                by_spec[spec] = len(self.groups)
                self.groups.append(CacheGroup(spec, [], PagePool(num_pages)))
            g = by_spec[spec]
            self.groups[g].positions.append(pos)
            self.group_of[pos] = g
        self.slots = SlotPool(max_requests)
        self.requests: dict = {}
        self.preemptions = 0
        self.on_free = None        # called with the slot index when a request gives its slot back

    # ---- requests ---------------------------------------------------------------------------------
    def has(self, rid) -> bool:
        return rid in self.requests

    def add_request(self, rid) -> int:
        if rid in self.requests:
            raise KeyError(f"request {rid!r} is already live")
        slot = self.slots.take()
        self.requests[rid] = RequestRecord(slot)
        for g in self.groups:
            g.tables[rid] = []
            g.arrays[rid] = np.full(16, -1, dtype=np.int32)
            g.passed[rid] = [0, []]
        return slot

    def length(self, rid) -> int:
        return self.requests[rid].length

    def slot(self, rid) -> int:
        return self.requests[rid].slot

    def pages_needed(self, rid, new_length: int) -> list[int]:
        """New pages each group must get so that positions ``[0, new_length)`` can be written (a
        request the manager does not know yet holds none)."""
        want_pages = -(-new_length // self.page_size)
        return [max(0, want_pages - len(g.tables.get(rid, ()))) for g in self.groups]

    def can_reserve(self, wants: dict) -> bool:
        """``wants``: request id -> new length.  True if every group can serve all of them together."""
        for gi, g in enumerate(self.groups):
            need = sum(self.pages_needed(rid, n)[gi] for rid, n in wants.items())
            if need > g.pool.free_count:
                return False
        return True

    def reserve(self, rid, new_length: int) -> None:
        """Give ``rid`` pages for positions up to ``new_length``; all groups or none."""
        rec = self.requests[rid]
        needs = self.pages_needed(rid, new_length)
        for g, n in zip(self.groups, needs):
            if n > g.pool.free_count:
                raise OutOfPages(f"request {rid!r} needs {n} more page(s) to hold {new_length} tokens; "
                                 f"{g.pool.free_count} free of {g.pool.num_pages}")
        for g, n in zip(self.groups, needs):
            if n == 0:
                continue
            table, new = g.tables[rid], g.pool.take(n)
            start = len(table)
            table.extend(new)
            arr = g.arrays[rid]
            if len(table) > arr.size:
                grown = np.full(max(2 * arr.size, len(table)), -1, dtype=np.int32)
                grown[:start] = arr[:start]
                arr = g.arrays[rid] = grown
            arr[start:len(table)] = new
        rec.reserved = max(rec.reserved, new_length)

    def advance(self, rid, n_tokens: int) -> None:
        """``n_tokens`` more tokens are in the cache; give back pages the window has passed."""
        rec = self.requests[rid]
        if rec.length + n_tokens > rec.reserved:
            raise RuntimeError(f"request {rid!r}: advancing to {rec.length + n_tokens} past its reservation {rec.reserved}")
        rec.length += n_tokens
        for g in self.groups:
            if not g.keeps_all:
                self._release_unneeded(g, rid, rec.length)

    def _release_unneeded(self, g: CacheGroup, rid, length: int) -> None:
        """Give back the pages of ``rid`` that no query at a position >= ``length`` reads.  The last range
        of the rule is open-ended and only moves forward; pages it has passed are looked at once when it
        passes them and again only while an earlier (closed) range still holds them."""
        ps = self.page_size
        ranges = g.spec.retention.needed_ranges(length)
        if not ranges or ranges[-1][1] is not None:
            raise ValueError(f"{type(g.spec.retention).__name__}.needed_ranges must end with an open range")
        table, state = g.tables[rid], g.passed[rid]
        upto = min(ranges[-1][0] // ps, len(table))
        if upto > state[0]:
            state[1].extend(range(state[0], upto))
            state[0] = upto
        closed = ranges[:-1]
        held, gone = [], []
        for i in state[1]:
            lo, hi = i * ps, (i + 1) * ps
            (held if any(a < hi and b > lo for a, b in closed) else gone).append(i)
        state[1] = held
        if gone:
            g.pool.give_back([table[i] for i in gone if table[i] >= 0])
            for i in gone:
                table[i] = -1
            g.arrays[rid][gone] = -1

    def free(self, rid) -> None:
        rec = self.requests.pop(rid)
        for g in self.groups:
            g.pool.give_back([p for p in g.tables.pop(rid) if p >= 0])
            g.arrays.pop(rid, None)
            g.passed.pop(rid, None)
        self.slots.give_back(rec.slot)
        if self.on_free is not None:
            self.on_free(rec.slot)

    # ---- views for a step ---------------------------------------------------------------------------
    def block_table_rows(self, group: int, rids: list) -> list[list[int]]:
        return [self.groups[group].tables[r] for r in rids]

    def block_table_matrix(self, group: int, rids: list, max_pages: int) -> np.ndarray:
        """int32 ``[len(rids), max_pages]``: the requests' page ids, -1 where a request holds none."""
        g = self.groups[group]
        out = np.full((len(rids), max_pages), -1, dtype=np.int32)
        for r, rid in enumerate(rids):
            n = min(len(g.tables[rid]), max_pages)
            out[r, :n] = g.arrays[rid][:n]
        return out

    def stats(self) -> dict:
        return {"groups": [{"pages": g.pool.num_pages, "used": g.pool.used_count,
                            "high_water": g.pool.high_water, "allocations": g.pool.allocations,
                            "window": g.window, "layers": len(g.positions)} for g in self.groups],
                "live_requests": len(self.requests), "preemptions": self.preemptions}

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; every live request holds one slot."""
        for g in self.groups:
            held = [p for t in g.tables.values() for p in t if p >= 0]
            if len(held) != len(set(held)):
                raise AssertionError("a page is held by two requests")
            free = list(g.pool._free)
            if set(free) & set(held):
                raise AssertionError("a held page is on the free list")
            if len(free) + len(held) != g.pool.num_pages or len(set(free)) != len(free):
                raise AssertionError("a page is lost or listed free twice")
            for rid, t in g.tables.items():
                if g.arrays[rid][: len(t)].tolist() != t:
                    raise AssertionError("the packed copy of a block table differs from the table")
        slots = [r.slot for r in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) + self.slots.free_count != self.slots.num_slots:
            raise AssertionError("state slots are inconsistent")
