"""Host side of the cache: pages, block tables, request slots.

The reference keeps one slot per token (page size 1), a free stack of token
ids on the CPU and a table request -> token ids on the GPU
(``litelang/models/cache.py:105-135,196-249,264-295``).  This manager keeps
pages of ``page_size`` tokens.  It knows nothing about tensors: device storage
lives in ``cache/storage.py`` and mirrors what is decided here.

Groups.  Mixers with equal needs (kv heads, head size, window) share a *group*:
one pool of pages and one block table per request.  A group with a window gives
pages back as soon as every position in them lies before the window of the
request's next token; a group without one keeps them until the request ends.
Beside the paged groups there are *state* groups: one record of fixed size per
request slot, for mixers whose memory does not grow with the sequence.

Nothing here raises when pages run out: ``reserve`` answers False and leaves
everything as it was, and the scheduler decides what happens next.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Tuple

import numpy as np


class CacheError(RuntimeError):
    """A misuse of the manager (double free, unknown slot): a bug in the caller."""


class PageAllocator:
    """LIFO stack of free page ids: a page given back is the next one handed out."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held: Set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        if n < 0:
            raise CacheError("negative page count")
        if n > len(self._free):
            return None
        got = [self._free.pop() for _ in range(n)]
        self._held.update(got)
        return got

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if p not in self._held:
                raise CacheError(f"page {p} is freed but not held")
            self._held.discard(p)
            self._free.append(p)

    def held(self) -> Set[int]:
        return set(self._held)


@dataclass(frozen=True)
class PagedGroupSpec:
    num_kv_heads: int
    head_dim: int               # width of a key
    window: Optional[int]
    planes: int                 # cache planes (one per run-step that writes into this group)
    value_head_dim: Optional[int] = None   # width of a value; None: head_dim; 0: the group has no value plane

    kind = "paged"

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.value_head_dim is None else self.value_head_dim

    def pages_a_request_needs(self, length: int, page_size: int, step_tokens: int) -> int:
        """The most pages a request of ``length`` tokens holds at a time when it grows by at most
        ``step_tokens`` a step: all of them without a window; with one, the window, the step's new tokens
        (pages are given back after the step) and the partly used pages at both ends."""
        full = (length + page_size - 1) // page_size
        if self.window is None:
            return full
        return min(full, (self.window + step_tokens + page_size - 1) // page_size + 1)


@dataclass(frozen=True)
class StateGroupSpec:
    shape: Tuple[int, ...]
    dtype: str
    planes: int

    kind = "state"


class _Request:
    __slots__ = ("length", "pages", "first_live")

    def __init__(self, n_groups: int):
        self.length = 0                                     # tokens whose keys are in the cache
        self.pages: List[List[int]] = [[] for _ in range(n_groups)]   # logical page -> physical (or -1)
        self.first_live: List[int] = [0] * n_groups         # first logical page not yet given back


class CacheManager:
    """Pages and slots for up to ``max_requests`` live requests."""

    def __init__(self, groups: Sequence[object], num_pages: Sequence[int], page_size: int, max_requests: int,
                 max_model_len: int):
        self.groups = list(groups)
        self.paged_ids = [i for i, g in enumerate(self.groups) if g.kind == "paged"]
        self.state_ids = [i for i, g in enumerate(self.groups) if g.kind == "state"]
        if len(num_pages) != len(self.paged_ids):
            raise ValueError("one page count per paged group is needed")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_model_len = int(max_model_len)
        self.max_blocks = (self.max_model_len + self.page_size - 1) // self.page_size
        self.allocators: Dict[int, PageAllocator] = {
            g: PageAllocator(int(n)) for g, n in zip(self.paged_ids, num_pages)
        }
        # block tables: [max_requests, max_blocks] per paged group, -1 = no page
        self.block_tables: Dict[int, np.ndarray] = {
            g: np.full((self.max_requests, self.max_blocks), -1, dtype=np.int32) for g in self.paged_ids
        }
        self.dirty_rows: Dict[int, Set[int]] = {g: set() for g in self.paged_ids}
        self.lengths = np.zeros(self.max_requests, dtype=np.int32)   # tokens cached per slot (0 if closed)
        self._free_slots: List[int] = list(range(self.max_requests - 1, -1, -1))
        self._requests: Dict[int, _Request] = {}
        self.opened_slots: List[int] = []     # slots opened since the storage last looked (state to be zeroed)
        self.pages_handed_out = 0             # counters for tests and reports
        self.pages_reused = 0
        self._ever_used: Dict[int, Set[int]] = {g: set() for g in self.paged_ids}

    # ------------------------------------------------------------------ slots
    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def open(self) -> Optional[int]:
        """A request slot (block-table row and state record), or None when all are taken."""
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._requests[slot] = _Request(len(self.groups))
        self.opened_slots.append(slot)
        return slot

    def close(self, slot: int) -> None:
        """Give back everything the request holds."""
        req = self._get(slot)
        for g in self.paged_ids:
            live = [p for p in req.pages[g] if p >= 0]
            self.allocators[g].free(live)
            n = len(req.pages[g])
            if n:
                self.block_tables[g][slot, :n] = -1
                self.dirty_rows[g].add(slot)
        del self._requests[slot]
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    def _get(self, slot: int) -> _Request:
        try:
            return self._requests[slot]
        except KeyError:
            raise CacheError(f"request slot {slot} is not open") from None

    def is_open(self, slot: int) -> bool:
        return slot in self._requests

    def length(self, slot: int) -> int:
        return self._get(slot).length

    # ------------------------------------------------------------------ pages
    def pages_needed(self, slot: Optional[int], new_length: int) -> Dict[int, int]:
        """Pages each paged group would have to hand out for the request to hold new_length tokens."""
        want = (new_length + self.page_size - 1) // self.page_size
        have = {g: (len(self._requests[slot].pages[g]) if slot is not None else 0) for g in self.paged_ids}
        return {g: max(0, want - have[g]) for g in self.paged_ids}

    def max_reservable(self, slot: int) -> int:
        """The largest length ``reserve`` would accept for the request now (every group asked)."""
        req = self._get(slot)
        most = self.max_model_len
        for g in self.paged_ids:
            most = min(most, (len(req.pages[g]) + self.allocators[g].num_free) * self.page_size)
        return most

    def can_ever_hold(self, length: int, step_tokens: int = 1) -> bool:
        """Whether a request of ``length`` tokens fits the pools when it is alone (growing by
        ``step_tokens`` a step at most)."""
        if length > self.max_model_len:
            return False
        return all(self.groups[g].pages_a_request_needs(length, self.page_size, step_tokens)
                   <= self.allocators[g].num_pages for g in self.paged_ids)

    def capacity_tokens(self) -> int:
        """Tokens of context the pools hold: what the scheduler's admission estimate is compared with.
        Groups that keep every position set it; if every group has a window, the number of requests
        whose windows fit, times the longest request."""
        full = [self.allocators[g].num_pages * self.page_size for g in self.paged_ids
                if self.groups[g].window is None]
        if full:
            return min(full)
        if not self.paged_ids:
            return self.max_requests * self.max_model_len
        fit = min(self.allocators[g].num_pages //
                  max(1, self.groups[g].pages_a_request_needs(self.max_model_len, self.page_size, 1))
                  for g in self.paged_ids)
        return fit * self.max_model_len

    def can_reserve(self, slot: Optional[int], new_length: int) -> bool:
        if new_length > self.max_model_len:
            return False
        need = self.pages_needed(slot, new_length)
        return all(self.allocators[g].num_free >= n for g, n in need.items())

    def reserve(self, slot: int, new_length: int) -> bool:
        """Make room for positions < new_length in every paged group; all or nothing."""
        req = self._get(slot)
        if new_length > self.max_model_len:
            return False
        need = self.pages_needed(slot, new_length)
        if any(self.allocators[g].num_free < n for g, n in need.items()):
            return False
        for g, n in need.items():
            if n == 0:
                continue
            got = self.allocators[g].alloc(n)
            assert got is not None
            start = len(req.pages[g])
            req.pages[g].extend(got)
            self.block_tables[g][slot, start:start + n] = got
            self.dirty_rows[g].add(slot)
            self.pages_handed_out += n
            for p in got:
                if p in self._ever_used[g]:
                    self.pages_reused += 1
                self._ever_used[g].add(p)
        return True

    def advance(self, slot: int, new_length: int) -> None:
        """The request now holds new_length tokens; pages a window has passed go back."""
        req = self._get(slot)
        if new_length < req.length:
            raise CacheError("a request cannot shrink")
        for g in self.paged_ids:
            if new_length > len(req.pages[g]) * self.page_size:
                raise CacheError(f"slot {slot}: {new_length} tokens were written but pages were reserved for "
                                 f"{len(req.pages[g]) * self.page_size}")
        req.length = new_length
        self.lengths[slot] = new_length
        for g in self.paged_ids:
            w = self.groups[g].window
            if w is None:
                continue
            # the next token sits at position new_length and reads positions > new_length - w
            first_needed = max(0, new_length - w + 1)
            first_live_page = first_needed // self.page_size
            if first_live_page > req.first_live[g]:
                gone = []
                for lp in range(req.first_live[g], min(first_live_page, len(req.pages[g]))):
                    if req.pages[g][lp] >= 0:
                        gone.append(req.pages[g][lp])
                        req.pages[g][lp] = -1
                        self.block_tables[g][slot, lp] = -1
                if gone:
                    self.allocators[g].free(gone)
                    self.dirty_rows[g].add(slot)
                req.first_live[g] = min(first_live_page, len(req.pages[g]))

    def slot_of_position(self, group: int, slot: int, position: int) -> int:
        """Physical token slot (page * page_size + offset) of a position of a request."""
        page = self._requests[slot].pages[group][position // self.page_size]
        if page < 0:
            raise CacheError(f"position {position} of slot {slot} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def pages_of(self, group: int, slot: int) -> List[int]:
        return list(self._get(slot).pages[group])

    def num_free_pages(self, group: Optional[int] = None) -> int:
        if group is None:
            return min(a.num_free for a in self.allocators.values()) if self.allocators else 0
        return self.allocators[group].num_free

    def total_pages(self, group: Optional[int] = None) -> int:
        if group is None:
            return min(a.num_pages for a in self.allocators.values()) if self.allocators else 0
        return self.allocators[group].num_pages

    def take_dirty_rows(self, group: int) -> List[int]:
        rows = sorted(self.dirty_rows[group])
        self.dirty_rows[group].clear()
        return rows

    def take_opened_slots(self) -> List[int]:
        s, self.opened_slots = self.opened_slots, []
        return s

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, none held twice, block tables equal to the per-request lists."""
        for g in self.paged_ids:
            alloc = self.allocators[g]
            seen: Set[int] = set()
            for slot, req in self._requests.items():
                for lp, p in enumerate(req.pages[g]):
                    if self.block_tables[g][slot, lp] != p:
                        raise CacheError(f"group {g} slot {slot}: block table differs from the page list")
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheError(f"group {g}: page {p} is held twice")
                    seen.add(p)
            if seen != alloc.held():
                raise CacheError(f"group {g}: held pages {sorted(alloc.held())} differ from the requests' {sorted(seen)}")
            if len(seen) + alloc.num_free != alloc.num_pages:
                raise CacheError(f"group {g}: {alloc.num_pages - len(seen) - alloc.num_free} pages are lost")
            if len(set(alloc._free)) != len(alloc._free):
                raise CacheError(f"group {g}: a page is on the free stack twice")
            for slot in range(self.max_requests):
                if slot not in self._requests and (self.block_tables[g][slot] != -1).any():
                    raise CacheError(f"group {g}: closed slot {slot} still has block-table entries")
        if len(self._free_slots) + len(self._requests) != self.max_requests:
            raise CacheError("a request slot is lost")
