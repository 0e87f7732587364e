"""The cache manager: keys and values in pages with a block table per request, one pool
and one set of tables per GROUP of layers with the same need (all keys / a window of
them), and slots for fixed-size per-request state.

What is held when:
  * `reserve(request, new_len)` makes sure every group has pages for tokens up to new_len;
    it either gets all of them or changes nothing and returns False (the scheduler decides
    what to do then).
  * `commit(request, new_len)` records the new length after a step ran, and gives back the
    pages of windowed groups that no later query can reach: a query at position p reads keys
    >= p - W + 1, so once the request holds n tokens, blocks that end at or before n - W + 1
    are dead.
  * `release(request)` gives back everything the request holds, pages and state slot.
Freed pages are not cleared; a key is valid because of the request's length, not because of
what the page holds.

The reference's cache is one [B, NKV, capacity, D] allocation per layer with a position
per row (include/microllm/inference/kv_cache.h:14-145), zero-filled when a row is released
(src/inference/kv_cache.cpp:11-29); its nearest thing to groups is a per-layer dtype
(kv_cache.h:38-55).  Nothing of that layout is kept.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional

import torch

from ..parts.base import FixedStateNeed, PagedKVNeed, PagedKVView, StateView
from .pages import PageError, PagePool, SlotPool

RELEASED = -1      # block-table entry of a block that was given back (or never existed)
GUARD_VALUE = -24576.0     # exact in bf16 and fp32; what a guard page holds


def group_key(need: PagedKVNeed) -> str:
    return "full" if need.window is None else f"window{int(need.window)}"


@dataclass
class _Request:
    length: int = 0
    tables: Dict[str, List[int]] = field(default_factory=dict)     # group -> physical page per block
    slot: Optional[int] = None


class CacheGroup:
    def __init__(self, key: str, window: Optional[int], num_pages: int):
        self.key, self.window = key, window
        self.pool = PagePool(num_pages)


class CacheManager:
    def __init__(self, entries: Dict[str, object], page_size: int, num_pages: int, max_requests: int,
                 device: Optional[torch.device] = None, kv_dtype: torch.dtype = torch.float32,
                 max_step_tokens: Optional[int] = None, guard_pages: bool = False):
        """entries: cache name -> PagedKVNeed | FixedStateNeed (from parts.Model.cache_entries).
        num_pages: pages of a group that keeps all keys.  device None: books only, no storage (for host tests).
        max_step_tokens: the most tokens one request brings in a step, when the caller promises one: a group
        with a window of W keys then never holds more than W - 1 + max_step_tokens tokens of a request, and its
        pool (and storage) is sized for max_requests such spans instead of for num_pages.
        guard_pages: a debugging aid.  Every paged entry's storage gets one more page in front and one behind,
        filled with a fixed pattern that no kernel may touch; check_guards() reads them back.  A store that runs off
        either end of the pool (a page index of -1 or num_pages that slipped through a kernel's checks) shows there."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.num_pages, self.max_requests = int(page_size), int(num_pages), int(max_requests)
        self.device, self.kv_dtype = device, kv_dtype
        self.groups: Dict[str, CacheGroup] = {}
        self.entry_group: Dict[str, str] = {}
        self.kv_storage: Dict[str, torch.Tensor] = {}
        self.state_storage: Dict[str, torch.Tensor] = {}
        self.state_needs: Dict[str, FixedStateNeed] = {}
        self.guarded: Dict[str, torch.Tensor] = {}       # entry -> the whole allocation, guards included
        for name, need in entries.items():
            need = getattr(need, "need", need)
            if isinstance(need, PagedKVNeed):
                key = group_key(need)
                if key not in self.groups:
                    self.groups[key] = CacheGroup(key, need.window, self.pages_for_group(need.window, max_step_tokens))
                self.entry_group[name] = key
                if device is not None:
                    pages = self.groups[key].pool.num_pages + 1        # the pool's pages, then the spare page (see pad_page)
                    whole = torch.zeros((pages + (2 if guard_pages else 0), 2, need.num_kv_heads, page_size, need.head_dim),
                                        dtype=need.dtype or kv_dtype, device=device)
                    if guard_pages:
                        whole[0].fill_(GUARD_VALUE)
                        whole[-1].fill_(GUARD_VALUE)
                        self.guarded[name] = whole
                        whole = whole[1:-1]                 # contiguous: the pool begins one page into the allocation
                    self.kv_storage[name] = whole
            elif isinstance(need, FixedStateNeed):
                self.state_needs[name] = need
                if device is not None:
                    self.state_storage[name] = torch.zeros((max_requests + 1, *need.shape), dtype=need.dtype, device=device)
            else:
                raise TypeError(f"cache entry {name!r} has an unknown need {need!r}")
        self.slots = SlotPool(max_requests)
        # One page behind every pool and one state slot behind the requests' slots belong to nobody: rows that
        # only fill a batch of fixed size up (a captured decode step run for fewer requests than it was
        # captured for) store their key and keep their state there.  What they hold is never read for a request.
        self.pad_page: Dict[str, int] = {k: g.pool.num_pages for k, g in self.groups.items()}
        self.pad_slot = max_requests
        self.requests: Dict[Hashable, _Request] = {}
        self.pages_released_by_window = 0
        self.tables_version = 0          # grows whenever any block table changes: lets a reader skip a comparison

    def pages_for_group(self, window: Optional[int], max_step_tokens: Optional[int]) -> int:
        """Pages of a group's pool: num_pages for all keys; for a window, what max_requests requests can hold at
        most while each keeps W - 1 old keys and brings up to max_step_tokens new ones (one more block for a span
        that does not start on a block's edge) -- never more than num_pages."""
        if window is None or not max_step_tokens:
            return self.num_pages
        span_blocks = self.blocks_for(int(window) - 1 + int(max_step_tokens)) + 1
        return max(1, min(self.num_pages, self.max_requests * span_blocks))

    # ----- requests -------------------------------------------------------------------------
    def add(self, request: Hashable) -> bool:
        """Start tracking a request: takes a state slot.  False when no slot is free."""
        if request in self.requests:
            raise KeyError(f"request {request!r} is already live")
        slot = self.slots.alloc()
        if slot is None:
            return False
        self.requests[request] = _Request(0, {k: [] for k in self.groups}, slot)
        self.tables_version += 1
        return True

    def has(self, request: Hashable) -> bool:
        return request in self.requests

    def length(self, request: Hashable) -> int:
        return self.requests[request].length

    def slot(self, request: Hashable) -> int:
        return self.requests[request].slot

    def blocks_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, request: Hashable, new_len: int) -> Dict[str, int]:
        r = self.requests[request]
        want = self.blocks_for(new_len)
        return {k: max(0, want - len(t)) for k, t in r.tables.items()}

    def reserve(self, request: Hashable, new_len: int) -> bool:
        """Pages for tokens [length, new_len) in every group, all or nothing."""
        r = self.requests[request]
        if new_len < r.length:
            raise ValueError("a request cannot shrink")
        want = (new_len + self.page_size - 1) // self.page_size
        for table in r.tables.values():
            if len(table) < want:
                break
        else:
            return True                                   # the usual decode step: the last page still has room
        needed = self.pages_needed(request, new_len)
        if any(n > self.groups[k].pool.free_count for k, n in needed.items()):
            return False
        for k, n in needed.items():
            for _ in range(n):
                page = self.groups[k].pool.alloc()
                if page is None:                                   # cannot happen after the check above
                    raise PageError("pool ran dry inside a checked reservation")
                r.tables[k].append(page)
                self.tables_version += 1
        return True

    def commit(self, request: Hashable, new_len: int) -> None:
        r = self.requests[request]
        if new_len < r.length:
            raise ValueError("a request cannot shrink")
        if self.blocks_for(new_len) > min((len(t) for t in r.tables.values()), default=self.blocks_for(new_len)):
            raise PageError(f"request {request!r} commits {new_len} tokens without pages for them")
        r.length = new_len
        for k, table in r.tables.items():
            window = self.groups[k].window
            if window is None:
                continue
            first_needed = new_len - window + 1          # the next query, at position new_len, reads from here
            dead_blocks = max(0, first_needed) // self.page_size     # blocks wholly before first_needed
            for b in range(min(dead_blocks, len(table))):
                if table[b] != RELEASED:
                    self.groups[k].pool.free(table[b])
                    table[b] = RELEASED
                    self.pages_released_by_window += 1
                    self.tables_version += 1

    def release(self, request: Hashable) -> None:
        r = self.requests.pop(request)
        self.tables_version += 1
        for k, table in r.tables.items():
            for page in table:
                if page != RELEASED:
                    self.groups[k].pool.free(page)
        if r.slot is not None:
            self.slots.free(r.slot)

    # ----- what a step needs ---------------------------------------------------------------
    def block_table(self, group: str, requests: List[Hashable], width: Optional[int] = None) -> List[List[int]]:
        rows = [self.requests[q].tables[group] for q in requests]
        width = width if width is not None else max([len(t) for t in rows] + [1])
        if any(len(t) > width for t in rows):
            raise ValueError("block table wider than asked for")
        return [t + [RELEASED] * (width - len(t)) for t in rows]

    def view(self, name: str, block_table: Optional[torch.Tensor], slots: Optional[torch.Tensor],
             slots_host: Optional[List[int]] = None):
        """The view a mixer gets of cache entry `name` for one step."""
        if name in self.entry_group:
            return PagedKVView(self.kv_storage[name], block_table, self.page_size, True)
        return StateView(self.state_storage[name], slots, list(slots_host or []), True)

    # ----- accounting and self-check -------------------------------------------------------
    def stats(self) -> Dict[str, object]:
        out = {"page_size": self.page_size, "live_requests": len(self.requests),
               "pages_released_by_window": self.pages_released_by_window}
        for k, g in self.groups.items():
            out[k] = {"pages": g.pool.num_pages, "used": g.pool.used_count, "peak": g.pool.peak_used,
                      "allocations": g.pool.total_allocations}
        return out

    def kv_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv_storage.values())

    def check_guards(self) -> None:
        """With guard_pages: the page in front of and the page behind every pool still hold their pattern."""
        for name, whole in self.guarded.items():
            for where, page in (("in front of", whole[0]), ("behind", whole[-1])):
                wrong = int((page != GUARD_VALUE).sum().item())
                if wrong:
                    raise PageError(f"cache entry {name!r}: {wrong} elements of the guard page {where} the pool were overwritten")

    def check(self) -> None:
        """No page lost, none held twice, books and pools agree."""
        for k, g in self.groups.items():
            g.pool.check()
            seen: Dict[int, Hashable] = {}
            for q, r in self.requests.items():
                for page in r.tables[k]:
                    if page == RELEASED:
                        continue
                    if page in seen:
                        raise PageError(f"group {k}: page {page} is held by {seen[page]!r} and {q!r}")
                    seen[page] = q
            if set(seen) != g.pool._held:
                raise PageError(f"group {k}: tables hold {sorted(seen)} but the pool says {sorted(g.pool._held)}")
        self.slots.check()
        slots = [r.slot for r in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) != self.slots._held:
            raise PageError("state slots and requests disagree")
