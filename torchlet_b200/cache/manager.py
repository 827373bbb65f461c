"""The cache manager: pages of keys and values with a block table for each request,
and slots for per-request state of fixed size.

Page bookkeeping follows the reference's allocator (v10_triton_paged_gqa/kvcache.py:
37-66: a free list with page 0 reserved as a harmless target of empty table entries,
a list of pages for each request in logical order, all-or-nothing growth) and its
decode slots (v05_decode_slots/scheduler.py:38-71: a stable index per live request).
Added here: GROUPS of layer executions with different needs.  A group is a set of
executions whose mixers keep the same kind of history (same KV heads, head size and
window); it has its own pool of pages and its own table per request.  A group with a
window gives a page back as soon as every position in it has left the window of the
request's next token; the table entry then points at page 0 and is never read.

This module is host-only bookkeeping (no device memory) so that it can be tested
without a GPU; ``torchlet_b200.cache.storage`` owns the device tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Optional

import numpy as np

NULL_PAGE = 0


class CacheError(RuntimeError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    """One group of layer executions that share pages."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int]  # None: every key is kept
    entries: tuple  # schedule entries that own a cache layer in this group
    num_pages: int  # pool size, page 0 included


class PagePool:
    """Free list over pages 1 .. num_pages-1 (page 0 is reserved)."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise ValueError("a pool needs at least 2 pages (page 0 is reserved)")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, 0, -1))  # pop() hands out 1, 2, ...
        self._held = [False] * num_pages
        self.peak_held = 0  # the most pages that were ever held at once (the pool's high-water mark)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, count: int) -> list[int]:
        if count > len(self._free):
            raise CacheError(f"asked for {count} pages, {len(self._free)} free")
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            self._held[page] = True
        self.peak_held = max(self.peak_held, self.num_pages - 1 - len(self._free))
        return pages

    def give_back(self, pages) -> None:
        for page in pages:
            if page == NULL_PAGE:
                continue
            if not (0 < page < self.num_pages) or not self._held[page]:
                raise CacheError(f"page {page} is given back but not held")
            self._held[page] = False
            self._free.append(page)


@dataclass
class _RequestPages:
    slot: int
    num_tokens: int = 0  # tokens whose keys and values are in pages (steps done so far)
    tables: list = field(default_factory=list)  # per group: logical page -> physical page
    first_live: list = field(default_factory=list)  # per group: first logical page still held
    capacity: int = 0  # tokens that fit the pages reserved so far, at most the length limit


class CacheManager:
    """Pages per group, block tables per request, and slots."""

    def __init__(self, groups: list[GroupSpec], page_size: int, max_slots: int, max_seq_len: int):
        if page_size <= 0 or max_slots <= 0:
            raise ValueError("page_size and max_slots must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_seq_len = max_seq_len
        self.max_pages_per_request = -(-max_seq_len // page_size)
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        # per group: the block tables of all slots as one int32 array [max_slots, pages per
        # request], kept equal to the per-request lists so that a step gathers rows at once
        self.table_arrays = [np.zeros((max_slots, self.max_pages_per_request), dtype=np.int32) for _ in self.groups]
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._requests: dict[Hashable, _RequestPages] = {}

    # ----------------------------------------------------------------- slots
    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def has(self, request_id: Hashable) -> bool:
        return request_id in self._requests

    def live_requests(self) -> list:
        return list(self._requests)

    def admit(self, request_id: Hashable) -> int:
        """Give the request a slot (and empty tables); returns the slot."""
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise CacheError("no free slot")
        slot = self._free_slots.pop()
        self._requests[request_id] = _RequestPages(
            slot=slot, tables=[[] for _ in self.groups], first_live=[0 for _ in self.groups]
        )
        return slot

    def slot_of(self, request_id: Hashable) -> int:
        return self._requests[request_id].slot

    def num_tokens(self, request_id: Hashable) -> int:
        return self._requests[request_id].num_tokens

    # ----------------------------------------------------------------- pages
    def _pages_needed(self, record: _RequestPages, new_len: int) -> list[int]:
        want = -(-new_len // self.page_size)
        return [max(0, want - len(table)) for table in record.tables]

    def can_extend(self, request_id: Hashable, new_len: int) -> bool:
        record = self._requests[request_id]
        if new_len <= record.capacity:
            return True
        need = self._pages_needed(record, new_len)
        return all(n <= pool.num_free for n, pool in zip(need, self.pools))

    def extend(self, request_id: Hashable, new_len: int) -> bool:
        """Make room for the request's tokens up to ``new_len`` in every group,
        all or nothing.  Returns False (nothing changed) when some pool is short.
        The request's length itself changes only with ``advance``."""
        if new_len > self.max_seq_len:
            raise CacheError(f"request {request_id!r} would hold {new_len} tokens, the limit is {self.max_seq_len}")
        record = self._requests[request_id]
        if new_len <= record.capacity:
            return True
        need = self._pages_needed(record, new_len)
        if any(n > pool.num_free for n, pool in zip(need, self.pools)):
            return False
        for g, (table, n, pool) in enumerate(zip(record.tables, need, self.pools)):
            if n:
                start = len(table)
                table.extend(pool.take(n))
                self.table_arrays[g][record.slot, start:start + n] = table[start:]
        # a model without any paged group (every mixer keeps fixed-size state only) is bounded
        # by the length limit alone
        pages = min((len(table) for table in record.tables), default=self.max_pages_per_request)
        record.capacity = min(pages * self.page_size, self.max_seq_len)
        return True

    def begin_decode(self, request_ids) -> tuple:
        """One more token for each request of a decode step, in one pass: makes room for it
        and returns (lengths so far, slots) as int32 arrays, or the index of the first
        request that gets no page (the requests before it keep what they reserved)."""
        n = len(request_ids)
        before = np.empty(n, dtype=np.int32)
        slots = np.empty(n, dtype=np.int32)
        requests = self._requests
        for i, request_id in enumerate(request_ids):
            record = requests[request_id]
            length = record.num_tokens
            before[i] = length
            slots[i] = record.slot
            if length + 1 > record.capacity and not self.extend(request_id, length + 1):
                return i
        return before, slots

    def end_decode(self, request_ids) -> None:
        """The step wrote one more token of each request (``advance`` by one, in one pass)."""
        windowed = any(group.window is not None for group in self.groups)
        requests = self._requests
        for request_id in request_ids:
            record = requests[request_id]
            if windowed or record.num_tokens + 1 > record.capacity:
                self.advance(request_id, record.num_tokens + 1)
            else:
                record.num_tokens += 1

    def advance(self, request_id: Hashable, new_len: int) -> int:
        """After a step wrote the request's tokens up to ``new_len``: record the length
        and give back the pages of windowed groups that the request's next token (at
        position ``new_len``) can no longer see.  Returns how many pages were given back."""
        record = self._requests[request_id]
        if new_len < record.num_tokens:
            raise CacheError("a request's length cannot shrink")
        if any(-(-new_len // self.page_size) > len(table) for table in record.tables):
            raise CacheError(f"request {request_id!r} advanced to {new_len} tokens without pages for them")
        record.num_tokens = new_len
        given = 0
        for g, (group, table, pool) in enumerate(zip(self.groups, record.tables, self.pools)):
            if group.window is None:
                continue
            first_needed_position = record.num_tokens - group.window + 1
            if first_needed_position <= 0:
                continue
            first_needed_page = min(first_needed_position // self.page_size, len(table))
            for logical in range(record.first_live[g], first_needed_page):
                pool.give_back([table[logical]])
                table[logical] = NULL_PAGE
                self.table_arrays[g][record.slot, logical] = NULL_PAGE
                given += 1
            record.first_live[g] = max(record.first_live[g], first_needed_page)
        return given

    def table(self, request_id: Hashable, group: int) -> list[int]:
        return self._requests[request_id].tables[group]

    def finish(self, request_id: Hashable) -> int:
        """Give back everything the request holds; returns its slot (now free)."""
        record = self._requests.pop(request_id)
        for g, (table, pool) in enumerate(zip(record.tables, self.pools)):
            pool.give_back(table)
            self.table_arrays[g][record.slot, :len(table)] = NULL_PAGE
        self._free_slots.append(record.slot)
        return record.slot

    def reset(self) -> None:
        for request_id in list(self._requests):
            self.finish(request_id)

    # ------------------------------------------------------------- invariants
    def check(self) -> None:
        """No page lost, held twice or free and held at once; no slot lost or shared."""
        for g, pool in enumerate(self.pools):
            held = []
            for record in self._requests.values():
                held += [p for p in record.tables[g] if p != NULL_PAGE]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page is held twice")
            free = list(pool._free)
            if len(free) != len(set(free)):
                raise CacheError(f"group {g}: a page is free twice")
            if set(free) & set(held):
                raise CacheError(f"group {g}: a page is both free and held")
            if len(free) + len(held) != pool.num_pages - 1:
                raise CacheError(f"group {g}: {pool.num_pages - 1 - len(free) - len(held)} pages lost")
            if NULL_PAGE in free:
                raise CacheError(f"group {g}: page 0 is in the free list")
            for record in self._requests.values():
                row = self.table_arrays[g][record.slot]
                if row[:len(record.tables[g])].tolist() != record.tables[g] or row[len(record.tables[g]):].any():
                    raise CacheError(f"group {g}: the table array differs from the table of slot {record.slot}")
        slots = [r.slot for r in self._requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots):
            raise CacheError("a slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_slots:
            raise CacheError("a slot is lost")
