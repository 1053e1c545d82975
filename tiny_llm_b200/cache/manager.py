"""Cache manager: keys and values in pages with a block table per request, one page pool per group
of layers with the same need, and slots for per-request state of fixed size.

What the reference has: one pool per layer, a block table per layer rebuilt and uploaded every
step, all pages of a request returned together when generation ends
(tiny_llm/runtime/cuda/cuda_runtime.cpp:505-526, 667-819), and a note that groups are still to come
(cuda_runtime.hpp:70).  Here one page id addresses the page in every cache entry of its group, so a
request has one block table per group, whatever the number of layers.

Groups.  A mixer declares its need (`KVNeed`: heads, head size, optional window; `StateNeed`: a
fixed shape per request).  Calls with the same KVNeed form one group with its own pool, sized for
the same number of tokens.  A group with a window gives a page back as soon as every position in it
lies before the window of the request's next token; its block-table entry becomes -1 and the
attention kernels never look there.

A request moves through reserve(n) -> (the step runs) -> commit(n).  `reserve` takes the pages the
next n tokens need in every group, or nothing at all."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Tuple

import torch

from .pages import PageError, PagePool


@dataclass(frozen=True)
class KVNeed:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: all keys; n: the last n keys (the token itself included)


@dataclass(frozen=True)
class StateNeed:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheEntryRef:
    """Where one layer call finds its cache: a KV entry of a group, or a state tensor."""
    group: Optional[int] = None
    entry: Optional[int] = None
    state: Optional[int] = None


class KVGroup:
    """All cache entries that share one KVNeed: one pool, one block table per request, and the
    tensor kv[entry, 0 = keys | 1 = values, page, kv_head, slot_in_page, head_dim]."""

    def __init__(self, need: KVNeed, num_entries: int, num_pages: int, page_size: int):
        self.need = need
        self.num_entries = num_entries
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.tables: Dict[Hashable, List[int]] = {}
        self.kv: Optional[torch.Tensor] = None

    def allocate_storage(self, dtype: torch.dtype, device) -> None:
        n = self.need
        self.kv = torch.zeros(self.num_entries, 2, self.pool.num_pages, n.num_kv_heads, self.page_size,
                              n.head_dim, dtype=dtype, device=device)

    def bytes_per_token(self, itemsize: int) -> int:
        return 2 * self.num_entries * self.need.num_kv_heads * self.need.head_dim * itemsize

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def first_needed_page(self, next_pos: int) -> int:
        """Index of the first page that the token at `next_pos` can still see."""
        if self.need.window is None:
            return 0
        lowest_visible = max(0, next_pos - self.need.window + 1)
        return lowest_visible // self.page_size


class StateSlots:
    """Per-request state of fixed size: `tensors[i][slot]` belongs to the request that holds `slot`.
    A slot is zeroed when it is handed out."""

    def __init__(self, max_slots: int):
        self.max_slots = max_slots
        self._free = list(range(max_slots - 1, -1, -1))
        self._slot_of: Dict[Hashable, int] = {}
        self.needs: List[StateNeed] = []
        self.tensors: List[torch.Tensor] = []

    def register(self, need: StateNeed) -> int:
        self.needs.append(need)
        return len(self.needs) - 1

    def allocate_storage(self, device) -> None:
        self.tensors = [torch.zeros((self.max_slots,) + tuple(n.shape), dtype=n.dtype, device=device)
                        for n in self.needs]

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, rid: Hashable) -> Optional[int]:
        if rid in self._slot_of:
            raise PageError(f"request {rid!r} already holds slot {self._slot_of[rid]}")
        if not self._free:
            return None
        s = self._free.pop()
        self._slot_of[rid] = s
        for t in self.tensors:
            t[s].zero_()
        return s

    def release(self, rid: Hashable) -> None:
        if rid not in self._slot_of:
            raise PageError(f"request {rid!r} holds no slot")
        self._free.append(self._slot_of.pop(rid))

    def slot_of(self, rid: Hashable) -> int:
        return self._slot_of[rid]

    def check(self) -> None:
        held = list(self._slot_of.values())
        if len(set(held)) != len(held) or set(held) & set(self._free) or \
                len(held) + len(self._free) != self.max_slots or len(set(self._free)) != len(self._free):
            raise PageError("slot bookkeeping is inconsistent")


class CacheManager:
    def __init__(self, needs: List[Optional[object]], max_tokens: int, page_size: int, max_slots: int):
        """`needs[i]` is the need of cache entry i (one per layer call that owns a cache): a KVNeed, a
        StateNeed or None.  `max_tokens` is the number of tokens every group's pool can hold."""
        if page_size <= 0 or max_tokens <= 0:
            raise ValueError("page_size and max_tokens must be positive")
        self.page_size = page_size
        self.max_tokens = max_tokens
        self.groups: List[KVGroup] = []
        self.slots = StateSlots(max_slots)
        self.refs: List[CacheEntryRef] = []
        by_need: Dict[KVNeed, int] = {}
        counts: Dict[KVNeed, int] = {}
        for need in needs:
            if isinstance(need, KVNeed):
                counts[need] = counts.get(need, 0) + 1
        num_pages = -(-max_tokens // page_size)
        for need in needs:
            if isinstance(need, KVNeed):
                if need not in by_need:
                    by_need[need] = len(self.groups)
                    self.groups.append(KVGroup(need, counts[need], num_pages, page_size))
                    counts[need] = 0
                g = by_need[need]
                self.refs.append(CacheEntryRef(group=g, entry=counts[need]))
                counts[need] += 1
            elif isinstance(need, StateNeed):
                self.refs.append(CacheEntryRef(state=self.slots.register(need)))
            elif need is None:
                self.refs.append(CacheEntryRef())
            else:
                raise TypeError(f"unknown cache need {need!r}")
        self.kv_len: Dict[Hashable, int] = {}
        self._reserved: Dict[Hashable, int] = {}
        self.birth: Dict[Hashable, int] = {}   # a number that differs between two lives of the same request id
        self._births = 0

    # ---- storage
    def allocate_storage(self, dtype: torch.dtype, device) -> None:
        for g in self.groups:
            g.allocate_storage(dtype, device)
        self.slots.allocate_storage(device)

    # ---- requests
    def add_request(self, rid: Hashable) -> Optional[int]:
        """Gives the request a state slot and empty block tables; None if no slot is free."""
        if rid in self.kv_len:
            raise PageError(f"request {rid!r} is already live")
        slot = self.slots.acquire(rid)
        if slot is None:
            return None
        self.kv_len[rid] = 0
        self._reserved[rid] = 0
        self._births += 1
        self.birth[rid] = self._births
        for g in self.groups:
            g.tables[rid] = []
        return slot

    def has_request(self, rid: Hashable) -> bool:
        return rid in self.kv_len

    def pages_missing(self, rid: Hashable, n_new: int) -> List[int]:
        """Pages each group still lacks for the request's next n_new tokens."""
        total = self.kv_len[rid] + n_new
        return [max(0, g.pages_for(total) - len(g.tables[rid])) for g in self.groups]

    def can_reserve(self, rid: Hashable, n_new: int) -> bool:
        return all(m <= g.pool.num_free for m, g in zip(self.pages_missing(rid, n_new), self.groups))

    def reserve(self, rid: Hashable, n_new: int) -> bool:
        """Takes the pages for the next n_new tokens in every group, or none at all."""
        if n_new <= 0:
            raise ValueError("reserve needs a positive token count")
        missing = self.pages_missing(rid, n_new)
        if any(missing):
            if any(m > g.pool.num_free for m, g in zip(missing, self.groups)):
                return False
            for m, g in zip(missing, self.groups):
                if m:
                    got = g.pool.allocate(m, rid)
                    assert got is not None
                    g.tables[rid].extend(got)
        if n_new > self._reserved[rid]:
            self._reserved[rid] = n_new
        return True

    def commit(self, rid: Hashable, n_new: int) -> None:
        """The step wrote n_new tokens.  Pages that a window has passed go back to their pool."""
        if n_new > self._reserved[rid]:
            raise PageError(f"request {rid!r} commits {n_new} tokens but reserved {self._reserved[rid]}")
        self._reserved[rid] = 0
        self.kv_len[rid] += n_new
        for g in self.groups:
            if g.need.window is None:
                continue
            table = g.tables[rid]
            first = min(g.first_needed_page(self.kv_len[rid]), len(table))
            gone = [p for p in table[:first] if p >= 0]
            if gone:
                g.pool.free(gone, rid)
                for i in range(first):
                    table[i] = -1

    def free_request(self, rid: Hashable) -> None:
        """The request has ended (or is pushed out): everything it holds goes back."""
        if rid not in self.kv_len:
            raise PageError(f"request {rid!r} is not live")
        for g in self.groups:
            held = [p for p in g.tables.pop(rid) if p >= 0]
            g.pool.free(held, rid)
        self.slots.release(rid)
        del self.kv_len[rid]
        del self._reserved[rid]
        del self.birth[rid]

    # ---- views for the step
    def block_table(self, group: int, rid: Hashable) -> List[int]:
        return self.groups[group].tables[rid]

    def slot_of(self, rid: Hashable) -> int:
        return self.slots.slot_of(rid)

    def live_requests(self):
        return list(self.kv_len)

    def check(self) -> None:
        """No page lost, held twice or freed twice; every table entry is owned by its request."""
        for g in self.groups:
            g.pool.check()
            seen = set()
            for rid, table in g.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise PageError(f"page {p} is in two block tables")
                    seen.add(p)
                    if g.pool.owner_of(p) != rid:
                        raise PageError(f"page {p} in the table of {rid!r} is owned by {g.pool.owner_of(p)!r}")
            if len(seen) != g.pool.num_used:
                raise PageError("a page is owned but in no block table")
        self.slots.check()
