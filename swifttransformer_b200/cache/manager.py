"""The cache manager: paged keys/values with block tables, and slots of
fixed-size per-request state.

Cache entries (one per layer step that writes a cache) are sorted into groups
by what they need: entries with the same PagedKVSpec (heads, head size,
window) share one pool of pages and one block table; each group has pages of
its own.  A page of a group holds ``page_size`` positions of every entry of
the group:

    kv[page][entry][0=K,1=V][kv_head][position in page][head_dim]

Pages are handed out when a step is about to write positions that have none,
and given back when the request ends, and - in a group with a window - as soon
as the window has moved past them.  Entries with a StateSpec get a tensor
``[max_seqs, *shape]``; a request's row is zeroed when the request gets its slot.

A request is known here by its slot (0..max_seqs-1), which is also its row in
every block table.  Everything in this file is host bookkeeping plus tensor
allocation; block-table changes are queued as (flat index, value) pairs which
the step function copies to the device together with the step's other
metadata.

Reference, for comparison: k_cache / v_cache [num_blocks, layers, heads,
block_size, head_dim] owned by the caller (src/csrc/model/gpt/gpt.cc:229-230),
block table int64 [batch, max_blocks] rebuilt per call
(src/csrc/model/gpt/gptop_base.cc:57-67), allocation by a counter that never
frees (src/examples/lib/inference_batch.cc:58-66).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import PagedKVSpec, StateSpec
from .pages import PagePool


@dataclasses.dataclass
class PagedCacheView:
    pool: torch.Tensor          # [pages, entries, 2, kv_heads, page_size, head_dim]
    layer: int                  # index of this entry inside the group
    block_table: torch.Tensor   # int32 [max_seqs, max_pages_per_seq]
    page_size: int
    writable: bool = True


@dataclasses.dataclass
class StateView:
    state: torch.Tensor         # [max_seqs, *shape]
    writable: bool = True


class _Entry:
    """What a layer step gets: ``view(writable)``."""

    def __init__(self, make):
        self._make = make
        self._views = {}

    def view(self, writable: bool = True):
        if writable not in self._views:
            self._views[writable] = self._make(writable)
        return self._views[writable]


class PagedGroup:
    def __init__(self, spec: PagedKVSpec, entries: List[int], page_size: int, num_pages: int, max_seqs: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device: torch.device):
        self.spec, self.entries, self.page_size = spec, entries, page_size
        self.max_pages_per_seq = max_pages_per_seq
        self.pool = PagePool(num_pages)
        self.kv = torch.zeros((num_pages, len(entries), 2, spec.num_kv_heads, page_size, spec.head_dim),
                              dtype=dtype, device=device)
        self.block_table = torch.full((max_seqs, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        # per slot: logical page index -> page id, and the first logical page still held
        self.pages: List[Dict[int, int]] = [dict() for _ in range(max_seqs)]
        # flat index into block_table -> newest value (one entry per index: the device applies them in parallel)
        self.updates: Dict[int, int] = {}

    @property
    def bytes_per_token(self) -> int:
        return len(self.entries) * 2 * self.spec.num_kv_heads * self.spec.head_dim * self.kv.element_size()

    def _first_needed_page(self, start: int) -> int:
        """Lowest logical page that queries at positions >= start can read."""
        if self.spec.window is None:
            return 0
        return max(0, start - self.spec.window + 1) // self.page_size

    def peak_pages(self, end: int, portion: int) -> int:
        """The most pages a request holds at any time while it is brought to ``end`` tokens in portions of at
        most ``portion``: all of them, or what a window and one portion span."""
        total = (end + self.page_size - 1) // self.page_size
        if self.spec.window is None:
            return total
        return min(total, (self.spec.window - 1 + portion + self.page_size - 1) // self.page_size + 1)

    def missing(self, slot: int, start: int, end: int) -> List[int]:
        """Logical pages that positions start..end-1 need and the slot does not hold."""
        if end <= start:
            return []
        held = self.pages[slot]
        last = (end - 1) // self.page_size
        if last >= self.max_pages_per_seq:
            raise ValueError(f"a request of {end} tokens needs more than {self.max_pages_per_seq} pages")
        return [j for j in range(self._first_needed_page(start), last + 1) if j not in held]

    def reserve(self, slot: int, start: int, end: int) -> bool:
        need = self.missing(slot, start, end)
        got = self.pool.alloc(len(need))
        if got is None:
            return False
        for j, p in zip(need, got):
            self.pages[slot][j] = p
            self.updates[slot * self.max_pages_per_seq + j] = p
        return True

    def _release(self, slot: int, logical: Sequence[int]) -> None:
        held = self.pages[slot]
        self.pool.free([held[j] for j in logical])
        for j in logical:
            del held[j]
            self.updates[slot * self.max_pages_per_seq + j] = -1

    def trim(self, slot: int, length: int) -> int:
        """Give back the pages that no query at a position >= length can read (window groups)."""
        if self.spec.window is None:
            return 0
        first = self._first_needed_page(length)
        gone = [j for j in self.pages[slot] if j < first]
        self._release(slot, gone)
        return len(gone)

    def release_all(self, slot: int) -> None:
        self._release(slot, list(self.pages[slot]))

    def take_updates(self) -> List[Tuple[int, int]]:
        u, self.updates = self.updates, {}
        return list(u.items())


class CacheManager:
    def __init__(self, cache_specs: Sequence[Any], dtype: torch.dtype, device, page_size: int,
                 num_pages: int, max_seqs: int, max_seq_len: int):
        """``num_pages`` pages for every paged group; ``max_seq_len`` bounds a block-table row."""
        if page_size <= 0 or max_seqs <= 0:
            raise ValueError("page_size and max_seqs must be positive")
        self.device = torch.device(device)
        self.dtype, self.page_size, self.max_seqs, self.max_seq_len = dtype, page_size, max_seqs, max_seq_len
        self.max_pages_per_seq = (max_seq_len + page_size - 1) // page_size
        self.groups: List[PagedGroup] = []
        self.states: Dict[int, torch.Tensor] = {}
        self._entries: List[Optional[_Entry]] = [None] * len(cache_specs)
        by_spec: Dict[PagedKVSpec, List[int]] = {}
        for i, spec in enumerate(cache_specs):
            if isinstance(spec, PagedKVSpec):
                by_spec.setdefault(spec, []).append(i)
            elif isinstance(spec, StateSpec):
                t = torch.zeros((max_seqs,) + tuple(spec.shape), dtype=spec.dtype, device=self.device)
                self.states[i] = t
                self._entries[i] = _Entry(lambda w, t=t: StateView(t, w))
            elif spec is None:
                self._entries[i] = _Entry(lambda w: None)
            else:
                raise TypeError(f"cache entry {i}: unknown cache spec {spec!r}")
        for spec, entries in by_spec.items():
            g = PagedGroup(spec, entries, page_size, num_pages, max_seqs, self.max_pages_per_seq, dtype, self.device)
            self.groups.append(g)
            for k, i in enumerate(entries):
                self._entries[i] = _Entry(
                    lambda w, g=g, k=k: PagedCacheView(g.kv, k, g.block_table, page_size, w))
        self._free_slots = list(range(max_seqs - 1, -1, -1))
        self._live = [False] * max_seqs
        self.lengths = [0] * max_seqs

    # ------------------------------------------------------------------ slots
    def entries(self) -> List[_Entry]:
        return list(self._entries)

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def alloc_slot(self) -> Optional[int]:
        if not self._free_slots:
            return None
        s = self._free_slots.pop()
        self._live[s] = True
        self.lengths[s] = 0
        for t in self.states.values():
            t[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        if not self._live[slot]:
            raise RuntimeError(f"slot {slot} is not live (freed twice?)")
        for g in self.groups:
            g.release_all(slot)
        self._live[slot] = False
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    # ------------------------------------------------------------------ pages
    def pages_missing(self, slot: int, start: int, end: int) -> int:
        """How many pages (summed over groups) positions start..end-1 still need."""
        return sum(len(g.missing(slot, start, end)) for g in self.groups)

    def pages_to_come(self, slot: Optional[int], end: int, portion: int) -> List[int]:
        """Per group: the pages a request will still ask for until it holds ``end`` tokens, beyond those its
        slot holds now (slot None: a request that holds nothing yet)."""
        return [max(0, g.peak_pages(end, portion) - (len(g.pages[slot]) if slot is not None else 0))
                for g in self.groups]

    def can_reserve(self, slot: int, start: int, end: int) -> bool:
        return all(len(g.missing(slot, start, end)) <= g.pool.num_free for g in self.groups)

    def reserve(self, slot: int, start: int, end: int) -> bool:
        """Pages for positions start..end-1 in every group, or nothing at all."""
        if not self._live[slot]:
            raise RuntimeError(f"slot {slot} is not live")
        if end > self.max_seq_len:
            raise ValueError(f"{end} tokens exceed the cache's per-request limit of {self.max_seq_len}")
        if not self.can_reserve(slot, start, end):
            return False
        for g in self.groups:
            ok = g.reserve(slot, start, end)
            assert ok
        return True

    def commit(self, slot: int, length: int) -> None:
        """The request now holds ``length`` tokens: drop what a window has passed."""
        self.lengths[slot] = length
        for g in self.groups:
            g.trim(slot, length)

    @property
    def free_pages(self) -> int:
        return min((g.pool.num_free for g in self.groups), default=0)

    @property
    def total_pages(self) -> int:
        return min((g.pool.num_pages for g in self.groups), default=0)

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token for g in self.groups)

    def check(self) -> None:
        """Invariants: no page lost, none held twice."""
        for g in self.groups:
            g.pool.check()
            held = [p for d in g.pages for p in d.values()]
            if len(held) != len(set(held)):
                raise RuntimeError("a page is held by two requests")
            if len(held) != g.pool.num_held:
                raise RuntimeError("a page is held but belongs to no request (lost)")
            for s, d in enumerate(g.pages):
                if d and not self._live[s]:
                    raise RuntimeError(f"free slot {s} still holds pages")
