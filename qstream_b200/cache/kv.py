"""The sequence cache: paged keys and values per layer group, per-sequence state.

A *slot* stands for one live sequence: its length, its pages in every group, its row
of every state tensor.  Cache entries (one per schedule run that writes keys and
values) with the same need (heads, head size, window) form a *group* with storage and
a page pool of its own: K and V as [entries][pages][kv_heads][page_tokens][head_dim].
Position p of a slot lies in page `page_table[slot][p // page_tokens]`, row
`p % page_tokens`.  A group with a window gives back the pages that have fallen out of
every future query's window.  Pages are handed out before a step runs and given back
when the sequence ends.  Reads are bounded by the length, with one exception: the
tensor-core prefill attention multiplies the value rows past a sequence's end, in its
last page, by weights of exactly zero, and 0 * Inf is NaN.  So a page that held another
sequence's values is zeroed when it is handed on, unless the step that takes it writes
all of its rows.

This replaces QStream's single-sequence cache (`QSFKVCache`, include/qsf/engine.h:35-51,
src/engine.c:296-327; `current_seq_len`), whose int8 storage is not taken over.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Sequence

import numpy as np
import torch

from ..errors import QsError, QStreamError
from .pages import PagePool, SlotTable

PAGE_TOKENS = 64
CANARY = 0x5EED5EED


@dataclass(frozen=True)
class KvNeed:
    """What a mixer asks of the cache for its keys and values."""
    n_kv_heads: int
    head_dim: int
    window: int = 0                     # 0: all keys; w: the last w


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence: one tensor of `shape` and `dtype` per slot,
    zero when the sequence starts."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class CacheView:
    """What a mixer gets for one cache entry."""
    k: torch.Tensor                     # [pages, kv_heads, page_tokens, head_dim]
    v: torch.Tensor
    page_table: torch.Tensor            # [slots, max_pages] int32, device
    page_tokens: int
    need: KvNeed


class KvGroup:
    def __init__(self, need: KvNeed, entries: Sequence[int], n_pages: int, n_slots: int,
                 max_pages: int, dtype: torch.dtype, device, page_tokens: int = PAGE_TOKENS):
        self.need = need
        self.entries = list(entries)
        self.page_tokens = page_tokens
        self.pool = PagePool(n_pages)
        self.max_pages = max_pages
        # one page more than the pool hands out: every entry's last page holds guard words (`check_canaries`)
        shape = (len(self.entries), n_pages + 1, need.n_kv_heads, page_tokens, need.head_dim)
        # Zeroed once here; a page that has been used is zeroed again (values only: scores of keys past
        # the end are replaced, not multiplied) when it is handed on to a step that leaves rows unwritten.
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self._used = np.zeros(n_pages, dtype=bool)
        self._to_zero: list[int] = []
        self.table_host = np.full((n_slots, max_pages), -1, dtype=np.int32)
        self.table_dev = torch.full((n_slots, max_pages), -1, dtype=torch.int32, device=device)
        self._dirty: set[int] = set()
        self.first_page = [0] * n_slots     # pages below this index were given back (window)
        self.held = [0] * n_slots           # pages held from first_page on (they are contiguous)
        self.n_pages = n_pages
        if self.k.is_cuda:
            from ..csrc import ops
            for store in (self.k, self.v):
                for e in range(len(self.entries)):
                    ops.canary_fill(store[e, n_pages], CANARY)

    def damaged_guard_words(self) -> int:
        """How many guard words behind the entries' pages no longer hold their pattern (0 on a host cache)."""
        if not self.k.is_cuda:
            return 0
        from ..csrc import ops
        damaged = torch.zeros(2, dtype=torch.int32, device=self.k.device)
        for store in (self.k, self.v):
            for e in range(len(self.entries)):
                ops.canary_check(store[e, self.n_pages], CANARY, damaged)
        return int(damaged[0].item())

    @property
    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def pages_needed(self, slot: int, new_length: int) -> int:
        return max(0, -(-new_length // self.page_tokens) - self.first_page[slot] - self.held[slot])

    def ensure(self, slot: int, new_length: int) -> None:
        """Pages for positions [0, new_length) of the slot (those not given back)."""
        n = -(-new_length // self.page_tokens)
        have = self.first_page[slot] + self.held[slot]
        if n <= have:
            return
        row = self.table_host[slot]
        for i in range(have, n):
            page = row[i] = self.pool.alloc()
            if self._used[page] and new_length < (i + 1) * self.page_tokens:
                self._to_zero.append(page)          # used before, and this step does not fill it
            self._used[page] = True
        self.held[slot] += n - have
        self._dirty.add(slot)

    def trim(self, slot: int, length: int) -> None:
        """Give back pages that no later query can reach: with a window w the next
        query, at position `length`, reads keys >= length - w + 1."""
        w = self.need.window
        if w <= 0:
            return
        keep_from = max(0, length - w + 1) // self.page_tokens
        if keep_from <= self.first_page[slot]:
            return
        row = self.table_host[slot]
        for i in range(self.first_page[slot], keep_from):
            if row[i] >= 0:
                self.pool.free(int(row[i]))
                row[i] = -1
                self.held[slot] -= 1
                self._dirty.add(slot)
        self.first_page[slot] = keep_from

    def release(self, slot: int) -> None:
        row = self.table_host[slot]
        for i in np.nonzero(row >= 0)[0]:
            self.pool.free(int(row[i]))
        row[:] = -1
        self.first_page[slot] = 0
        self.held[slot] = 0
        self._dirty.add(slot)

    def upload(self) -> None:
        """Bring the device page table up to date (rows that changed); clear handed-on pages."""
        if self._to_zero:
            if self.v.is_cuda:
                from ..csrc import ops
                ids = torch.tensor(self._to_zero, dtype=torch.int32).pin_memory().to(self.v.device, non_blocking=True)
                ops.zero_pages(self.v, ids)
            else:
                self.v[:, self._to_zero] = 0
            self._to_zero.clear()
        if not self._dirty:
            return
        rows = sorted(self._dirty)
        self._dirty.clear()
        if self.table_dev.is_cuda:
            idx = torch.tensor(rows, dtype=torch.int64)
            src = torch.from_numpy(self.table_host[rows]).pin_memory()
            self.table_dev.index_copy_(0, idx.to(self.table_dev.device, non_blocking=True),
                                       src.to(self.table_dev.device, non_blocking=True))
        else:
            self.table_dev[rows] = torch.from_numpy(self.table_host[rows])

    def view(self, cache_id: int) -> CacheView:
        e = self.entries.index(cache_id)
        return CacheView(self.k[e], self.v[e], self.table_dev, self.page_tokens, self.need)


class StateStore:
    """Per-sequence state of fixed size: for each name a tensor [slots, *shape].
    It is there for mixers that carry state from token to token; a model whose
    mixers need none has an empty store."""

    def __init__(self, needs: Mapping[object, StateNeed], n_slots: int, device):
        self.tensors = {key: torch.zeros((n_slots, *need.shape), dtype=need.dtype, device=device)
                        for key, need in needs.items()}

    def reset(self, slot: int) -> None:
        for t in self.tensors.values():
            t[slot].zero_()

    def get(self, key):
        return self.tensors.get(key)

    @property
    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())


class SequenceCache:
    """Slots, page groups and state together; the step function's only door to them.

    kv_needs: cache entry id -> KvNeed (entries of mixers without keys and values are
    absent); state_needs: key -> StateNeed.  `max_tokens` is the number of tokens all
    live sequences may hold together, each sequence rounded up to whole pages.
    """

    def __init__(self, kv_needs: Mapping[int, KvNeed], state_needs: Mapping[object, StateNeed],
                 max_tokens: int, max_slots: int, max_context: int, dtype: torch.dtype, device,
                 page_tokens: int = PAGE_TOKENS):
        if max_tokens < 1 or max_context < 1:
            raise QStreamError(QsError.INVALID_INPUT, f"cache of {max_tokens} tokens, context {max_context}")
        self.page_tokens = page_tokens
        self.max_context = max_context
        self.max_tokens = max_tokens
        n_pages = -(-max_tokens // page_tokens)
        max_slots = max(1, min(max_slots, n_pages))
        self.slots = SlotTable(max_slots)
        max_pages = -(-max_context // page_tokens)
        by_need: dict[KvNeed, list[int]] = {}
        for cid in sorted(kv_needs):
            by_need.setdefault(kv_needs[cid], []).append(cid)
        self.groups = [KvGroup(need, ids, n_pages, max_slots, max_pages, dtype, device, page_tokens)
                       for need, ids in by_need.items()]
        self._group_of = {cid: g for g in self.groups for cid in g.entries}
        self.state = StateStore(state_needs, max_slots, device)

    # ------------------------------------------------------------------ sequences
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.state.reset(slot)
        return slot

    def release(self, slot: int) -> None:
        self.slots.release(slot)
        for g in self.groups:
            g.release(slot)

    def length(self, slot: int) -> int:
        return self.slots.length[slot]

    # ------------------------------------------------------------------ steps
    def prepare(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """Check the step and hand out its pages; nothing has run yet, so an error
        here leaves every sequence as it was."""
        if len(set(slots)) != len(slots):
            raise QStreamError(QsError.INVALID_INPUT, "a sequence appears twice in one step")
        need = [0] * len(self.groups)
        lengths = self.slots.length
        for slot, n in zip(slots, n_new):
            self.slots.require(slot)
            new_len = lengths[slot] + n
            if new_len > self.max_context:
                raise QStreamError(QsError.SEQ_TOO_LONG,
                                   f"sequence in slot {slot} would hold {new_len} tokens; the context is {self.max_context}")
            for gi, g in enumerate(self.groups):
                need[gi] += g.pages_needed(slot, new_len)
        if not any(need):
            return                                      # every token of the step lands in a page already held
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.n_free:
                raise QStreamError(
                    QsError.BUDGET_EXCEEDED,
                    f"the step needs {need[gi]} more cache pages of {self.page_tokens} tokens, "
                    f"{g.pool.n_free} of {g.pool.n_pages} are free (cache sized for {self.max_tokens} tokens)")
        for slot, n in zip(slots, n_new):
            for g in self.groups:
                g.ensure(slot, self.slots.length[slot] + n)
        for g in self.groups:
            g.upload()

    def commit(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """The step has been launched: lengths grow, windows let go of old pages."""
        windowed = [g for g in self.groups if g.need.window > 0]
        for slot, n in zip(slots, n_new):
            self.slots.length[slot] += n
            for g in windowed:
                g.trim(slot, self.slots.length[slot])

    def view(self, cache_id: int) -> CacheView:
        return self._group_of[cache_id].view(cache_id)

    def has_entry(self, cache_id: int) -> bool:
        return cache_id in self._group_of

    @property
    def bytes(self) -> int:
        return sum(g.bytes for g in self.groups) + self.state.bytes

    def check_canaries(self) -> None:
        """Device check: the guard page behind every cache entry's pages is as it was written."""
        for g in self.groups:
            n = g.damaged_guard_words()
            if n:
                raise QStreamError(QsError.INTERNAL, f"{n} guard words behind the cache pages of group {g.need} were overwritten")

    def check(self) -> None:
        """Host invariants: no slot or page lost, held twice or shared."""
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            held = g.table_host[g.table_host >= 0]
            if len(set(held.tolist())) != len(held):
                raise QStreamError(QsError.INTERNAL, "a page belongs to two sequences")
            if len(held) != g.pool.n_pages - g.pool.n_free:
                raise QStreamError(QsError.INTERNAL, "pages held by the pool and by the tables differ")
            for s in range(self.slots.n_slots):
                if not self.slots.active[s] and (g.table_host[s] >= 0).any():
                    raise QStreamError(QsError.INTERNAL, f"free slot {s} still holds pages")
