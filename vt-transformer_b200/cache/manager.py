"""The cache manager: pages of keys and values with a block table for each request, in
groups, and slots of fixed size for per-request state.

After vt-transformer's ``PageTable`` and ``CacheManager`` (vt-transformer/core/vt_pages.hpp:31-134,
vt-transformer/core/vt_cache.hpp:29-312): a LIFO free list of pages (:50-57,:74-82), a row
for each running request (``alloc_row`` :60-65), allocation that takes all pages of a
step or none (``allocate_pages`` vt_cache.hpp:187-252) and skips positions whose page is
there already (:209-213).  What differs:

* a block table holds one entry for each page, not one for each token (vt_pages.hpp:17-22);
* there is no prefix tree: when a request ends, all its pages go back to the free list at
  once and its row is cleared (the reference leaves a freed row's entries in place,
  vt_pages.hpp:66-70, and never calls ``evict``, vt_cache.hpp:264-269);
* cache slots with different needs are in different groups, each with its own pool and
  tables: a group whose layers see a window of keys gives pages back as soon as the
  window has passed them;
* a row also owns a slot of fixed size in every state tensor a mixer declared.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheView, KVCacheSpec, StateSpec


class OutOfPages(RuntimeError):
    """A step needs more pages than a group has free.  Nothing was allocated."""

    def __init__(self, group: int, needed: int, free: int):
        super().__init__(f"cache group {group} needs {needed} pages and has {free} free")
        self.group, self.needed, self.free = group, needed, free


class OutOfRows(RuntimeError):
    """All request rows are taken."""


# Tokens in a page where the caller names none.  The kernels read keys in runs of 16, so any multiple of 16
# works; the tcgen05 attention kernel brings a page's keys with one TMA box of up to 128 rows, and a box costs
# the TMA unit about the same whatever its size, so pages of 64 serve long prompts better than pages of 16.
DEFAULT_PAGE_SIZE = 64


class PagePool:
    """Pages 0..n-1 with a LIFO free list.  ``give`` refuses a page that is free already
    or that the pool does not have."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # pop() hands out 0, 1, 2, ...
        self._is_free = [True] * num_pages

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(-1, n, len(self._free))
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._is_free[p] = False
        return out

    def give(self, pages: Iterable[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} does not belong to a pool of {self.num_pages} pages")
            if self._is_free[p]:
                raise ValueError(f"page {p} is freed twice")
            self._is_free[p] = True
            self._free.append(p)


@dataclass
class _Group:
    index: int
    spec: KVCacheSpec
    slots: List[int]
    pool: PagePool
    kv: Optional[torch.Tensor]          # [slots, 2, pages, kv_heads, page_size, head_dim]
    table: np.ndarray                   # [rows, max_pages] int32, -1 where no page is held
    first_live: np.ndarray              # [rows] first logical page that may still be held


class CacheManager:
    """``slot_specs``: cache slot id -> ``KVCacheSpec`` or ``StateSpec`` (``DecoderModel.cache_slots()``).

    A request lives in a *row*.  ``admit`` takes a row, ``extend`` makes sure that pages
    cover its positions below a new length (all-or-nothing over a list of requests),
    ``commit`` records the new length and frees what windows have passed, ``release`` gives
    everything back.  ``views`` hands the model a ``CacheView`` for each slot.
    """

    def __init__(self, slot_specs: Dict[int, object], *, page_size: int, num_pages: int, max_requests: int,
                 max_seq_len: int, dtype: torch.dtype, device, window_pages: Optional[int] = None,
                 allocate: bool = True):
        if page_size < 1 or page_size % 16:
            raise ValueError(f"page_size {page_size} must be a positive multiple of 16 (the attention kernels "
                             f"read keys in runs of 16)")
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self.max_pages = -(-max_seq_len // page_size)
        self.dtype, self.device = dtype, device
        self.groups: List[_Group] = []
        self.slot_group: Dict[int, Tuple[int, int]] = {}     # slot -> (group index, index inside the group)
        self.state: Dict[int, torch.Tensor] = {}
        self.state_specs: Dict[int, StateSpec] = {}
        by_key: Dict[Tuple, List[int]] = {}
        for slot in sorted(slot_specs):
            spec = slot_specs[slot]
            if isinstance(spec, KVCacheSpec):
                by_key.setdefault((spec.kv_heads, spec.head_dim, spec.window), []).append(slot)
            elif isinstance(spec, StateSpec):
                self.state_specs[slot] = spec
                self.state[slot] = (torch.zeros((max_requests,) + tuple(spec.shape), dtype=spec.dtype, device=device)
                                    if allocate else None)
            else:
                raise TypeError(f"cache slot {slot}: unknown kind of cache spec {spec!r}")
        for key, slots in by_key.items():
            kv_heads, head_dim, window = key
            n = num_pages if (window is None or window_pages is None) else window_pages
            kv = None
            if allocate:
                kv = torch.zeros((len(slots), 2, n, kv_heads, page_size, head_dim), dtype=dtype, device=device)
            g = _Group(len(self.groups), KVCacheSpec(kv_heads, head_dim, window), slots, PagePool(n), kv,
                       np.full((max_requests, self.max_pages), -1, dtype=np.int32),
                       np.zeros(max_requests, dtype=np.int64))
            for i, s in enumerate(slots):
                self.slot_group[s] = (g.index, i)
            self.groups.append(g)
        self._free_rows = list(range(max_requests - 1, -1, -1))
        self._live = [False] * max_requests
        self.lengths = np.zeros(max_requests, dtype=np.int64)

    # ---- rows ------------------------------------------------------------------------
    @property
    def free_rows(self) -> int:
        return len(self._free_rows)

    def admit(self) -> int:
        """Takes a row for a new request: length 0, no pages, state slots zero."""
        if not self._free_rows:
            raise OutOfRows(f"all {self.max_requests} request rows are taken")
        row = self._free_rows.pop()
        self._live[row] = True
        self.lengths[row] = 0
        for t in self.state.values():
            if t is not None:
                t[row].zero_()
        return row

    def release(self, row: int) -> None:
        """Ends a request: every page it holds goes back to its pool, its tables are
        cleared, its row is free."""
        self._check_row(row)
        for g in self.groups:
            held = g.table[row]
            idx = np.nonzero(held >= 0)[0]
            g.pool.give(int(p) for p in held[idx])
            held[idx] = -1
            g.first_live[row] = 0
        self.lengths[row] = 0
        self._live[row] = False
        self._free_rows.append(row)

    def _check_row(self, row: int) -> None:
        if not (0 <= row < self.max_requests and self._live[row]):
            raise ValueError(f"row {row} holds no request")

    def length(self, row: int) -> int:
        return int(self.lengths[row])

    # ---- pages -----------------------------------------------------------------------
    def _first_needed_page(self, g: _Group, length: int) -> int:
        """First logical page that a token at position >= length may still read."""
        if g.spec.window is None:
            return 0
        return max(0, length - g.spec.window + 1) // self.page_size

    def _missing(self, g: _Group, row: int, new_len: int) -> List[int]:
        lo = self._first_needed_page(g, int(self.lengths[row]))
        hi = -(-new_len // self.page_size)
        seg = g.table[row, lo:hi]
        return [lo + int(i) for i in np.nonzero(seg < 0)[0]]

    def pages_needed(self, items: Sequence[Tuple[int, int]]) -> List[int]:
        """Pages each group would have to hand out to cover ``(row, new_len)`` for all items."""
        need = [0] * len(self.groups)
        for row, new_len in items:
            for g in self.groups:
                need[g.index] += len(self._missing(g, row, new_len))
        return need

    def pages_for_new(self, n_tokens: int) -> List[int]:
        """Pages each group needs for the first ``n_tokens`` of a request not yet admitted."""
        return [-(-n_tokens // self.page_size) for _ in self.groups]

    def free_pages(self) -> List[int]:
        return [g.pool.free for g in self.groups]

    def extend(self, items: Sequence[Tuple[int, int]]) -> None:
        """Makes sure pages cover positions < new_len of every (row, new_len).  Either all
        pages of all items and groups are found, or ``OutOfPages`` is raised and nothing
        has changed."""
        plans = []
        for row, new_len in items:
            self._check_row(row)
            if new_len > self.max_seq_len:
                raise ValueError(f"row {row}: length {new_len} is above max_seq_len {self.max_seq_len}")
            if new_len < self.lengths[row]:
                raise ValueError(f"row {row}: length {new_len} is below the cached length {self.lengths[row]}")
        for g in self.groups:
            want = [(row, self._missing(g, row, new_len)) for row, new_len in items]
            total = sum(len(m) for _, m in want)
            if total > g.pool.free:
                raise OutOfPages(g.index, total, g.pool.free)
            plans.append((g, want, total))
        for g, want, total in plans:
            pages = g.pool.take(total)
            at = 0
            for row, missing in want:
                for logical in missing:
                    g.table[row, logical] = pages[at]
                    at += 1

    def commit(self, row: int, new_len: int) -> None:
        """Records that positions < new_len are cached, and gives back the pages of window
        groups that no later token can read."""
        self._check_row(row)
        self.lengths[row] = new_len
        for g in self.groups:
            if g.spec.window is None:
                continue
            lo = self._first_needed_page(g, new_len)
            first = int(g.first_live[row])
            if lo > first:
                seg = g.table[row, first:lo]
                idx = np.nonzero(seg >= 0)[0]
                g.pool.give(int(p) for p in seg[idx])
                seg[idx] = -1
                g.first_live[row] = lo

    # ---- what a step sees --------------------------------------------------------------
    def table_rows(self, group: int, rows: Sequence[int], n_pages: int) -> np.ndarray:
        """[len(rows), n_pages] int32 copy of the block-table rows of a group."""
        return self.groups[group].table[np.asarray(rows, dtype=np.int64), :n_pages]

    def views(self, block_tables: Dict[int, torch.Tensor]) -> Dict[int, CacheView]:
        """slot -> ``CacheView``; ``block_tables[group]`` is the device table of this step."""
        out: Dict[int, CacheView] = {}
        for slot, (gi, si) in self.slot_group.items():
            g = self.groups[gi]
            out[slot] = CacheView(spec=g.spec, k=g.kv[si, 0], v=g.kv[si, 1], block_table=block_tables[gi],
                                  page_size=self.page_size)
        for slot, t in self.state.items():
            out[slot] = CacheView(spec=self.state_specs[slot], state=t)
        return out

    def bytes_per_token(self) -> int:
        """Bytes of keys and values one cached token takes, over all slots."""
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * g.spec.kv_heads * g.spec.head_dim * item * len(g.slots) for g in self.groups)

    # ---- invariants (tests) --------------------------------------------------------------
    def check(self) -> None:
        """No page lost, none held twice, none both held and free; rows consistent."""
        for g in self.groups:
            held = g.table[g.table >= 0]
            if len(np.unique(held)) != len(held):
                raise AssertionError(f"group {g.index}: a page is held twice")
            if any(g.pool._is_free[int(p)] for p in held):
                raise AssertionError(f"group {g.index}: a held page is on the free list")
            if len(held) + g.pool.free != g.pool.num_pages:
                raise AssertionError(f"group {g.index}: {g.pool.num_pages - len(held) - g.pool.free} pages are lost")
            if len(set(g.pool._free)) != len(g.pool._free):
                raise AssertionError(f"group {g.index}: a page is on the free list twice")
            for row in range(self.max_requests):
                if not self._live[row] and (g.table[row] >= 0).any():
                    raise AssertionError(f"group {g.index}: free row {row} still holds pages")
        if len(set(self._free_rows)) != len(self._free_rows):
            raise AssertionError("a row is on the free list twice")
        if sum(self._live) + len(self._free_rows) != self.max_requests:
            raise AssertionError("a row is lost")
