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

from ..parts.base import CacheView, PagedLayout, StateLayout, cache_layout


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


def _host():
    from ..csrc import build
    return build.load_host()


class PagePool:
    """Pages 0..n-1 with a LIFO free list (the pool of ``csrc/host_runtime.cpp``).  ``give`` refuses a
    page that is free already or that the pool does not have."""

    def __init__(self, num_pages: int):
        self._pool = _host().Pool(num_pages)

    @property
    def num_pages(self) -> int:
        return self._pool.num_pages

    @property
    def free(self) -> int:
        return self._pool.free

    def take(self, n: int) -> List[int]:
        out = self._pool.take(n)
        if out is None:
            raise OutOfPages(-1, n, self._pool.free)
        return out

    def give(self, pages: Iterable[int]) -> None:
        self._pool.give([int(p) for p in pages])


class _GroupPool:
    """What is read of a group's pool from outside: its size and how many pages are free."""

    def __init__(self, book, index: int):
        self._book, self._index = book, index

    @property
    def num_pages(self) -> int:
        return self._book.pool_pages(self._index)

    @property
    def free(self) -> int:
        return self._book.free_pages()[self._index]


@dataclass
class _Group:
    index: int
    layout: PagedLayout
    slots: List[int]
    pool: _GroupPool
    tensors: Optional[Dict[str, torch.Tensor]]   # name -> [slots, pages, outer, page_size, inner]
    table: np.ndarray                   # [rows, max_pages] int32, -1 where no page is held: a view of the book's table

    @property
    def spec(self):
        """The group's layout (its ``tensors`` and its ``window``)."""
        return self.layout


class CacheManager:
    """``slot_specs``: cache slot id -> a cache spec (``DecoderModel.cache_slots()``): ``KVCacheSpec``, ``StateSpec``,
    or any kind that ``parts.register_cache_kind`` has given a layout.  Slots with equal paged layouts form a group.

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
        self.state_specs: Dict[int, object] = {}
        by_layout: Dict[PagedLayout, List[int]] = {}
        self.slot_specs = dict(slot_specs)
        for slot in sorted(slot_specs):
            try:
                layout = cache_layout(slot_specs[slot])
            except TypeError as e:
                raise TypeError(f"cache slot {slot}: {e}") from None
            if isinstance(layout, PagedLayout):
                by_layout.setdefault(layout, []).append(slot)
            elif isinstance(layout, StateLayout):
                self.state_specs[slot] = slot_specs[slot]
                self.state[slot] = (torch.zeros((max_requests,) + tuple(layout.shape), dtype=layout.dtype, device=device)
                                    if allocate else None)
            else:
                raise TypeError(f"cache slot {slot}: a layout must be a PagedLayout or a StateLayout, found {layout!r}")
        plan = [(layout, slots, num_pages if (layout.window is None or window_pages is None) else window_pages)
                for layout, slots in by_layout.items()]
        # the bookkeeping (rows, lengths, free lists, block tables) is the C++ object; the tensors stay here
        self.book = _host().CacheBook(page_size, max_requests, max_seq_len,
                                      [(-1 if layout.window is None else int(layout.window), n) for layout, _, n in plan])
        for layout, slots, n in plan:
            tensors = None
            if allocate:
                tensors = {name: torch.zeros((len(slots), n, outer, page_size, inner), dtype=dtype, device=device)
                           for name, outer, inner in layout.tensors}
            index = len(self.groups)
            g = _Group(index, layout, slots, _GroupPool(self.book, index), tensors, self.book.table(index))
            for i, s in enumerate(slots):
                self.slot_group[s] = (g.index, i)
            self.groups.append(g)
        self.lengths = self.book.lengths()        # [rows] int64: a view of the book's lengths

    # ---- rows ------------------------------------------------------------------------
    @property
    def free_rows(self) -> int:
        return self.book.free_rows

    def admit(self) -> int:
        """Takes a row for a new request: length 0, no pages, state slots zero."""
        row = self.book.admit()
        if row < 0:
            raise OutOfRows(f"all {self.max_requests} request rows are taken")
        self.zero_state(row)
        return row

    def zero_state(self, row: int) -> None:
        """Clears the row's slot in every state tensor (for a row that the book has just admitted)."""
        for t in self.state.values():
            if t is not None:
                t[row].zero_()

    def release(self, row: int) -> None:
        """Ends a request: every page it holds goes back to its pool, its tables are
        cleared, its row is free."""
        self.book.release(row)

    def length(self, row: int) -> int:
        return self.book.length(row)

    # ---- pages -----------------------------------------------------------------------
    def pages_needed(self, items: Sequence[Tuple[int, int]]) -> List[int]:
        """Pages each group would have to hand out to cover ``(row, new_len)`` for all items."""
        return self.book.pages_needed([(int(r), int(n)) for r, n in items])

    def pages_for_new(self, n_tokens: int) -> List[int]:
        """Pages each group needs for the first ``n_tokens`` of a request not yet admitted."""
        return [-(-n_tokens // self.page_size) for _ in self.groups]

    def free_pages(self) -> List[int]:
        return self.book.free_pages()

    def extend(self, items: Sequence[Tuple[int, int]]) -> None:
        """Makes sure pages cover positions < new_len of every (row, new_len).  Either all
        pages of all items and groups are found, or ``OutOfPages`` is raised and nothing
        has changed."""
        group, needed, free = self.book.extend([(int(r), int(n)) for r, n in items])
        if group >= 0:
            raise OutOfPages(group, needed, free)

    def commit(self, row: int, new_len: int) -> None:
        """Records that positions < new_len are cached, and gives back the pages of window
        groups that no later token can read."""
        self.book.commit(row, int(new_len))

    # ---- what a step sees --------------------------------------------------------------
    def table_rows(self, group: int, rows: Sequence[int], n_pages: int) -> np.ndarray:
        """[len(rows), n_pages] int32 copy of the block-table rows of a group."""
        return self.groups[group].table[np.asarray(rows, dtype=np.int64), :n_pages]

    def views(self, block_tables: Dict[int, torch.Tensor]) -> Dict[int, CacheView]:
        """slot -> ``CacheView``; ``block_tables[group]`` is the device table of this step."""
        out: Dict[int, CacheView] = {}
        for slot, (gi, si) in self.slot_group.items():
            g = self.groups[gi]
            pages = {name: t[si] for name, t in g.tensors.items()}
            out[slot] = CacheView(spec=self.slot_specs[slot], k=pages.get("k"), v=pages.get("v"), pages=pages,
                                  block_table=block_tables[gi], page_size=self.page_size)
        for slot, t in self.state.items():
            out[slot] = CacheView(spec=self.state_specs[slot], state=t)
        return out

    def bytes_per_token(self) -> int:
        """Bytes of keys and values one cached token takes, over all slots."""
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(outer * inner * item * len(g.slots) for g in self.groups for _, outer, inner in g.layout.tensors)

    # ---- invariants (tests) --------------------------------------------------------------
    def check(self) -> None:
        """No page lost, none held twice, none both held and free; rows consistent."""
        problem = self.book.check()
        if problem:
            raise AssertionError(problem)
