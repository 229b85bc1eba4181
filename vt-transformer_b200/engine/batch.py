"""What one step runs: a flat batch of (request, its next tokens), and the device-side
description of it that the kernels read.

vt-transformer's engines take either a padded [batch, tokens] rectangle with masks (v1:
v1/tensortype/nn_kvcache.cpp:365-393) or a batch that is all prompts or all single tokens
(v2: vt-transformer/core/vt_engine.hpp:13-17), and the host fills several mirrors that are
copied one by one (vt-transformer/models/qwen3-0.6b/kernels/prefill.h:95-115).  Here a
step is one flat list of tokens: portions of prompts of any length beside single decoded
tokens, described by a handful of int32 arrays that travel to the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """``row``: the request's row in the cache manager.  ``tokens``: its next tokens, which
    follow the ones already cached.  ``want``: indices into ``tokens`` whose logits are
    asked for."""
    row: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class SeqSlice:
    """One entry as the parts see it on the host: tokens [offset, offset + length) of the
    flat batch are positions [start, start + length) of the request in ``row``."""
    row: int
    start: int
    length: int
    offset: int


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    seqs: List[SeqSlice]
    token_ids: torch.Tensor        # [T] int32
    positions: torch.Tensor        # [T] int32, position of the token in its request
    token_seq: torch.Tensor        # [T] int32, index of the token's entry in this step (-1: padding)
    cu_q: torch.Tensor             # [n + 1] int32, offsets of the entries in the flat batch
    q_start: torch.Tensor          # [n] int32, tokens cached before this step
    kv_len: torch.Tensor           # [n] int32, tokens cached after this step
    rows: torch.Tensor             # [n] int32, request rows (index of per-request state)
    want_rows: torch.Tensor        # [W] int32, flat indices of the tokens whose logits are wanted
    block_tables: Dict[int, torch.Tensor]   # cache group -> [n, pages] int32
    max_q_len: int
    max_kv_len: int
    status: Optional[torch.Tensor] = None   # [2] int32 on the device: code, detail
    want_inverse: Optional[np.ndarray] = None   # set if wanted rows repeat: logits[want_inverse]
    extras: dict = field(default_factory=dict)  # per-step scratch of the kernels' wrappers
    h2d_bytes: int = 0                          # bytes of the description copied to the device
    min_kv_len: int = 0                         # a lower bound of the cached lengths, if the caller knows one (else 0)


def _align4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class Layout:
    """Where the arrays of a step lie in its one int32 buffer."""
    T: int
    n: int
    W: int
    n_pages: int
    n_groups: int
    offs: List[int]
    sizes: List[int]
    total: int

    @staticmethod
    def make(T: int, n: int, W: int, n_pages: int, n_groups: int) -> "Layout":
        sizes = [T, T, T, n + 1, n, n, n, W] + [n * n_pages] * n_groups
        offs, total = [], 0
        for sz in sizes:
            offs.append(total)
            total += _align4(max(sz, 1))
        return Layout(T, n, W, n_pages, n_groups, offs, sizes, total)

    def seg(self, buf, i):
        return buf[self.offs[i]:self.offs[i] + self.sizes[i]]


def fill_host(host: np.ndarray, lay: Layout, entries: Sequence[StepEntry], seqs: List[SeqSlice], want_flat: List[int],
              cache) -> None:
    """Writes the step's arrays into ``host``.  The layout may be larger than the step (a fixed
    layout of a captured graph): the rest is padding -- tokens of no sequence (id and sequence -1),
    sequences without tokens, block-table entries -1, wanted rows that point at themselves."""
    book = getattr(cache, "book", None)
    if book is not None and host.dtype == np.int32 and host.flags.c_contiguous and host.flags.writeable:
        # the C++ side of the cache manager packs the step (csrc/host_runtime.cpp)
        book.fill_step(host, lay.T, lay.n, lay.W, lay.n_pages, lay.offs, lay.sizes,
                       [(e.row, e.tokens) for e in entries], [int(w) for w in want_flat])
        return
    T, n = sum(s.length for s in seqs), len(seqs)
    tok, pos, tseq = lay.seg(host, 0), lay.seg(host, 1), lay.seg(host, 2)
    tok[T:], pos[T:], tseq[T:] = -1, 0, -1
    for i, (e, sl) in enumerate(zip(entries, seqs)):
        a, b = sl.offset, sl.offset + sl.length
        tok[a:b] = np.asarray(e.tokens, dtype=np.int32)
        pos[a:b] = np.arange(sl.start, sl.start + sl.length, dtype=np.int32)
        tseq[a:b] = i
    cu = lay.seg(host, 3)
    cu[:n] = [sl.offset for sl in seqs]
    cu[n:] = T
    q_start, kv_len, rows, want = lay.seg(host, 4), lay.seg(host, 5), lay.seg(host, 6), lay.seg(host, 7)
    q_start[:n] = [sl.start for sl in seqs]
    kv_len[:n] = [sl.start + sl.length for sl in seqs]
    rows[:n] = [sl.row for sl in seqs]
    q_start[n:], kv_len[n:], rows[n:] = 0, 0, 0
    w = len(want_flat)
    want[:w] = want_flat
    want[w:] = np.arange(lay.T - (lay.W - w), lay.T, dtype=np.int32)   # padding rows want themselves
    live = [sl.row for sl in seqs]
    for g in range(lay.n_groups):
        bt = lay.seg(host, 8 + g).reshape(lay.n, lay.n_pages)
        bt[n:] = -1
        bt[:n] = cache.table_rows(g, live, lay.n_pages)


def context_from(buf: torch.Tensor, lay: Layout, seqs: List[SeqSlice], max_q_len: int, max_kv_len: int, status,
                 want_inverse=None) -> StepContext:
    return StepContext(
        n_tokens=lay.T, n_seqs=lay.n, seqs=seqs, token_ids=lay.seg(buf, 0), positions=lay.seg(buf, 1),
        token_seq=lay.seg(buf, 2), cu_q=lay.seg(buf, 3), q_start=lay.seg(buf, 4), kv_len=lay.seg(buf, 5),
        rows=lay.seg(buf, 6), want_rows=lay.seg(buf, 7),
        block_tables={g: lay.seg(buf, 8 + g).view(lay.n, lay.n_pages) for g in range(lay.n_groups)},
        max_q_len=max_q_len, max_kv_len=max_kv_len, status=status, want_inverse=want_inverse, h2d_bytes=lay.total * 4)


def slices_of(entries: Sequence[StepEntry], cache) -> List[SeqSlice]:
    seqs, off = [], 0
    for e in entries:
        seqs.append(SeqSlice(e.row, cache.length(e.row), len(e.tokens), off))
        off += len(e.tokens)
    return seqs


def build_context(entries: Sequence[StepEntry], cache, device, status=None, carried=None) -> StepContext:
    """Packs the description of a step into one int32 buffer, copies it to the device in
    one transfer and returns views into it.  ``cache`` gives each row's cached length and
    block-table rows; pages for the new tokens must have been allocated already.
    ``carried``: an int32 tensor on the device whose element i is the token of entry i (every
    entry then brings one token, whose id the host does not know yet: the step before sampled it
    and may still be running); it is copied over the token ids on the device."""
    seqs = slices_of(entries, cache)
    T = sum(s.length for s in seqs)
    want_flat = [sl.offset + int(w) for e, sl in zip(entries, seqs) for w in e.want]
    want_inverse = None
    if len(set(want_flat)) != len(want_flat):
        uniq, inverse = np.unique(np.asarray(want_flat, dtype=np.int64), return_inverse=True)
        want_flat, want_inverse = [int(u) for u in uniq], inverse
    max_kv = max((s.start + s.length for s in seqs), default=0)
    lay = Layout.make(T, len(seqs), len(want_flat), max(1, -(-max_kv // cache.page_size)), len(cache.groups))
    dev = torch.device(device)
    if dev.type == "cuda":
        pinned = torch.empty(lay.total, dtype=torch.int32, pin_memory=True)
        fill_host(pinned.numpy(), lay, entries, seqs, want_flat, cache)
        buf = pinned.to(dev, non_blocking=True)
    else:
        host = np.empty(lay.total, dtype=np.int32)
        fill_host(host, lay, entries, seqs, want_flat, cache)
        buf = torch.from_numpy(host).to(dev)
    if carried is not None:
        if any(len(e.tokens) != 1 for e in entries) or carried.numel() < len(entries):
            raise ValueError("carried tokens stand for one token of every entry")
        buf[:len(entries)].copy_(carried[:len(entries)])
    return context_from(buf, lay, seqs, max((s.length for s in seqs), default=0), max_kv, status, want_inverse)
