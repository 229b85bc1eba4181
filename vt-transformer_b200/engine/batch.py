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


def _align4(n: int) -> int:
    return (n + 3) & ~3


def build_context(entries: Sequence[StepEntry], cache, device, status=None) -> StepContext:
    """Packs the description of a step into one int32 buffer, copies it to the device in
    one transfer and returns views into it.  ``cache`` gives each row's cached length and
    block-table rows; pages for the new tokens must have been allocated already."""
    n = len(entries)
    lens = [len(e.tokens) for e in entries]
    T = sum(lens)
    starts = [cache.length(e.row) for e in entries]
    seqs, off = [], 0
    for e, s, l in zip(entries, starts, lens):
        seqs.append(SeqSlice(e.row, s, l, off))
        off += l
    want_flat = [sl.offset + int(w) for e, sl in zip(entries, seqs) for w in e.want]
    want_inverse = None
    if len(set(want_flat)) != len(want_flat):
        uniq, inverse = np.unique(np.asarray(want_flat, dtype=np.int64), return_inverse=True)
        want_flat, want_inverse = [int(u) for u in uniq], inverse
    W = len(want_flat)
    max_kv = max((s + l for s, l in zip(starts, lens)), default=0)
    n_pages = max(1, -(-max_kv // cache.page_size))
    n_groups = len(cache.groups)

    sizes = [T, T, T, n + 1, n, n, n, W] + [n * n_pages] * n_groups
    offs, total = [], 0
    for sz in sizes:
        offs.append(total)
        total += _align4(max(sz, 1))
    host = np.empty(total, dtype=np.int32)

    def seg(i):
        return host[offs[i]:offs[i] + sizes[i]]

    tok, pos, tseq = seg(0), seg(1), seg(2)
    for i, (e, sl) in enumerate(zip(entries, seqs)):
        a, b = sl.offset, sl.offset + sl.length
        tok[a:b] = np.asarray(e.tokens, dtype=np.int32)
        pos[a:b] = np.arange(sl.start, sl.start + sl.length, dtype=np.int32)
        tseq[a:b] = i
    seg(3)[:] = np.asarray([sl.offset for sl in seqs] + [T], dtype=np.int32)
    seg(4)[:] = np.asarray(starts, dtype=np.int32)
    seg(5)[:] = np.asarray([s + l for s, l in zip(starts, lens)], dtype=np.int32)
    seg(6)[:] = np.asarray([e.row for e in entries], dtype=np.int32)
    seg(7)[:] = np.asarray(want_flat, dtype=np.int32)
    rows = [e.row for e in entries]
    for g in range(n_groups):
        seg(8 + g)[:] = cache.table_rows(g, rows, n_pages).reshape(-1)

    dev = torch.device(device)
    if dev.type == "cuda":
        pinned = torch.empty(total, dtype=torch.int32, pin_memory=True)
        pinned.numpy()[:] = host
        buf = pinned.to(dev, non_blocking=True)
    else:
        buf = torch.from_numpy(host.copy()).to(dev)

    def dseg(i):
        return buf[offs[i]:offs[i] + sizes[i]]

    return StepContext(
        n_tokens=T, n_seqs=n, seqs=seqs, token_ids=dseg(0), positions=dseg(1), token_seq=dseg(2), cu_q=dseg(3),
        q_start=dseg(4), kv_len=dseg(5), rows=dseg(6), want_rows=dseg(7),
        block_tables={g: dseg(8 + g).view(n, n_pages) for g in range(n_groups)},
        max_q_len=max(lens, default=0), max_kv_len=max_kv, status=status, want_inverse=want_inverse,
        h2d_bytes=total * 4)
