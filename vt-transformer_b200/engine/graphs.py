"""CUDA graphs of single-token steps.

A decode step of a small batch is some hundreds of short kernels; launched one by one from
Python their launch cost is most of the step.  A step in which every request brings one
token has a shape that depends on the number of requests only, so it is captured once as a
CUDA graph for a padded batch size and replayed: the step's description is copied into the
graph's fixed buffer and everything else (positions, block tables, cached lengths) is read
by the kernels from there.  Padding tokens belong to no sequence; kernels skip them.
"""
from __future__ import annotations

import gc

from typing import Sequence

import torch

from .batch import Layout, StepEntry, context_from, fill_host, slices_of

BATCH_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def batch_bucket(n: int):
    for b in BATCH_BUCKETS:
        if n <= b:
            return b
    return None


def context_bucket(max_kv_len: int) -> int:
    """Upper bound of the cached length that a captured graph serves (it sets how many CTAs the
    keys of a sequence are split over): powers of two from 256."""
    b = 256
    while b < max_kv_len:
        b *= 2
    return b


class DecodeGraph:
    """One captured step for ``batch`` single-token entries and cached lengths up to ``kv_bound``
    (``like_lengths``: all of them at least a quarter of it)."""

    def __init__(self, runner, batch: int, kv_bound: int, like_lengths: bool = False):
        cache, dev = runner.cache, runner.rt.device
        self.runner, self.batch, self.kv_bound = runner, batch, kv_bound
        self.layout = Layout.make(batch, batch, batch, cache.max_pages, len(cache.groups))
        # The host may run ahead of the device: a staging buffer is written again only after the
        # copy that read it last has been done (an event for each buffer of a small ring).
        self.ring = [torch.empty(self.layout.total, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self.events = [None] * len(self.ring)
        self.turn = 0
        self.device_buf = torch.zeros(self.layout.total, dtype=torch.int32, device=dev)
        for pinned in self.ring:
            pinned.zero_()
            fill_host(pinned.numpy(), self.layout, [], [], [], cache)  # all padding: a valid step of nothing
        self.device_buf.copy_(self.ring[0], non_blocking=True)
        self.ctx = context_from(self.device_buf, self.layout, [], 1, kv_bound, runner.status)
        self.ctx.min_kv_len = kv_bound // 4 if like_lengths else 0
        views = cache.views(self.ctx.block_tables)
        # warm up on a side stream (first calls of kernels set attributes and allocate), then capture
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.ctx.extras.clear()
                runner.model.forward(self.ctx, views)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        launches_before = runner.rt.ops.launches
        # No garbage collection while the stream is capturing: collecting an older graph there (a runner that
        # is no longer used) destroys it, which CUDA does not allow inside a capture and which would spoil this one.
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.ctx.extras.clear()
                self.logits = runner.model.forward(self.ctx, views)
        finally:
            if was_enabled:
                gc.enable()
        self.launches = runner.rt.ops.launches - launches_before

    def run(self, entries: Sequence[StepEntry], carried=None) -> torch.Tensor:
        cache = self.runner.cache
        seqs = [] if hasattr(cache, "book") else slices_of(entries, cache)     # the C++ side packs from its own lengths
        slot = self.turn
        self.turn = (self.turn + 1) % len(self.ring)
        if self.events[slot] is not None:
            self.events[slot].synchronize()
        fill_host(self.ring[slot].numpy(), self.layout, entries, seqs, list(range(len(entries))), cache)
        self.ctx.seqs = seqs
        self.device_buf.copy_(self.ring[slot], non_blocking=True)
        if self.events[slot] is None:
            self.events[slot] = torch.cuda.Event()
        self.events[slot].record()
        if carried is not None:                     # the ids that the step before sampled, still on the device
            self.device_buf[:len(entries)].copy_(carried[:len(entries)])
        self.graph.replay()
        self.runner.rt.ops.launches += self.launches
        return self.logits[:len(entries)]
