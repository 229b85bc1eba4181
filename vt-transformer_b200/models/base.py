"""A decoder model put together from a ``ModelSpec``: an embedding part, blocks in their run
order, a head part.  It names no architecture and knows no part's kind."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..parts.base import CacheView, ParamSpec, ResidualStream, Runtime, build_part
from ..parts.specs import ModelSpec
from ..weights.loader import WeightSource, check_against, load_report


class DecoderModel:
    """The model of vt-transformer's ``gpu_main`` (v1/models/qwen2-7b/inference_fp16.dag:368-396):
    embed the tokens, run the layers, norm, logits at the wanted rows only.

    ``order`` is data: ``spec.order[n] = RunSpec(block, cache, writes)``.  The cache slots
    that the runs name are declared by ``cache_slots()``: slot id -> the cache spec of the
    block whose run writes it."""

    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = build_part("embedding", spec.embedding, spec.embedding.name, rt)
        self.blocks = [build_part("block", b, b.prefix, rt) for b in spec.blocks]
        self.head = build_part("head", spec.head, spec.head.name, rt)
        self.load_info, self.load_warnings = [], []
        self._check_order()

    # ---- structure -----------------------------------------------------------------
    def _check_order(self) -> None:
        slots: Dict[int, object] = {}
        for n, run in enumerate(self.spec.order):
            if not 0 <= run.block < len(self.blocks):
                raise ValueError(f"run {n} names block {run.block}; the model has {len(self.blocks)}")
            need = self.blocks[run.block].cache_spec()
            if need is None:
                continue
            if run.cache is None:
                raise ValueError(f"run {n}: block {run.block} keeps a cache but the run names no slot")
            if run.writes:
                if run.cache in slots:
                    raise ValueError(f"run {n}: cache slot {run.cache} is written by an earlier run already")
                slots[run.cache] = need
            else:
                if run.cache not in slots:
                    raise ValueError(f"run {n} reads cache slot {run.cache} before any run wrote it")
                have = slots[run.cache]
                if type(have) is not type(need) or getattr(have, "kv_heads", None) != getattr(need, "kv_heads", None) \
                        or getattr(have, "head_dim", None) != getattr(need, "head_dim", None):
                    raise ValueError(f"run {n}: cache slot {run.cache} has another layout than block {run.block} reads")
        self._slots = slots

    def cache_slots(self) -> Dict[int, object]:
        return dict(self._slots)

    def graph_safe(self) -> bool:
        """True if a step of this model may be captured as a CUDA graph and replayed."""
        return all(p.graph_safe for p in (self.embedding, *self.blocks, self.head))

    def param_specs(self) -> Dict[str, ParamSpec]:
        out = dict(self.embedding.param_specs())
        for b in self.blocks:
            out.update(b.param_specs())
        for name, spec in self.head.param_specs().items():
            out.setdefault(name, spec)          # a head tied to the embedding names the same tensor
        return out

    # ---- weights -------------------------------------------------------------------
    def load(self, source: WeightSource) -> None:
        """Checks the source against the parameter table (one error for all differences),
        then hands each part its tensors."""
        aside = check_against(source, self.param_specs(), self.spec.ignored)
        self.rt.notes.clear()
        for part in (self.embedding, *self.blocks, self.head):
            part.load(source.get)
        self.rt.loaded.clear()                  # the parts hold what they share; nothing else needs the table
        self.load_info, self.load_warnings = load_report(source, self.rt.notes, aside)
        self._link_runs()

    def _link_runs(self) -> None:
        """Tells every run's block which matrix the step streams after it: the first product of the block of the
        next run, of the head after the last.  (A block that runs twice keeps what follows its last run.)"""
        runs = self.spec.order
        for n, run in enumerate(runs):
            after = self.blocks[runs[n + 1].block] if n + 1 < len(runs) else self.head
            self.blocks[run.block].link(after.first_product())

    def weight_bytes(self, n_tokens: int = 1) -> int:
        """Bytes of weights a step reads: every block's weights once for each of its runs,
        the head with its norm, and the embedding rows of the step's tokens."""
        n = sum(self.blocks[r.block].weight_bytes() for r in self.spec.order)
        return n + self.head.weight_bytes() + self.embedding.step_bytes(n_tokens)

    # ---- forward -------------------------------------------------------------------
    def forward(self, ctx, views: Dict[int, CacheView]) -> torch.Tensor:
        """Runs the step's tokens and returns float32 logits [wanted rows, vocab].
        ``views[slot]`` is the cache view of a slot for this step."""
        stream = ResidualStream(self.embedding.forward(ctx), status=ctx.status)
        for run in self.spec.order:
            view: Optional[CacheView] = None
            if run.cache is not None and run.cache in views:
                view = views[run.cache]
                if view.writes != run.writes:
                    view = CacheView(**{**view.__dict__, "writes": run.writes})
            self.blocks[run.block].forward(stream, ctx, view)
        return self.head.forward(stream, ctx)
