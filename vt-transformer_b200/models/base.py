"""A decoder model put together from a ``ModelSpec``: embedding, blocks in their run
order, final norm, output head.  It names no architecture."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..parts.base import CacheView, ParamSpec, ResidualStream, Runtime, build_part
from ..parts.specs import ModelSpec
from ..weights.loader import WeightSource, check_against


class DecoderModel:
    """The model of vt-transformer's ``gpu_main`` (v1/models/qwen2-7b/inference_fp16.dag:368-396):
    embed the tokens, run the layers, norm, logits at the wanted rows only.

    ``order`` is data: ``spec.order[n] = RunSpec(block, cache, writes)``.  The cache slots
    that the runs name are declared by ``cache_slots()``: slot id -> the cache spec of the
    block whose run writes it."""

    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.blocks = [build_part("block", b, b.prefix, rt) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm_name, rt)
        self.embed = None
        self.head = None
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
        return all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = self.spec
        out = {s.embed_name: ParamSpec((s.vocab, s.hidden))}
        out[s.head_name] = ParamSpec((s.vocab, s.hidden), optional=s.tied_head)
        for b in self.blocks:
            out.update(b.param_specs())
        out.update(self.final_norm.param_specs())
        return out

    # ---- weights -------------------------------------------------------------------
    def load(self, source: WeightSource) -> None:
        """Checks the source against the parameter table (one error for all differences),
        then hands each part its tensors."""
        check_against(source, self.param_specs())
        s = self.spec
        self.embed = self.rt.param(source.get(s.embed_name))
        if s.head_name in source.entries() and not s.tied_head:
            self.head = self.rt.param(source.get(s.head_name))
        else:
            self.head = self.embed
        for b in self.blocks:
            b.load(source.get)
        self.final_norm.load(source.get)

    def weight_bytes(self, n_tokens: int = 1) -> int:
        """Bytes of weights a step reads: every block's weights once for each of its runs,
        the head, the final norm, and the embedding rows of the step's tokens."""
        n = sum(self.blocks[r.block].weight_bytes() for r in self.spec.order)
        n += self.final_norm.weight_bytes()
        n += self.head.numel() * self.head.element_size()
        n += n_tokens * self.spec.hidden * self.embed.element_size()
        return n

    # ---- forward -------------------------------------------------------------------
    def forward(self, ctx, views: Dict[int, CacheView]) -> torch.Tensor:
        """Runs the step's tokens and returns float32 logits [wanted rows, vocab].
        ``views[slot]`` is the cache view of a slot for this step."""
        ops, s = self.rt.ops, self.spec
        x = torch.empty((ctx.n_tokens, s.hidden), dtype=torch.float32, device=self.rt.device)
        ops.embedding(self.embed, ctx.token_ids, x, status=ctx.status)
        stream = ResidualStream(x, status=ctx.status)
        for run in s.order:
            view: Optional[CacheView] = None
            if run.cache is not None and run.cache in views:
                view = views[run.cache]
                if view.writes != run.writes:
                    view = CacheView(**{**view.__dict__, "writes": run.writes})
            self.blocks[run.block].forward(stream, ctx, view)
        n_want = ctx.want_rows.numel()
        logits = torch.empty((n_want, s.vocab), dtype=torch.float32, device=self.rt.device)
        if n_want == 0:
            return logits
        h = stream.normed(self.final_norm, rows=ctx.want_rows)
        ops.linear(h, self.head, None, logits)
        return logits
