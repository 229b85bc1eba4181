"""The two ends of a model: token ids into the residual stream, and the stream's wanted rows into logits."""
from __future__ import annotations

import torch

from .base import Embedding, Head, ParamSpec, build_part, register_part


@register_part("embedding", "table")
class TableEmbedding(Embedding):
    """x[t,:] = scale * table[id[t],:] as a copy of rows into 32-bit (v1/tensortype/host_tensor.cpp:189-198 has no
    scale: ``scale`` is 1 there).  ``prefix`` is the table's tensor name."""

    graph_safe = True

    def param_specs(self):
        return {self.prefix: ParamSpec((self.spec.vocab, self.spec.hidden))}

    def load(self, get) -> None:
        self.table = self.rt.load(get, self.prefix)

    def step_bytes(self, n_tokens: int) -> int:
        return n_tokens * self.spec.hidden * self.table.element_size()

    def forward(self, ctx):
        x = torch.empty((ctx.n_tokens, self.spec.hidden), dtype=torch.float32, device=self.rt.device)
        self.rt.ops.embedding(self.table, ctx.token_ids, x, status=ctx.status, scale=self.spec.scale)
        return x


@register_part("head", "linear")
class LinearHead(Head):
    """Norm of the wanted rows only, then their product with the [vocab, hidden] matrix into float32 logits
    (v1/models/qwen2-7b/inference_fp16.dag:383-384, v1/tensortype/cuda_tensor.cpp:946-992: logits for the selected
    positions only), then the optional scale and soft cap.  ``prefix`` is unused: the names are the spec's."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        self.norm = build_part("norm", spec.norm, spec.norm_name, rt)

    @property
    def graph_safe(self):
        return self.norm.graph_safe

    def param_specs(self):
        s = self.spec
        out = {s.name: ParamSpec((s.vocab, s.hidden), optional=s.tied_to is not None)}
        out.update(self.norm.param_specs())
        return out

    def load(self, get) -> None:
        s = self.spec
        self.weight = self.rt.load(get, s.tied_to if s.tied_to is not None else s.name)
        self.norm.load(get)

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size() + self.norm.weight_bytes()

    def first_product(self):
        return self.rt.ops.product_hint(self.weight, "linear")

    def forward(self, stream, ctx):
        s, ops = self.spec, self.rt.ops
        n_want = ctx.want_rows.numel()
        logits = torch.empty((n_want, s.vocab), dtype=torch.float32, device=self.rt.device)
        if n_want == 0:
            return logits
        h = stream.normed(self.norm, rows=ctx.want_rows)
        ops.linear(h, self.weight, None, logits)
        if s.logit_scale != 1.0 or s.logit_cap > 0.0:
            ops.logits_scale_cap(logits, s.logit_scale, s.logit_cap)
        return logits
