"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from .base import FeedForward, ParamSpec, register_part


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    """down(silu(gate(h)) * up(h)) without biases, silu(z) = z / (1 + exp(-z)) in 32-bit
    (v1/models/qwen2-7b/inference_fp16.dag:333-337,
    v1/tensortype/cuda_kernels/silu_product.cu:15-17).  Gate and up are one product over
    the rows of the two matrices interleaved in runs of 8 (``ops.interleave_gate_up``), so
    that the activation can be formed in the product's epilogue."""

    graph_safe = True

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation '{spec.activation}' is not built; known: silu")

    def param_specs(self):
        s, p = self.spec, self.prefix
        g, u, d = s.names
        return {
            f"{p}{g}.weight": ParamSpec((s.inter, s.hidden)),
            f"{p}{u}.weight": ParamSpec((s.inter, s.hidden)),
            f"{p}{d}.weight": ParamSpec((s.hidden, s.inter)),
        }

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        g, u, d = s.names
        mats = [rt.param(get(f"{p}{n}.weight")) for n in (g, u)]
        if mats[0].dtype != mats[1].dtype:
            mats = [m.float() for m in mats]
        self.w_gate_up = rt.ops.interleave_gate_up(mats[0], mats[1])
        del mats
        self.w_down = rt.param(get(f"{p}{d}.weight"))

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() * self.w_gate_up.element_size()
                + self.w_down.numel() * self.w_down.element_size())

    def first_product(self):
        return self.rt.ops.product_hint(self.w_gate_up, "silu_mul")

    def forward(self, h, ctx):
        s, ops = self.spec, self.rt.ops
        T = h.shape[0]
        act = torch.empty((T, s.inter), dtype=h.dtype, device=h.device)
        ops.linear_silu_mul(h, self.w_gate_up, act, then=ops.product_hint(self.w_down, "stream"))
        return ops.linear_to_stream(act, self.w_down, None, then=self.then)
