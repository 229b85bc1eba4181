"""The arrangement of parts in a layer."""
from __future__ import annotations

from .base import Block, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))
    (the order of v1/models/qwen2-7b/inference_fp16.dag:287-345).  The two sums are formed
    in 32-bit inside the next norm (``ResidualStream``)."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        self.norm1 = build_part("norm", spec.norm1, prefix + spec.norm1_name, rt)
        self.norm2 = build_part("norm", spec.norm2, prefix + spec.norm2_name, rt)
        self.mixer = build_part("mixer", spec.mixer, prefix + spec.mixer_prefix, rt)
        self.ffn = build_part("feed_forward", spec.ffn, prefix + spec.ffn_prefix, rt)
        self.parts = (self.norm1, self.mixer, self.norm2, self.ffn)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def param_specs(self):
        out = {}
        for p in self.parts:
            out.update(p.param_specs())
        return out

    def load(self, get) -> None:
        for p in self.parts:
            p.load(get)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts)

    def first_product(self):
        return self.mixer.first_product()

    def link(self, then) -> None:
        self.mixer.then = self.ffn.first_product()
        self.ffn.then = then

    def forward(self, stream, ctx, cache):
        h = stream.normed(self.norm1)
        stream.add(self.mixer.forward(h, ctx, cache))
        h = stream.normed(self.norm2)
        stream.add(self.ffn.forward(h, ctx))
