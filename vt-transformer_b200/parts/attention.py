"""Grouped-query attention over a paged cache of keys and values."""
from __future__ import annotations

import math

import torch

from .base import KVCacheSpec, Mixer, ParamSpec, build_part, register_part


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    """q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv (one product over the packed rows of
    the three matrices, which equals the three separate products of
    v1/models/qwen2-7b/inference_fp16.dag:296,302,312 element for element); q and k are
    rotated by their positions (:297,:303); k and v go into the pages (:298,:313);
    softmax(q k^T / sqrt(d)) v over the keys the token may see (:307-318); then the o
    projection (:322).  All sizes come from the spec."""

    graph_safe = True

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.position.kind != "none" and spec.position.dim != spec.head_dim:
            # the rotation kernels turn the whole head, pairs (i, i + head_dim / 2), from a table [positions, head_dim / 2, 2]
            raise ValueError(f"attention: the position encoding covers {spec.position.dim} of the head's {spec.head_dim} "
                             f"dimensions; a rotation of part of the head is not built")
        self.position = build_part("position", spec.position, prefix, rt)
        self.q_dim = spec.heads * spec.head_dim
        self.kv_dim = spec.kv_heads * spec.head_dim
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)

    def cache_spec(self):
        return KVCacheSpec(self.spec.kv_heads, self.spec.head_dim, self.spec.window)

    def param_specs(self):
        s, p = self.spec, self.prefix
        q, k, v, o = s.names
        out = {
            f"{p}{q}.weight": ParamSpec((self.q_dim, s.hidden)),
            f"{p}{k}.weight": ParamSpec((self.kv_dim, s.hidden)),
            f"{p}{v}.weight": ParamSpec((self.kv_dim, s.hidden)),
            f"{p}{o}.weight": ParamSpec((s.hidden, self.q_dim)),
        }
        if s.qkv_bias:
            out[f"{p}{q}.bias"] = ParamSpec((self.q_dim,), role="vector")
            out[f"{p}{k}.bias"] = ParamSpec((self.kv_dim,), role="vector")
            out[f"{p}{v}.bias"] = ParamSpec((self.kv_dim,), role="vector")
        if s.out_bias:
            out[f"{p}{o}.bias"] = ParamSpec((s.hidden,), role="vector")
        return out

    def load(self, get) -> None:
        s, p, rt = self.spec, self.prefix, self.rt
        q, k, v, o = s.names
        mats = [rt.param(get(f"{p}{n}.weight")) for n in (q, k, v)]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        del mats
        self.b_qkv = (torch.cat([rt.param(get(f"{p}{n}.bias"), "vector") for n in (q, k, v)]).contiguous()
                      if s.qkv_bias else None)
        self.w_o = rt.param(get(f"{p}{o}.weight"))
        self.b_o = rt.param(get(f"{p}{o}.bias"), "vector") if s.out_bias else None
        self.position.load(get)

    def weight_bytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        for b in (self.b_qkv, self.b_o):
            if b is not None:
                n += b.numel() * b.element_size()
        return n

    def first_product(self):
        return self.rt.ops.product_hint(self.w_qkv, "stream")

    def forward(self, h, ctx, cache):
        s, ops = self.spec, self.rt.ops
        T = h.shape[0]
        after = ops.product_hint(self.w_o, "stream")
        if ops.single_token_step_is_one_kernel(ctx, h.dtype, s.heads, s.kv_heads, s.head_dim):
            qkv = ops.linear_to_stream(h, self.w_qkv, self.b_qkv, then=after)      # that kernel adds the shares of k itself
        else:
            qkv = torch.empty((T, self.q_dim + 2 * self.kv_dim), dtype=h.dtype, device=h.device)
            ops.linear(h, self.w_qkv, self.b_qkv, qkv, then=after)
        o = torch.empty((T, self.q_dim), dtype=h.dtype, device=h.device)
        ops.rope_attention(qkv, o, self.position.table, cache.k, cache.v, ctx, cache.block_table, s.heads, s.kv_heads,
                           s.head_dim, s.window, self.scale, store=cache.writes, status=ctx.status)
        return ops.linear_to_stream(o, self.w_o, self.b_o, then=self.then)
