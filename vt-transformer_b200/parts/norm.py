"""RMS norm over the residual stream, with the residual sum folded in."""
from __future__ import annotations

import torch

from .base import Norm, ParamSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """out = w * v * rsqrt(mean(v^2) + eps) with v = x (+ delta), everything in 32-bit and
    one rounding at the end; the weight multiplies as it is, not as 1 + w
    (v1/tensortype/cuda_kernels/rmsnorm.cu:20-47).  ``prefix`` is the tensor's name
    without ".weight"."""

    graph_safe = True
    takes_shares = True        # the kernel adds a product's unadded shares while it reads them

    def param_specs(self):
        return {self.prefix + ".weight": ParamSpec((self.spec.size,), role="vector", init="one_plus_normal")}

    def load(self, get) -> None:
        self.weight = self.rt.param(get(self.prefix + ".weight"), "vector")

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x, delta=None, rows=None, status=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.rt.dtype, device=x.device)
        return self.rt.ops.rmsnorm(x, self.weight, self.spec.eps, out, delta=delta, rows=rows, status=status)
