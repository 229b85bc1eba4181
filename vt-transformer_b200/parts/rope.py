"""Position encodings of attention: the rotation of pairs, or none."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_part


def rotation_table(max_positions: int, dim: int, base: float) -> torch.Tensor:
    """[max_positions, dim / 2, 2] of (cos, sin) in float32, built as vt-transformer builds
    its table (v1/tensortype/common.cpp:6-24): inv_freq[i] = 1 / pow(base, 2i / dim) in
    double, rounded to float; the angle is the float product position * inv_freq; cos and
    sin of that angle.  The pairing (i, i + dim/2) is the kernel's
    (v1/tensortype/cuda_kernels/rotary_embed.cu:19-29)."""
    base32 = torch.tensor(base, dtype=torch.float32).item()
    inv = torch.tensor([1.0 / math.pow(base32, (2.0 * i) / dim) for i in range(dim // 2)],
                       dtype=torch.float64).to(torch.float32)
    pos = torch.arange(max_positions, dtype=torch.float32)
    angle = (pos[:, None] * inv[None, :]).to(torch.float64)
    return torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).contiguous()


@register_part("position", "rotary")
class RotaryEmbedding(PositionEncoding):
    """Holds the (cos, sin) table on the device; one table for all layers of equal
    (dim, base, max_positions)."""

    _tables = {}

    def load(self, get) -> None:
        key = (self.spec.dim, float(self.spec.base), self.spec.max_positions, str(self.rt.device))
        table = RotaryEmbedding._tables.get(key)
        if table is None:
            table = rotation_table(self.spec.max_positions, self.spec.dim, self.spec.base).to(self.rt.device)
            RotaryEmbedding._tables[key] = table
        self.table = table


@register_part("position", "none")
class NoPosition(PositionEncoding):
    table = None

    def load(self, get) -> None:
        self.table = None
