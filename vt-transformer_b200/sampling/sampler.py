"""Picks the next token of each request from the float32 logits of a step.

vt-transformer samples inside the engine with an argmax kernel or a top-3 kernel fed by
one host random number a step from mt19937(1979) for the whole batch
(v1/tensortype/cuda_tensor.cpp:997-1049, v1/tensortype/context.cpp:45).  Here sampling
stands above the step function, runs as one kernel launch over the rows of the logits
(``csrc/sampling.cu``), and the random number of a draw is a function of the request's
seed and the index of the output token.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .params import SamplingParams

_MASK = (1 << 64) - 1


def uniform(seed: int, index: int, stream: int = 0) -> float:
    """A number in [0, 1) from (seed, stream, index): splitmix64 finaliser, top 24 bits."""
    z = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + index * 0x94D049BB133111EB
         + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], indices: Sequence[int],
               streams: Sequence[int] = None) -> torch.Tensor:
        """``logits`` [rows, vocab] float32 on the device; row r belongs to a request with
        ``params[r]`` about to produce its output number ``indices[r]``.  Returns the token
        ids, int32 [rows], on the device."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if rows == 0:
            return out
        if all(p.is_greedy for p in params):
            self.ops.argmax(logits, out)
            return out
        streams = streams if streams is not None else [0] * rows
        host = torch.empty((4, rows), dtype=torch.float32, pin_memory=logits.is_cuda)
        for r, p in enumerate(params):
            host[0, r] = p.temperature if not p.is_greedy else 0.0
            host[1, r] = float(p.top_k)
            host[2, r] = p.top_p
            host[3, r] = uniform(p.seed, indices[r], streams[r])
        dev = host.to(logits.device, non_blocking=True)
        self.ops.sample(logits, dev[0].contiguous(), dev[1].to(torch.int32), dev[2].contiguous(),
                        dev[3].contiguous(), out)
        return out
