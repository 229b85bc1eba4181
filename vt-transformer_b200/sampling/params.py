"""Sampling parameters of a request, with the names and defaults of vt-transformer's front
end (sglfront/sglfront/core.py:6-17)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass
class SamplingParams:
    """``temperature`` <= 0 (or ``top_k`` == 1) is greedy.  ``top_k`` <= 0 keeps the whole
    vocabulary.  ``seed`` feeds the request's own random numbers: output i of the request
    is drawn with a number that depends on (seed, i) only, so the tokens of a request do
    not change with the batch it runs in or with a pre-emption."""
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    ignore_eos: bool = False
    max_tokens: int = 1024
    seed: int = 0
    eos_token_ids: Optional[Tuple[int, ...]] = None   # None: the model's config decides

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, found {self.max_tokens}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must lie in (0, 1], found {self.top_p}")
