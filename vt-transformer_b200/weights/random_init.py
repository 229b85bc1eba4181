"""Random-weights mode: writes a model folder from a configuration and a seed.

vt-transformer has no such mode (its weights come from a checkpoint dump,
v1/models/qwen2-7b/dump_from_huggingface.py).  The folder holds config.json and
model.safetensors with every tensor the model's parameter table names, in bfloat16, and
loads through the same path as a real checkpoint.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..config.base import ModelConfig
from ..config.registry import get_architecture
from ..parts.base import ParamSpec, Runtime
from . import safetensors_io as st
from .loader import random_tensor


def parameter_table(config: ModelConfig) -> Dict[str, ParamSpec]:
    """The tensors the architecture's model expects, from its spec alone (no device)."""
    from ..models.base import DecoderModel
    spec = get_architecture(config.architecture).model_spec(config)
    model = DecoderModel(spec, Runtime(device=torch.device("cpu"), dtype=torch.bfloat16, ops=None))
    return model.param_specs()


def write_random_model(config: ModelConfig, folder: str, seed: int = 0, sigma: float = 0.02) -> str:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``: matrices, embeddings
    and biases N(0, sigma), norm weights 1 + N(0, sigma), each tensor seeded by
    (seed, its name).  Returns the folder."""
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    table = {n: s for n, s in parameter_table(config).items() if not s.optional}
    layout = [(n, torch.int32 if s.role == "table" else torch.bfloat16, tuple(s.shape)) for n, s in table.items()]

    def tensors():
        for name, spec in table.items():
            yield name, random_tensor(name, spec, seed, sigma)

    st.write_file(os.path.join(folder, "model.safetensors"), tensors(), layout,
                  metadata={"format": "pt", "seed": seed, "sigma": sigma})
    return folder
