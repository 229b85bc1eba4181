"""Plain, slow implementation of the Qwen2 dense decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function for each part.  It shares no
code with the package: it reads config.json with ``json`` and the weights with the
``safetensors`` library, and computes with torch on the CPU in ``float64`` (or
``float32``) from the formulas of viitrix/vt-transformer's own files, cited at each
function by the file's path in that project.

vt-transformer's own model code cannot run on a CPU (every op of its host tensor
returns OP_TODO_ERROR, v1/tensortype/computing.hpp:32-150), so there is no golden output
of its whole forward pass to compare with.  What of it does run anchors the functions
below (tests/golden/, compared in tests/test_plain.py): the rotation table of
v1/tensortype/common.cpp:6-24, compiled on the CPU; and its CUDA kernels for the RMS norm,
the rotation, silu(a) * b, the causal mask and the samplers
(v1/tensortype/cuda_kernels/{rmsnorm,rotary_embed,silu_product,causal_mask,easy_sampling}.cu),
compiled unchanged and run once on a B200 on small seeded inputs.  The matrix products,
the softmax and the order of the parts in a layer rest on the formulas of the graph
(v1/models/qwen2-7b/inference_fp16.dag) and of v1/tensortype/cuda_tensor.cpp.

What vt-transformer does not have (a window on the keys, a run order that names
a layer twice or shares a cache) is defined here in the simplest way and marked.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- config


@dataclass
class PlainConfig:
    vocab: int
    hidden: int
    inter: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    eps: float
    theta: float
    max_pos: int
    tied: bool
    # window[i] is None for a layer that sees all keys, else the number of keys it sees
    window: List[Optional[int]] = field(default_factory=list)


def read_config(folder: str) -> PlainConfig:
    """The sizes and constants that v1/models/qwen2-7b/inference_fp16.dag:1-14 fixes
    in code, read from config.json instead."""
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    layers = c["num_hidden_layers"]
    heads = c["num_attention_heads"]
    window: List[Optional[int]] = [None] * layers
    if c.get("use_sliding_window", False) and c.get("sliding_window") is not None:
        first = c.get("max_window_layers", layers)
        for i in range(layers):
            if i >= first:
                window[i] = int(c["sliding_window"])
    return PlainConfig(
        vocab=c["vocab_size"], hidden=c["hidden_size"], inter=c["intermediate_size"],
        layers=layers, heads=heads, kv_heads=c.get("num_key_value_heads", heads),
        head_dim=c.get("head_dim", c["hidden_size"] // heads),
        eps=c["rms_norm_eps"], theta=c["rope_theta"],
        max_pos=c["max_position_embeddings"],
        tied=c.get("tie_word_embeddings", False), window=window)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    """Tensors by their names in the model folder; the names are those that
    v1/models/qwen2-7b/dump_from_huggingface.py:48-99 reads."""
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name).to(dtype)
    return out


# --------------------------------------------------------------------------- parts


def embed(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[t,:] = wte[id[t],:], no scaling (v1/tensortype/host_tensor.cpp:189-198)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """out = w * x * rsqrt(mean(x^2) + eps); the weight multiplies as it is
    (v1/tensortype/cuda_kernels/rmsnorm.cu:20-47)."""
    r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return w * x * r


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b), W stored [out, in] (v1/tensortype/cuda_tensor.cpp:507-566)."""
    y = x @ w.t()
    return y if b is None else y + b


def rotation_table(n_pos: int, dim: int, base: float):
    """cos and sin [n_pos, dim/2].  inv_freq[i] = float(1 / pow(base, 2i/dim)) computed
    in double and rounded to float; the angle is the float product pos * inv_freq; cos
    and sin of that float angle (v1/tensortype/common.cpp:6-24)."""
    base32 = float(torch.tensor(base, dtype=torch.float32))  # "float base" argument
    inv = torch.tensor([1.0 / math.pow(base32, (2.0 * i) / dim) for i in range(dim // 2)],
                       dtype=torch.float64).to(torch.float32)
    pos = torch.arange(n_pos, dtype=torch.float32)
    ang = (pos[:, None] * inv[None, :]).to(torch.float64)   # the float product, exactly
    return torch.cos(ang), torch.sin(ang)


def rotate(x: torch.Tensor, positions: Sequence[int], cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, n, d].  Pairs (i, i + d/2): out[i] = x[i] cos - x[i+d/2] sin,
    out[i+d/2] = x[i+d/2] cos + x[i] sin (v1/tensortype/cuda_kernels/rotary_embed.cu:19-29)."""
    p = torch.as_tensor(list(positions), dtype=torch.long)
    c = cos[p].to(x.dtype)[:, None, :]
    s = sin[p].to(x.dtype)[:, None, :]
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """q [T, nh, d], k and v [T, nkv, d], all at positions 0..T-1.  Head h reads KV
    head h // (nh / nkv) (v1/tensortype/cuda_kernels/transpose_0213.cu:93-105); scores
    q.k / sqrt(d) (v1/tensortype/cuda_tensor.cpp:730,761-773); key j is seen by row t if
    j <= t (v1/tensortype/cuda_kernels/causal_mask.cu:69-84); softmax over the keys
    (cuda_tensor.cpp:796-800); o = P V (cuda_tensor.cpp:869-881).
    Not in vt-transformer: with a window w, key j is seen only if also j > t - w."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    t_idx = torch.arange(T)
    seen = t_idx[None, :] <= t_idx[:, None]
    if window is not None:
        seen = seen & (t_idx[None, :] > t_idx[:, None] - window)
    for h in range(nh):
        s = (q[:, h, :] @ k[:, h // g, :].t()) / math.sqrt(d)
        s = s.masked_fill(~seen, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, h // g, :]
    return out


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(z) = z / (1 + exp(-z)), no biases
    (v1/models/qwen2-7b/inference_fp16.dag:333-337, v1/tensortype/cuda_kernels/silu_product.cu:15-17)."""
    gate = linear(x, w_gate)
    up = linear(x, w_up)
    return linear(gate / (1.0 + torch.exp(-gate)) * up, w_down)


# --------------------------------------------------------------------------- model


def layer_keys_values(cfg: PlainConfig, w: Dict[str, torch.Tensor], i: int, x: torch.Tensor, cos, sin):
    """Roped keys and raw values of layer i for its input x (the rows that
    v1/models/qwen2-7b/inference_fp16.dag:296-298,312-313 stores in the cache)."""
    T = x.shape[0]
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps)
    k = linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(T, cfg.kv_heads, cfg.head_dim)
    v = linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(T, cfg.kv_heads, cfg.head_dim)
    return rotate(k, range(T), cos, sin), v


def layer(cfg: PlainConfig, w: Dict[str, torch.Tensor], i: int, x: torch.Tensor, cos, sin,
          shared_kv=None) -> torch.Tensor:
    """One block in the order of v1/models/qwen2-7b/inference_fp16.dag:287-345:
    norm, q/k/v with bias, rotation of q and k, attention, o projection, residual,
    norm, feed-forward, residual.  Not in vt-transformer: with ``shared_kv`` the layer
    reads the given keys and values (another layer's cache) instead of its own."""
    T = x.shape[0]
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps)
    q = linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, cfg.heads, cfg.head_dim)
    q = rotate(q, range(T), cos, sin)
    if shared_kv is None:
        k, v = layer_keys_values(cfg, w, i, x, cos, sin)
    else:
        k, v = shared_kv
    o = attention(q, k, v, cfg.window[i] if cfg.window else None).reshape(T, cfg.heads * cfg.head_dim)
    x = x + linear(o, w[p + "self_attn.o_proj.weight"])
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.eps)
    f = swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return x + f


def forward(cfg: PlainConfig, w: Dict[str, torch.Tensor], ids: Sequence[int], order=None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence ``ids`` (v1/models/qwen2-7b/inference_fp16.dag:368-396).
    ``order`` (not in vt-transformer) is the list of runs; a run is a layer index, or a
    pair (layer, source run) whose layer reads the keys and values that run ``source``
    stored.  By default the layers run once each in their order."""
    dtype = w["model.embed_tokens.weight"].dtype
    cos, sin = rotation_table(max(cfg.max_pos, len(ids)), cfg.head_dim, cfg.theta)
    x = embed(w["model.embed_tokens.weight"], ids)
    runs = list(range(cfg.layers)) if order is None else list(order)
    stored = {}
    for n, run in enumerate(runs):
        if isinstance(run, (tuple, list)):
            i, source = run
            x = layer(cfg, w, i, x, cos, sin, shared_kv=stored[source])
        else:
            stored[n] = layer_keys_values(cfg, w, run, x, cos, sin)
            x = layer(cfg, w, run, x, cos, sin)
    x = rms_norm(x, w["model.norm.weight"], cfg.eps)
    head = w["model.embed_tokens.weight"] if cfg.tied or "lm_head.weight" not in w else w["lm_head.weight"]
    return linear(x, head).to(dtype)


# --------------------------------------------------------------------------- sampling


def sample_greedy(logits: torch.Tensor) -> int:
    """Largest logit (v1/tensortype/cuda_kernels/easy_sampling.cu:141-169); the lowest
    index wins a tie (the reference leaves ties to the order of its reduction)."""
    return int(torch.argmax(logits.double()))  # torch returns the first maximum


def uniform_from_counter(seed: int, request: int, index: int) -> float:
    """A uniform number in [0, 1) for output ``index`` of a request: splitmix64 of the
    three numbers, top 24 bits.  vt-transformer draws one host number a step from
    mt19937(1979) for the whole batch (v1/tensortype/context.cpp:45,
    cuda_tensor.cpp:1036-1037); a draw for each (request, index) keeps a request's tokens
    the same however it is batched."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + index * 0x94D049BB133111EB + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def kept_probabilities(logits: torch.Tensor, temperature: float, top_k: int = -1, top_p: float = 1.0) -> torch.Tensor:
    """Probabilities [vocab] after temperature, top-k and top-p, zero outside the kept set.
    The parameters are those of the front end (sglfront/sglfront/core.py:6-17).  The kept set:
    the top_k largest logits (values equal to the k-th are all kept; top_k <= 0 keeps all),
    then the smallest set of largest probabilities whose sum reaches top_p of the total (equal
    values again kept together)."""
    z = logits.double() / temperature
    e = torch.exp(z - z.max())
    if 0 < top_k < z.numel():
        kth = torch.topk(z, top_k).values[-1]
        e = torch.where(z >= kth, e, torch.zeros_like(e))
    if top_p < 1.0:
        vals = torch.sort(e[e > 0], descending=True).values
        need = top_p * float(vals.sum())
        c = torch.cumsum(vals, 0)
        n = int((c < need).sum()) + 1                      # the shortest head whose sum reaches `need`
        thr = vals[min(n, vals.numel()) - 1]
        e = torch.where(e >= thr, e, torch.zeros_like(e))
    return e / e.sum()


def sample(logits: torch.Tensor, temperature: float, u: float, top_k: int = -1, top_p: float = 1.0) -> int:
    """The first index, in index order, at which the running sum of the kept probabilities
    exceeds u (inverse CDF).  temperature <= 0 or top_k == 1 is the argmax."""
    if temperature <= 0 or top_k == 1:
        return sample_greedy(logits)
    p = kept_probabilities(logits, temperature, top_k, top_p)
    c = torch.cumsum(p, dim=-1)
    idx = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=torch.float64), right=True))
    return min(idx, logits.numel() - 1)


def sample_top3_reference(logits: torch.Tensor, temperature: float, u: float) -> int:
    """vt-transformer's own sampler, literally (v1/tensortype/cuda_kernels/easy_sampling.cu:32-104):
    logits / temperature, the three largest, softmax over those, then walk them from the
    third to the first and stop when the running sum reaches u.  It draws from the same
    distribution as ``sample(..., top_k=3)``; only the order of the walk differs."""
    vals, idxs = torch.topk(logits.double() / temperature, 3)   # descending
    p = torch.softmax(vals, dim=-1)
    s = 0.0
    for i in range(2, -1, -1):
        s += float(p[i])
        if s >= u:
            return int(idxs[i])
    return int(idxs[0])
