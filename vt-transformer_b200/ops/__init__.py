"""The kernels as Python functions over torch tensors.

Every function runs a hand-written sm_100a kernel of ``csrc`` (or, for the bfloat16
matrix products of large batches, the library product that vt-transformer's engine also
uses: cuBLASLt, v1/tensortype/cuda_kernels/lt_sgemm.cu:55-126).  There is no CPU path and
no fallback: if the extension cannot be loaded or built, the first call raises.

``backend()`` returns the extension module.  Tests of the host-side logic may put an
object with the same functions in its place (``use_backend``); nothing in the package
does.
"""
from __future__ import annotations

from typing import Optional

import torch

_backend = None
launches = 0          # kernels of this package enqueued so far (one for each call below)


def backend():
    global _backend
    if _backend is None:
        if not torch.cuda.is_available():
            raise RuntimeError("vt_transformer_b200 runs on a CUDA device (B200, sm_100a) only; "
                               "torch.cuda.is_available() is False and there is no CPU path")
        from ..csrc import build
        _backend = build.load()
    return _backend


def use_backend(obj) -> None:
    """Replaces the kernel module (for tests of the host-side logic).  ``None`` restores
    the real one at the next call."""
    global _backend
    _backend = obj


# --------------------------------------------------------------------------- elementwise


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status=None) -> torch.Tensor:
    backend().embedding(table, ids, out, status)
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None, status=None) -> torch.Tensor:
    backend().rmsnorm(x, delta, weight, float(eps), out, rows, status)
    return out


def silu_mul(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    backend().silu_mul(gu, out)
    return out


def rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads: int, kv_heads: int,
               head_dim: int, store: bool = True, status=None) -> None:
    backend().rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads, kv_heads,
                         head_dim, bool(store), status)


# --------------------------------------------------------------------------- matrix products


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, status=None) -> torch.Tensor:
    """out[T, N] = x[T, K] w[N, K]^T (+ bias).  ``out`` is float32 or the dtype of x.

    float32 x and w: the 32-bit kernel (FFMA in a fixed order, no TF32).  A weight kept in
    32-bit beside bfloat16 activations goes the same way, with x widened.  bfloat16: the
    tcgen05 kernel (TMA, tensor memory), with w as the 128-row operand for up to 64 rows of x
    and x beyond.
    """
    be = backend()
    if w.dtype == torch.float32:
        xf = x if x.dtype == torch.float32 else x.float()
        if out.dtype == torch.float32:
            be.gemm_simt(xf, w, bias, out)
        else:
            tmp = torch.empty(out.shape, dtype=torch.float32, device=out.device)
            be.gemm_simt(xf, w, bias, tmp)
            out.copy_(tmp)
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError(f"linear: unsupported dtypes x {x.dtype}, w {w.dtype}")
    m = x.shape[0]
    if m <= SKINNY_MAX_ROWS and SMALL_BATCH_KERNEL == "skinny":
        be.gemm_skinny(x, w, bias, out)
    else:
        scratch, counters = _split_workspace(x.device)
        be.gemm_tc(x, w, bias, out, status, scratch, counters)
    return out


_workspaces = {}


def _split_workspace(device):
    """Scratch and arrival counters with which the tcgen05 kernel cuts k over CTAs for small batches:
    4M floats and 4,096 counters a device, made once.  Launches that use them run in one stream."""
    ws = _workspaces.get(device)
    if ws is None:
        ws = (torch.empty(4 << 20, dtype=torch.float32, device=device), torch.zeros(4096, dtype=torch.int32, device=device))
        _workspaces[device] = ws
    return ws


SKINNY_MAX_ROWS = 64            # rows of x up to which the small-batch kernel may run
# "tc": the tcgen05 kernel with w as the 128-row operand; "skinny": mma.sync weight streaming.
# The environment variable VTB200_SMALL_BATCH_KERNEL overrides it (for measurements).
import os as _os
SMALL_BATCH_KERNEL = _os.environ.get("VTB200_SMALL_BATCH_KERNEL", "tc")
ATTENTION_KERNEL = "auto"   # "auto", or "simt" to force the plain kernel (tests compare the two)


# --------------------------------------------------------------------------- attention


def _attention_tiles(ctx, tokens_per_tile: int, device):
    """(sequence, first token) for every tile of the step: each sequence's new tokens in runs of
    ``tokens_per_tile``.  Built once a step and kept in ``ctx.extras``."""
    key = ("attention_tiles", tokens_per_tile)
    tiles = ctx.extras.get(key)
    if tiles is None:
        pairs = [(i, a) for i, s in enumerate(ctx.seqs) for a in range(0, s.length, tokens_per_tile)]
        host = torch.tensor(pairs, dtype=torch.int32).view(-1, 2)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        tiles = host.to(device, non_blocking=True)
        ctx.extras[key] = tiles
    return tiles


def paged_attention(qkv, out, k_cache, v_cache, ctx, block_table, heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float, status=None) -> torch.Tensor:
    """Attention of the step's tokens over the paged keys and values of their sequences.
    ``ctx`` is the step's ``StepContext``.  bfloat16 runs on the tensor cores where the kernel
    takes the sizes (head_dim a multiple of 16 up to 128): single-token steps with the keys of a
    sequence split over several CTAs, other steps in tiles of 64 rows of (token, head of the
    group).  Everything else, and all of float32, runs the plain kernel."""
    be = backend()
    w = int(window) if window else 0
    group = heads // kv_heads
    if qkv.dtype == torch.bfloat16 and ATTENTION_KERNEL == "auto":
        if ctx.max_q_len == 1 and be.attention_mma_supports(head_dim, heads, kv_heads, 1):
            span = ctx.max_kv_len if not w else min(ctx.max_kv_len, w + 63)
            n_blocks = max(1, -(-span // 64))
            splits = max(1, min(n_blocks, -(-DECODE_TARGET_CTAS // (ctx.n_seqs * kv_heads)), 32))
            part_o = part_ml = None
            if splits > 1:
                part_o = torch.empty((splits, ctx.n_tokens, heads, head_dim), dtype=torch.float32, device=qkv.device)
                part_ml = torch.empty((splits, ctx.n_tokens, heads, 2), dtype=torch.float32, device=qkv.device)
            be.attention_mma(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, None, heads, kv_heads,
                             head_dim, w, float(scale), 1, splits, part_o, part_ml, status)
            return out
        if be.attention_mma_supports(head_dim, heads, kv_heads, 4):
            tiles = _attention_tiles(ctx, 64 // group, qkv.device)
            be.attention_mma(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, tiles, heads, kv_heads,
                             head_dim, w, float(scale), 4, 1, None, None, status)
            return out
    be.attention_simt(qkv, out, k_cache, v_cache, ctx.positions, ctx.token_seq, block_table, heads, kv_heads,
                      head_dim, w, float(scale), status)
    return out


DECODE_TARGET_CTAS = 444    # three one-warp CTAs of the split-key kernel fit an SM (shared memory), 148 SMs


# --------------------------------------------------------------------------- sampling


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    backend().argmax(logits, out)
    return out


def sample(logits, temperature, top_k, top_p, u, out) -> torch.Tensor:
    backend().sample(logits, temperature, top_k, top_p, u, out)
    return out


def _counted(fn):
    import functools

    @functools.wraps(fn)
    def wrapper(*a, **k):
        global launches
        launches += 1
        return fn(*a, **k)
    return wrapper


for _name in ("embedding", "rmsnorm", "silu_mul", "rope_store", "linear", "paged_attention", "argmax", "sample"):
    globals()[_name] = _counted(globals()[_name])
