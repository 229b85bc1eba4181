"""The kernels as Python functions over torch tensors.

Every function runs a hand-written sm_100a kernel of ``csrc``; the matrix products too (the
reference's engine calls cuBLASLt for them, v1/tensortype/cuda_kernels/lt_sgemm.cu:55-126; here
they are tcgen05 kernels of the package, and an FFMA kernel in 32-bit).  There is no CPU path and
no fallback: if the extension cannot be loaded or built, the first call raises.

``backend()`` returns the extension module.  Tests of the host-side logic may put an
object with the same functions in its place (``use_backend``); nothing in the package
does.
"""
from __future__ import annotations

import os
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


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status=None, scale: float = 1.0) -> torch.Tensor:
    """out[t] = scale * table[ids[t]] as float32 rows (id -1: a row of zeros)."""
    backend().embedding(table, ids, out, status, float(scale))
    return out


def logits_scale_cap(logits: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """logits = cap * tanh(scale * logits / cap) in place, in 32-bit; cap 0 applies the scale alone."""
    backend().logits_scale_cap(logits, float(scale), float(cap))
    return logits


class SplitSum:
    """The result [T, N] of a matrix product as the unadded 32-bit shares [shares, T, N] that the CTAs working
    on different parts of the inner dimension have left (``linear_to_stream``).  ``rmsnorm`` takes it as its
    delta and adds the shares, in the order of their index, while it reads them: the product's kernel is spared
    the merge of the shares at its end, and the delta reaches the 32-bit residual stream unrounded."""

    def __init__(self, shares: torch.Tensor):
        self.shares = shares

    @property
    def shape(self):
        return self.shares.shape[1:]

    @property
    def device(self):
        return self.shares.device

    def dense(self, dtype=None) -> torch.Tensor:
        """The sum as an ordinary tensor (tests, and parts that need one)."""
        total = self.shares[0].clone()
        for i in range(1, self.shares.shape[0]):
            total += self.shares[i]
        return total if dtype is None else total.to(dtype)


def dense(t, dtype=None) -> torch.Tensor:
    """``t`` as an ordinary tensor, whether it is one or a ``SplitSum``."""
    if isinstance(t, SplitSum):
        return t.dense(dtype)
    return t if dtype is None else t.to(dtype)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta=None,
            rows: Optional[torch.Tensor] = None, status=None) -> torch.Tensor:
    """out = weight * v * rsqrt(mean(v^2) + eps) over the rows ``rows`` (all) of v = x + delta, which is
    written back to x.  ``delta``: None, a tensor of out's dtype, or a ``SplitSum``."""
    if isinstance(delta, SplitSum):
        delta = delta.shares
    backend().rmsnorm(x, delta, weight, float(eps), out, rows, status)
    return out


def silu_mul(gu: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """out = silu(gate) * up.  ``interleave`` 0: gu = [gate | up]; 8: gate and up columns alternate in
    runs of 8 (``interleave_gate_up``)."""
    backend().silu_mul(gu, out, interleave)
    return out


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Packs the rows of the gate and up matrices [I, H] into one matrix [2 I, H] in runs of 8:
    g0..g7, u0..u7, g8..g15, u8..u15, ...  One product over it gives gate and up of the same 8
    features side by side, so that silu(gate) * up can be formed where the product's result lies
    (a thread's registers) and only [T, I] is written."""
    inter, hidden = w_gate.shape
    if inter % 8:
        raise ValueError(f"intermediate size {inter} must be a multiple of 8")
    return torch.stack([w_gate.view(inter // 8, 8, hidden), w_up.view(inter // 8, 8, hidden)], dim=1).reshape(
        2 * inter, hidden).contiguous()


# Bytes of the next product's weights that a weight-streaming product asks into L2 while it ends (0: none).
LOOK_AHEAD_BYTES = int(os.environ.get("VTB200_LOOK_AHEAD_BYTES", str(8 << 20)))
_PRODUCT_KINDS = {"linear": 0, "silu_mul": 1, "stream": 2}


def product_hint(w: torch.Tensor, kind: str):
    """What a part tells the product before one of its own: the matrix ``w`` [N, K] will be streamed next, by
    ``linear`` ("linear"), ``linear_silu_mul`` ("silu_mul") or ``linear_to_stream`` ("stream").  None for a
    matrix that the tcgen05 kernel does not take.  Passed as ``then=``; it changes no result."""
    if w is None or w.dtype != torch.bfloat16 or w.dim() != 2 or not w.is_cuda or not w.is_contiguous():
        return None
    return (w, _PRODUCT_KINDS[kind])


def _ahead(then) -> dict:
    if then is None or LOOK_AHEAD_BYTES <= 0:
        return {}
    return {"next_w": then[0], "next_epilogue": then[1], "next_bytes": LOOK_AHEAD_BYTES}


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, status=None, then=None) -> torch.Tensor:
    """out[T, I] = silu(x Wg^T) * (x Wu^T) for ``w_gate_up = interleave_gate_up(Wg, Wu)``.  bfloat16: one
    tcgen05 kernel whose epilogue forms the product from the 32-bit sums.  Otherwise the product
    into [T, 2 I] and the elementwise kernel."""
    be = backend()
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and FUSE_SILU and \
            not (x.shape[0] <= SKINNY_MAX_ROWS and SMALL_BATCH_KERNEL == "skinny"):
        scratch, counters = _split_workspace(x.device)
        global launches
        launches += 1
        be.gemm_tc(x, w_gate_up, None, out, status, scratch, counters, 1, **_ahead(then))
        return out
    gu = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
    linear(x, w_gate_up, None, gu, status)
    be.silu_mul(gu, out, 8)
    return out


FUSE_SILU = True    # False: always the separate elementwise kernel (tests compare the two)


def rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads: int, kv_heads: int,
               head_dim: int, store: bool = True, status=None) -> None:
    backend().rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads, kv_heads,
                         head_dim, bool(store), status)


# --------------------------------------------------------------------------- matrix products


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, status=None,
           then=None) -> torch.Tensor:
    """out[T, N] = x[T, K] w[N, K]^T (+ bias).  ``out`` is float32 or the dtype of x.  ``then``: the
    ``product_hint`` of the product that runs next, if the caller knows it.

    float32 x and w: the 32-bit kernel (FFMA in a fixed order, no TF32).  A weight kept in
    32-bit beside bfloat16 activations goes the same way, with x widened.  bfloat16: the
    tcgen05 kernel (TMA, tensor memory), with w as the 128-row operand for up to 256 rows of x
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
        be.gemm_tc(x, w, bias, out, status, scratch, counters, **_ahead(then))
    return out


STREAM_SHARES = os.environ.get("VTB200_STREAM_SHARES", "1") != "0"   # False: linear_to_stream always adds the shares itself


def linear_to_stream(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], status=None, then=None):
    """x w^T (+ bias) for a result that goes straight into the residual stream (``ResidualStream.add``): a
    tensor [T, N] of x's dtype, or, for bfloat16 batches small enough that the kernel cuts the inner dimension
    over CTAs, a ``SplitSum`` of the unadded 32-bit shares, which the next norm adds."""
    m = x.shape[0]
    # (a small matrix under a wide batch is faster with x as the 128-row operand and no shares: measured on a B200,
    # 256 rows by [1152, 896]: 21 us with shares, 15 us without; at 128 rows they are level)
    small_under_wide = m > 128 and w.shape[0] * w.shape[1] * 2 <= STREAM_SMALL_WEIGHT_BYTES
    if (STREAM_SHARES and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < m <= STREAM_MAX_ROWS
            and not small_under_wide and not (SMALL_BATCH_KERNEL == "skinny" and m <= SKINNY_MAX_ROWS)):
        be = backend()
        n, k = w.shape
        shares = torch.empty((be.gemm_tc_shares(m, n, k), m, n), dtype=torch.float32, device=x.device)
        global launches
        launches += 1
        be.gemm_tc(x, w, bias, shares, status, None, None, 2, **_ahead(then))
        return SplitSum(shares)
    out = torch.empty((m, w.shape[0]), dtype=x.dtype, device=x.device)
    return linear(x, w, bias, out, status, then)


_workspaces = {}


def _split_workspace(device):
    """Scratch and arrival counters with which the tcgen05 kernel cuts k over CTAs for small batches:
    8M floats and 4,096 counters a device, made once.  Launches that use them run in one stream."""
    ws = _workspaces.get(device)
    if ws is None:
        ws = (torch.empty(8 << 20, dtype=torch.float32, device=device), torch.zeros(4096, dtype=torch.int32, device=device))
        _workspaces[device] = ws
    return ws


SKINNY_MAX_ROWS = 64            # rows of x up to which the small-batch kernel may run
STREAM_MAX_ROWS = 256           # rows up to which w is the 128-row operand and products may leave their shares of k unadded
STREAM_SMALL_WEIGHT_BYTES = 8 << 20   # ... unless the matrix is this small and the batch has more than 128 rows
# "tc": the tcgen05 kernel with w as the 128-row operand; "skinny": mma.sync weight streaming.
# The environment variable VTB200_SMALL_BATCH_KERNEL overrides it (for measurements).
import os as _os
SMALL_BATCH_KERNEL = _os.environ.get("VTB200_SMALL_BATCH_KERNEL", "tc")
# "auto"; "mma": no tcgen05 attention (the mma.sync kernels only); "simt": the plain kernel (tests compare them)
ATTENTION_KERNEL = "auto"


# --------------------------------------------------------------------------- attention


def _attention_tiles(ctx, tokens_per_tile: int, device, first_seq: int = 0):
    """(sequence, first token) for every tile of the step: each sequence's new tokens in runs of
    ``tokens_per_tile``, ordered by falling number of keys; the sequences before ``first_seq`` are left out.
    Built once a step and kept in ``ctx.extras``."""
    key = ("attention_tiles", tokens_per_tile, first_seq)
    tiles = ctx.extras.get(key)
    if tiles is None:
        pairs = [(i, a) for i, s in enumerate(ctx.seqs) if i >= first_seq for a in range(0, s.length, tokens_per_tile)]
        # the tiles with the most keys first: the CTAs that start last are then the short ones
        pairs.sort(key=lambda p: -(ctx.seqs[p[0]].start + p[1]))
        host = torch.tensor(pairs, dtype=torch.int32).view(-1, 2)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        tiles = host.to(device, non_blocking=True)
        ctx.extras[key] = tiles
    return tiles


MIXED_STEP_MIN_SINGLES = 2    # single tokens at the head of a mixed step from which they get a launch of their own


def _leading_single_tokens(ctx) -> int:
    """How many entries at the head of the step bring one token each (0 if all do: that is no mixed step)."""
    n = 0
    for s in ctx.seqs:
        if s.length != 1:
            break
        n += 1
    return n if n < len(ctx.seqs) else 0


def single_token_step_is_one_kernel(ctx, dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether ``rope_attention`` will run rotation, cache store and attention of this step as one kernel: a
    bfloat16 step of single tokens at sizes the tensor-core kernel takes.  That kernel also takes q, k and v as
    the unadded shares of the product before it (``linear_to_stream``)."""
    return (dtype == torch.bfloat16 and ATTENTION_KERNEL in ("auto", "mma") and FUSE_ROPE and ctx.max_q_len == 1
            and ctx.n_tokens == ctx.n_seqs and backend().attention_mma_supports(head_dim, heads, kv_heads, 1))


def rope_attention(qkv, out, cos_sin, k_cache, v_cache, ctx, block_table, heads: int, kv_heads: int, head_dim: int,
                   window: Optional[int], scale: float, store: bool = True, status=None) -> torch.Tensor:
    """Rotation of q and k by the tokens' positions, store of k and v into their pages (if ``store``),
    and attention over the pages: the three steps of the attention mixer between its two products.
    In a bfloat16 step of single tokens they are one kernel (the attention kernel rotates q in its
    registers and puts the token's own k and v into its key block and into the page); otherwise the
    rotation kernel runs first.  ``qkv`` may be a ``SplitSum`` where ``single_token_step_is_one_kernel``."""
    global launches
    be = backend()
    shares = None
    if isinstance(qkv, SplitSum):
        if qkv.shares.shape[0] <= 8 and single_token_step_is_one_kernel(ctx, out.dtype, heads, kv_heads, head_dim):
            shares = qkv.shares
            qkv = torch.empty(tuple(qkv.shape), dtype=out.dtype, device=out.device)     # for its shape only
        else:
            qkv = qkv.dense(out.dtype)
    if single_token_step_is_one_kernel(ctx, qkv.dtype, heads, kv_heads, head_dim):
        launches += 1
        w = int(window) if window else 0
        span = ctx.max_kv_len if not w else min(ctx.max_kv_len, w + 31)
        splits, run, scratch = _decode_plan(ctx.n_seqs * kv_heads, span, qkv.device, getattr(ctx, "min_kv_len", 0))
        part_o = part_ml = counters = None
        if scratch or splits > 8:
            part_o = torch.empty((splits, ctx.n_tokens, heads, head_dim), dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty((splits, ctx.n_tokens, heads, 2), dtype=torch.float32, device=qkv.device)
            counters = _attention_counters(qkv.device, ctx.n_seqs * kv_heads)
        long_runs = _decode_long_runs(ctx.n_seqs * kv_heads, span, splits, run, head_dim, qkv.device)
        be.attention_decode(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, heads, kv_heads, head_dim, w,
                            float(scale), splits, part_o, part_ml, counters, True, cos_sin, bool(store), status, shares,
                            long_runs, run)
        return out
    rope_store(qkv, ctx.positions, cos_sin, k_cache, v_cache, ctx.token_seq, block_table, heads, kv_heads, head_dim,
               store=store, status=status)
    return paged_attention(qkv, out, k_cache, v_cache, ctx, block_table, heads, kv_heads, head_dim, window, scale,
                           status=status)


FUSE_ROPE = True    # False: always the separate rotation kernel (tests compare the two)


def paged_attention(qkv, out, k_cache, v_cache, ctx, block_table, heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float, status=None) -> torch.Tensor:
    """Attention of the step's tokens over the paged keys and values of their sequences.
    ``ctx`` is the step's ``StepContext``.  bfloat16 runs on the tensor cores where the kernel
    takes the sizes (head_dim a multiple of 16 up to 128; tcgen05 for prompt portions at 64 and 128): single-token steps with the keys of a
    sequence split over several CTAs, other steps in tiles of 64 or 128 rows of (token, head of
    the group).  Everything else, and all of float32, runs the plain kernel."""
    global launches
    be = backend()
    w = int(window) if window else 0
    group = heads // kv_heads
    if qkv.dtype == torch.bfloat16 and ATTENTION_KERNEL in ("auto", "mma"):
        if ctx.max_q_len == 1 and be.attention_mma_supports(head_dim, heads, kv_heads, 1):
            span = ctx.max_kv_len if not w else min(ctx.max_kv_len, w + 31)
            splits, run, scratch = _decode_plan(ctx.n_seqs * kv_heads, span, qkv.device, getattr(ctx, "min_kv_len", 0))
            part_o = part_ml = counters = None
            if scratch or splits > 8:
                part_o = torch.empty((splits, ctx.n_tokens, heads, head_dim), dtype=torch.float32, device=qkv.device)
                part_ml = torch.empty((splits, ctx.n_tokens, heads, 2), dtype=torch.float32, device=qkv.device)
                counters = _attention_counters(qkv.device, ctx.n_seqs * kv_heads)
            long_runs = _decode_long_runs(ctx.n_seqs * kv_heads, span, splits, run, head_dim, qkv.device)
            be.attention_decode(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, heads, kv_heads,
                                head_dim, w, float(scale), splits, part_o, part_ml, counters, long_runs=long_runs,
                                run_blocks=run)
            return out
        # portions long enough to fill tiles of 128 rows: the tcgen05 kernel where it takes the sizes
        if (ATTENTION_KERNEL == "auto" and ctx.max_q_len * group >= 128
                and be.attention_tc_supports(head_dim, heads, kv_heads) and k_cache.shape[2] % 16 == 0):
            # A mixed step: the single tokens at the head of the batch (a scheduler puts the decoding requests first)
            # would each be a tile of 128 rows with 7 of them live, its keys walked by one CTA.  They go to the
            # single-token kernel instead, which cuts their keys over CTAs; the two launches write disjoint rows.
            lead = _leading_single_tokens(ctx)
            if lead >= MIXED_STEP_MIN_SINGLES and be.attention_mma_supports(head_dim, heads, kv_heads, 1):
                longest = max(s.start + 1 for s in ctx.seqs[:lead])
                span = longest if not w else min(longest, w + 31)
                splits, run, scratch = _decode_plan(lead * kv_heads, span, qkv.device)
                part_o = part_ml = counters = None
                if scratch or splits > 8:
                    part_o = torch.empty((splits, lead, heads, head_dim), dtype=torch.float32, device=qkv.device)
                    part_ml = torch.empty((splits, lead, heads, 2), dtype=torch.float32, device=qkv.device)
                    counters = _attention_counters(qkv.device, lead * kv_heads)
                long_runs = _decode_long_runs(lead * kv_heads, span, splits, run, head_dim, qkv.device)
                launches += 1
                be.attention_decode(qkv[:lead], out[:lead], k_cache, v_cache, ctx.cu_q[:lead + 1], ctx.q_start[:lead],
                                    block_table[:lead], heads, kv_heads, head_dim, w, float(scale), splits, part_o, part_ml,
                                    counters, long_runs=long_runs, run_blocks=run)
            else:
                lead = 0
            tiles = _attention_tiles(ctx, 128 // group, qkv.device, first_seq=lead)
            be.attention_tc(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, tiles, heads, kv_heads,
                            head_dim, w, float(scale), status)
            return out
        # mma.sync tiles of 128 rows (8 warps) where the portions are long enough to fill them, else of 64
        warps = 8 if ctx.max_q_len * group >= 128 and be.attention_mma_supports(head_dim, heads, kv_heads, 8) else 4
        if be.attention_mma_supports(head_dim, heads, kv_heads, warps):
            tiles = _attention_tiles(ctx, (16 * warps) // group, qkv.device)
            be.attention_mma(qkv, out, k_cache, v_cache, ctx.cu_q, ctx.q_start, block_table, tiles, heads, kv_heads,
                             head_dim, w, float(scale), warps, 1, None, None, status)
            return out
    be.attention_simt(qkv, out, k_cache, v_cache, ctx.positions, ctx.token_seq, block_table, heads, kv_heads,
                      head_dim, w, float(scale), status)
    return out


_sm_counts = {}
_counters = {}


DECODE_BLOCK = 16         # keys in a block of the single-token attention kernel (one warp's unit of work)
# CTAs a step's attention aims at, in SMs (the fixed cost of a CTA against the spread of the work): where the runs of
# a sequence are a thread-block cluster, and where they meet in scratch memory
DECODE_CTAS_PER_SM = float(os.environ.get("VTB200_DECODE_CTAS_PER_SM", "0.65"))
DECODE_CTAS_PER_SM_LONG = float(os.environ.get("VTB200_DECODE_CTAS_PER_SM_LONG", "1.5"))
DECODE_MIN_RUN = int(os.environ.get("VTB200_DECODE_MIN_RUN", "8"))        # blocks below which a run of keys is not cut further
DECODE_MIN_RUN_LONG = int(os.environ.get("VTB200_DECODE_MIN_RUN_LONG", "32"))   # the same where the runs meet in scratch memory
DECODE_LONG_BOUND = int(os.environ.get("VTB200_DECODE_LONG_BOUND", "4096"))   # keys from which the runs meet in scratch memory


def _decode_plan(pairs: int, span: int, device, floor: int = 0):
    """How a single-token step's keys are cut over CTAs: (runs a sequence at most, blocks a run, whether the runs
    meet in scratch memory).  ``pairs``: sequences times KV heads; ``span``: the most keys a sequence of the step can
    hold (the bound of a captured graph).  A sequence takes about (its blocks / blocks a run) CTAs, so that
    sequences of different lengths give CTAs of like work; a step's typical sequence is taken to hold half the bound
    (a graph serves lengths between half its bound and the bound at the top, shorter ones below).

    Short bounds: the runs of a sequence are the CTAs of a thread-block cluster, which merge through shared memory;
    the cluster is sized for the typical sequence (a CTA without keys still has to be placed and to wait at the
    cluster's barriers, which costs the step more than a longer run does), and longer sequences get longer runs.
    Long bounds (the lengths of a step then differ by thousands of keys): as many runs as the longest sequence needs,
    met in scratch memory and merged by the CTA that arrives last; a CTA without keys leaves at once, a sequence of
    one run stores its result itself."""
    sms = _sm_counts.get(device)
    if sms is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _sm_counts[device] = sms
    blocks = max(1, -(-span // DECODE_BLOCK))
    typical = blocks / 2
    if blocks < 2 * DECODE_MIN_RUN:
        return 1, 0, False
    # ``floor``: a lower bound of the step's lengths.  Sequences of like lengths (all at least a quarter of the bound)
    # keep the cluster at any bound, if eight runs a sequence are CTAs enough: measured inside the step on a B200 (7B
    # sizes, every sequence at 3,000 to 30,000 keys), 4 to 32 sequences 3 to 14 % faster a step than through scratch
    # memory; one or two sequences, and sequences of very different lengths, are faster through scratch memory.
    like = floor > 0 and 4 * floor >= span and pairs >= 16
    if span < DECODE_LONG_BOUND or like:
        per_pair = DECODE_CTAS_PER_SM * sms / max(pairs, 1)
        if per_pair < 1.5:
            return 1, 0, False
        run = max(DECODE_MIN_RUN, int(-(-typical // per_pair)))
        splits = min(8, int(-(-typical // run)))
        return (splits, run, False) if splits > 1 else (1, 0, False)
    # (measured on a B200, every sequence at the bound: a run below 32 blocks costs a lone sequence of 8,192 keys a
    # third more (27 against 20 us), two of them twice (37 against 19); with few sequences, one CTA an SM with all
    # eight warps beats two with six (one sequence of 32,768 keys: 24 against 33 us))
    per_pair = DECODE_CTAS_PER_SM_LONG * sms / max(pairs, 1)
    run = max(DECODE_MIN_RUN_LONG, int(-(-typical // max(per_pair, 1.0))))
    splits = min(64, -(-blocks // run))
    if pairs * 16 <= sms:
        splits = min(splits, max(1, sms // pairs))
    return (splits, run, True) if splits > 1 else (1, 0, False)


# "auto" | "always" | "never": tensor-map boxes for the keys and values of single-token steps
DECODE_BOXES = os.environ.get("VTB200_DECODE_BOXES", "auto")
LONG_RUN_BLOCKS = 16     # blocks of 16 keys a warp from which the boxes pay where the CTAs run in one round


def _decode_long_runs(pairs: int, span: int, splits: int, run: int, head_dim: int, device) -> bool:
    """Whether a single-token step's keys and values come as boxes of a tensor map (head sizes 64 and 128):
    a box arrives later than a cp.async copy but costs the warp one instruction, not 32, so it pays where a
    warp streams many blocks (16 or more: 64 sequences of 4,096 keys, a step of 5.78 against 5.94 ms); it loses
    where a warp has few, however many CTAs there are (head size 128, 24 to 128 sequences of 1,040 keys: steps 0.2
    to 1.8 % slower with boxes, measured inside the step)."""
    if head_dim not in (64, 128) or DECODE_BOXES == "never":
        return False
    if DECODE_BOXES == "always":
        return True
    sms = _sm_counts.get(device, 148)
    if head_dim == 64 and pairs * splits > sms:
        # (blocks of half the bytes: the copies' 16 instructions a lane weigh more; 256 sequences of 512 keys at
        # 0.5B sizes: a step of 1.84 ms with boxes against 1.97)
        return True
    warps = 6 if pairs * splits > sms else 8            # the kernel's shape: two CTAs an SM, or one
    blocks = max(1, -(-span // DECODE_BLOCK))
    # (the bound is that of a captured graph: a typical sequence holds half of it, as in _decode_plan)
    return (run if run else blocks // 2) >= LONG_RUN_BLOCKS * warps


def _attention_counters(device, n: int) -> torch.Tensor:
    """Arrival counters of the decode attention's runs: zero, and left zero by every launch."""
    c = _counters.get(device)
    if c is None or c.numel() < n:
        c = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _counters[device] = c
    return c


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


for _name in ("embedding", "logits_scale_cap", "rmsnorm", "silu_mul", "rope_store", "linear", "paged_attention", "argmax", "sample"):  # the others count where they launch
    globals()[_name] = _counted(globals()[_name])
