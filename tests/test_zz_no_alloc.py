"""The entry point that allocates nothing (csrc/attention_noalloc.h), called as a program without
torch would call it: through its exported C symbol, with plain device pointers.  It must give what
the ordinary entry point gives, on calls in a row that share its fixed scratch array, and both must
give what the plain attention (float64, no pages, no runs) gives.

This file is collected last, so that a run that stops at the first failure has run every other
test before it."""
import ctypes
import math

import pytest
import torch

from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def library():
    from vt_transformer_b200 import ops
    from vt_transformer_b200.csrc import build
    ops.backend()                                   # builds the library if it is not built yet
    lib = ctypes.CDLL(build.find_built())
    fn = lib.vtb_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    return fn


def case(seed, seq_lens, heads, kv_heads, d, page_size, sharp=3.0):
    """Queries, and keys and values scattered over shuffled pages whose unused rows hold NaN.  Queries and keys are
    scaled up so that the scores are sharp: each query attends to a few keys of its own, near or far, and a key
    read from the wrong place, or a run merged with the wrong weight, moves the result by far more than the
    tolerance (flat scores of random numbers would average such a fault away).  Returns the device tensors and the
    dense keys and values (float64, per sequence) for the plain computation."""
    g = torch.Generator().manual_seed(seed)
    n = len(seq_lens)
    max_pages = max(-(-s // page_size) for s in seq_lens)
    n_pages = sum(-(-s // page_size) for s in seq_lens) + 3
    k_cache = torch.full((n_pages, kv_heads, page_size, d), float("nan")).to(torch.bfloat16)
    v_cache = torch.full((n_pages, kv_heads, page_size, d), float("nan")).to(torch.bfloat16)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n, max_pages), -1, dtype=torch.int32)
    dense = []
    for i, s in enumerate(seq_lens):
        k = (torch.randn(s, kv_heads, d, generator=g) * sharp ** 0.5).to(torch.bfloat16)
        v = torch.randn(s, kv_heads, d, generator=g).to(torch.bfloat16)
        dense.append((k.double(), v.double()))
        for p in range(-(-s // page_size)):
            page = order.pop()
            table[i, p] = page
            cnt = min(page_size, s - p * page_size)
            k_cache[page, :, :cnt] = k[p * page_size:p * page_size + cnt].transpose(0, 1)
            v_cache[page, :, :cnt] = v[p * page_size:p * page_size + cnt].transpose(0, 1)
    q = (torch.randn(n, heads, d, generator=g) * sharp ** 0.5).to(torch.bfloat16)
    qkv = torch.cat([q.view(n, -1), torch.full((n, 2 * kv_heads * d), float("nan")).to(torch.bfloat16)], dim=1).contiguous()
    cu_q = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    q_start = torch.tensor([s - 1 for s in seq_lens], dtype=torch.int32, device=DEV)
    return qkv.to(DEV), k_cache.to(DEV), v_cache.to(DEV), cu_q, q_start, table.to(DEV), q.double(), dense


def plain_rows(q, dense, window):
    """The plain implementation's attention (float64, whole sequences) for the last token of every sequence."""
    rows = []
    for i, (k, v) in enumerate(dense):
        n = k.shape[0]
        qq = torch.zeros(n, q.shape[1], q.shape[2], dtype=torch.float64)
        qq[n - 1] = q[i]
        rows.append(plain.attention(qq, k, v, window or None)[n - 1].reshape(-1))
    return torch.stack(rows)


# two calls in a row with different shapes and contents (the second finds the first one's scratch), then: a token
# whose position is window - 1, window and window + 1; tokens in the last slot of a page and in the first of the
# next; more runs than a sequence has blocks of keys (runs without keys); one run (no merge)
CASES = [(1, [700, 1, 64, 333], 28, 4, 128, 16, 0, 6),
         (2, [90, 513, 40, 17, 260, 129], 6, 2, 64, 32, 100, 3),
         (3, [99, 100, 101, 102, 300], 8, 2, 64, 16, 100, 4),
         (4, [16, 17, 32, 33, 64, 65, 128], 4, 4, 32, 16, 0, 2),
         (5, [5, 40, 70], 14, 2, 64, 16, 0, 16),
         (6, [250, 31], 7, 1, 128, 64, 0, 1)]


def test_no_alloc_entry_point_equals_the_ordinary_one_and_the_plain_attention():
    from vt_transformer_b200 import ops
    fn = library()
    be = ops.backend()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, seq_lens, heads, kv_heads, d, page_size, window, splits in CASES:
        qkv, kc, vc, cu_q, q_start, table, q, dense = case(seed, seq_lens, heads, kv_heads, d, page_size)
        n = len(seq_lens)
        scale = 1.0 / math.sqrt(d)
        ref = plain_rows(q, dense, window)
        flat = torch.stack([v[:, :, :].mean(dim=0)[torch.arange(heads) // (heads // kv_heads)].reshape(-1) for _, v in dense])
        assert float((ref - flat).abs().max()) > 0.5           # the scores are sharp: the result is no plain mean of v
        want = torch.empty(n, heads * d, dtype=torch.bfloat16, device=DEV)
        part_o = torch.empty(splits, n, heads, d, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(splits, n, heads, 2, dtype=torch.float32, device=DEV)
        be.attention_mma(qkv, want, kc, vc, cu_q, q_start, table, None, heads, kv_heads, d, window, scale, 1, splits,
                         part_o if splits > 1 else None, part_ml if splits > 1 else None, None)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = fn(qkv.data_ptr(), qkv.shape[1], got.data_ptr(), kc.data_ptr(), vc.data_ptr(), cu_q.data_ptr(),
                q_start.data_ptr(), table.data_ptr(), table.shape[1], n, kc.shape[0], heads, kv_heads, d, page_size,
                window, scale, splits, stream)
        torch.cuda.synchronize()
        assert rc == 0, seed
        # neither torch's allocator nor the driver has handed out memory: the device's free bytes are the same
        # (the first call of a process may load the kernel's code lazily, which the driver charges to the device)
        assert torch.cuda.memory_allocated() == before
        if seed != CASES[0][0]:
            assert torch.cuda.mem_get_info()[0] == free_before, seed
        assert torch.isfinite(got.float()).all(), seed
        # against the plain attention, within the tolerance of the kernel tests (four roundings of bfloat16)
        err = float((got.double().cpu() - ref).abs().max())
        bound = 4.0 / 256 * max(1.0, float(ref.abs().max()))
        assert err <= bound, (seed, err, bound)
        # against the ordinary entry point: the same kernels on the same inputs
        err = float((got.float() - want.float()).abs().max())
        assert err <= (1.0 / 256) * max(1.0, float(want.float().abs().max())), (seed, err)
        assert torch.equal(got, want), seed


def test_no_alloc_entry_point_refuses_what_it_cannot_hold_or_run():
    fn = library()
    qkv, kc, vc, cu_q, q_start, table, _, _ = case(3, [40, 50], 4, 2, 64, 16)
    out = torch.zeros(2, 4 * 64, dtype=torch.bfloat16, device=DEV)

    def call(n_seqs=2, heads=4, kv=2, d=64, splits=2, page_size=16, qkv_stride=None, table_stride=None, n_pages=None,
             null=None):
        ptr = dict(qkv=qkv.data_ptr(), out=out.data_ptr(), k=kc.data_ptr(), v=vc.data_ptr(), cu_q=cu_q.data_ptr(),
                   q_start=q_start.data_ptr(), table=table.data_ptr())
        if null:
            ptr[null] = None
        return fn(ptr["qkv"], qkv.shape[1] if qkv_stride is None else qkv_stride, ptr["out"], ptr["k"], ptr["v"], ptr["cu_q"],
                  ptr["q_start"], ptr["table"], table.shape[1] if table_stride is None else table_stride, n_seqs,
                  kc.shape[0] if n_pages is None else n_pages, heads, kv, d, page_size, 0, 0.125, splits, None)

    assert call(n_seqs=4096, heads=28, kv=4, d=128, splits=8, qkv_stride=4608) == 1     # 8 * 4096 * 28 * 130 floats: beyond the fixed array
    assert call(d=72) == 2                                              # a head size the kernel does not take
    assert call(splits=0) == 2 and call(splits=65) == 2                 # no runs, too many
    assert call(page_size=0) == 2 and call(page_size=-16) == 2 and call(page_size=24) == 2
    assert call(qkv_stride=4 * 64 - 1) == 2                             # a row too short for the queries
    assert call(table_stride=0) == 2 and call(n_pages=0) == 2
    assert call(heads=5, kv=2, qkv_stride=4608) == 2 and call(heads=40, kv=2, d=32, qkv_stride=4608) == 2  # heads no multiple of the KV heads; 20 heads a KV head
    for name in ("qkv", "out", "k", "v", "cu_q", "q_start", "table"):
        assert call(null=name) == 2, name
    assert call(n_seqs=0) == 0                                          # nothing to do
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0                       # a refused call touches nothing
