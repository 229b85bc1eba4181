"""The entry point that allocates nothing (csrc/attention_noalloc.h), called as a program without
torch would call it: through its exported C symbol, with plain device pointers.  It must give what
the ordinary entry point gives, on two calls in a row that share its fixed scratch array.

This file is collected last, so that a run that stops at the first failure has run every other
test before it."""
import ctypes
import math

import pytest
import torch

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


def case(seed, seq_lens, heads, kv_heads, d, page_size):
    """Random queries, and keys and values scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    n = len(seq_lens)
    max_pages = max(-(-s // page_size) for s in seq_lens)
    n_pages = sum(-(-s // page_size) for s in seq_lens) + 3
    k_cache = torch.randn(n_pages, kv_heads, page_size, d, generator=g).to(torch.bfloat16).to(DEV)
    v_cache = torch.randn(n_pages, kv_heads, page_size, d, generator=g).to(torch.bfloat16).to(DEV)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n, max_pages), -1, dtype=torch.int32)
    for i, s in enumerate(seq_lens):
        for p in range(-(-s // page_size)):
            table[i, p] = order.pop()
    qkv = (torch.randn(n, (heads + 2 * kv_heads) * d, generator=g) * 2).to(torch.bfloat16).to(DEV)
    cu_q = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    q_start = torch.tensor([s - 1 for s in seq_lens], dtype=torch.int32, device=DEV)
    return qkv, k_cache, v_cache, cu_q, q_start, table.to(DEV)


def test_no_alloc_entry_point_equals_the_ordinary_one_twice_in_a_row():
    from vt_transformer_b200 import ops
    fn = library()
    be = ops.backend()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes and contents: the second finds the first one's scratch
    for seed, seq_lens, heads, kv_heads, d, page_size, window, splits in (
            (1, [700, 1, 64, 333], 28, 4, 128, 16, 0, 6),
            (2, [90, 513, 40, 17, 260, 129], 6, 2, 64, 32, 100, 3)):
        qkv, kc, vc, cu_q, q_start, table = case(seed, seq_lens, heads, kv_heads, d, page_size)
        n = len(seq_lens)
        scale = 1.0 / math.sqrt(d)
        want = torch.empty(n, heads * d, dtype=torch.bfloat16, device=DEV)
        part_o = torch.empty(splits, n, heads, d, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(splits, n, heads, 2, dtype=torch.float32, device=DEV)
        be.attention_mma(qkv, want, kc, vc, cu_q, q_start, table, None, heads, kv_heads, d, window, scale, 1, splits,
                         part_o, part_ml, None)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(qkv.data_ptr(), qkv.shape[1], got.data_ptr(), kc.data_ptr(), vc.data_ptr(), cu_q.data_ptr(),
                q_start.data_ptr(), table.data_ptr(), table.shape[1], n, kc.shape[0], heads, kv_heads, d, page_size,
                window, scale, splits, stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        # the same kernel on the same inputs: within the tolerance of the kernel tests (it is equal bit for bit)
        err = float((got.float() - want.float()).abs().max())
        assert err <= (1.0 / 256) * max(1.0, float(want.float().abs().max())), err
        assert torch.equal(got, want)


def test_no_alloc_entry_point_refuses_what_it_cannot_hold_or_run():
    fn = library()
    qkv, kc, vc, cu_q, q_start, table = case(3, [40, 50], 4, 2, 64, 16)
    out = torch.zeros(2, 4 * 64, dtype=torch.bfloat16, device=DEV)
    args = lambda n_seqs, heads, kv, d, splits: (qkv.data_ptr(), qkv.shape[1], out.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                 cu_q.data_ptr(), q_start.data_ptr(), table.data_ptr(), table.shape[1], n_seqs,
                                                 kc.shape[0], heads, kv, d, 16, 0, 0.125, splits, None)
    assert fn(*args(4096, 28, 4, 128, 8)) == 1          # 8 * 4096 * 28 * 130 floats: beyond the fixed array
    assert fn(*args(2, 4, 2, 72, 2)) == 2               # a head size the kernel does not take
    assert fn(*args(2, 4, 2, 64, 0)) == 2               # no runs
    assert fn(*args(0, 4, 2, 64, 2)) == 0               # nothing to do
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0       # a refused call touches nothing
