"""Each kernel alone against a plain float64 computation of the same op (the plain
implementation's functions where it has one), at sizes other than the engine's tests use."""
import math
import random

import pytest
import torch

from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    # one rounding of the result: 2^-24 relative in 32-bit (sums of a few hundred terms: 1e-5), 2^-9 in bfloat16
    return (2e-5 if dtype == torch.float32 else 1.0 / 256) * scale


def close(got, ref, dtype, roundings=1.0):
    """|got - ref| within `roundings` roundings of the dtype at the scale of the reference."""
    ref = ref.double()
    err = float((got.double().cpu() - ref).abs().max())
    bound = tol(dtype, roundings) * max(1.0, float(ref.abs().max()))
    assert err <= bound, f"error {err:.3e} above {bound:.3e}"


@pytest.fixture(params=["never", "always"])
def key_fetch(request):
    """Single-token steps fetch keys and values by cp.async or, at head sizes 64 and 128, as boxes of a tensor
    map; the engine chooses by the length of the contexts, the tests run both."""
    from vt_transformer_b200 import ops as o
    old = o.DECODE_BOXES
    o.DECODE_BOXES = request.param
    yield request.param
    o.DECODE_BOXES = old


def ops():
    from vt_transformer_b200 import ops as o
    return o


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    torch.manual_seed(0)
    table = torch.randn(1000, 200, device=DEV).to(dtype)
    ids = torch.tensor([0, 999, 5, 5, 123, -1], dtype=torch.int32, device=DEV)
    out = torch.full((6, 200), 7.0, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    ops().embedding(table, ids, out, status=status)
    ref = plain.embed(table.cpu().double(), [0, 999, 5, 5, 123])
    assert torch.equal(out[:5].cpu().double(), ref) and float(out[5].abs().sum()) == 0.0     # a negative id pads
    assert status.tolist() == [0, 0]
    ops().embedding(table, torch.tensor([1000], dtype=torch.int32, device=DEV), out[:1], status=status)
    assert status.tolist() == [1, 1000]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 1000, 3584, 8200])
def test_rmsnorm_with_residual_sum_and_rows(dtype, hidden):
    torch.manual_seed(1)
    T = 37
    x = torch.randn(T, hidden, device=DEV) * 3
    delta = torch.randn(T, hidden, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    ref_sum = x.cpu().double() + delta.cpu().double()
    out = torch.empty(T, hidden, device=DEV, dtype=dtype)
    x1 = x.clone()
    ops().rmsnorm(x1, w, 1e-5, out)                                                   # plain norm
    assert float((out.cpu().double() - plain.rms_norm(x.cpu().double(), w.cpu().double(), 1e-5)).abs().max()) <= tol(dtype, 8)
    assert torch.equal(x1, x)
    ops().rmsnorm(x1, w, 1e-5, out, delta=delta)                                      # with the sum
    assert float((x1.cpu().double() - ref_sum).abs().max()) <= 1e-6                   # the stream holds the 32-bit sum
    assert float((out.cpu().double() - plain.rms_norm(ref_sum, w.cpu().double(), 1e-5)).abs().max()) <= tol(dtype, 8)
    rows = torch.tensor([36, 0, 17], dtype=torch.int32, device=DEV)                   # some rows only, in that order
    x2, out2 = x.clone(), torch.empty(3, hidden, device=DEV, dtype=dtype)
    ops().rmsnorm(x2, w, 1e-5, out2, delta=delta, rows=rows)
    assert torch.equal(out2, out[rows.long()])
    assert torch.equal(x2[1], x[1]) and torch.equal(x2[17], x1[17])                   # other rows are untouched


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    torch.manual_seed(2)
    gu = (torch.randn(19, 2 * 344, device=DEV) * 4).to(dtype)
    out = torch.empty(19, 344, device=DEV, dtype=dtype)
    ops().silu_mul(gu, out)
    g, u = gu[:, :344].cpu().double(), gu[:, 344:].cpu().double()
    ref = g / (1 + torch.exp(-g)) * u
    close(out, ref, dtype, 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 40, 64), (77, 130, 200), (64, 64, 16), (5, 301, 72), (200, 1000, 344)])
def test_gemm_simt(dtype, m, n, k):
    torch.manual_seed(3)
    a = torch.randn(m, k, device=DEV).to(dtype)
    w = torch.randn(n, k, device=DEV).to(dtype)
    bias = torch.randn(n, device=DEV)
    ref = plain.linear(a.cpu().double(), w.cpu().double(), bias.cpu().double())
    for out_dtype in {dtype, torch.float32}:
        c = torch.empty(m, n, device=DEV, dtype=out_dtype)
        ops().linear(a, w, bias, c)
        close(c, ref, out_dtype, 3 if out_dtype == torch.bfloat16 else 40)
        ops().linear(a, w, None, c)
        close(c, ref - bias.cpu().double(), out_dtype, 3 if out_dtype == torch.bfloat16 else 40)
        if dtype == torch.bfloat16:                       # the plain twin itself, whatever `linear` picks
            ops().backend().gemm_simt(a, w, bias, c)
            close(c, ref, out_dtype, 2 if out_dtype == torch.bfloat16 else 40)


def test_gemm_f32_is_a_true_32_bit_product_and_does_not_depend_on_the_batch():
    torch.manual_seed(4)
    a = torch.randn(50, 256, device=DEV)
    w = torch.randn(96, 256, device=DEV)
    c = torch.empty(50, 96, device=DEV)
    ops().linear(a, w, None, c)
    ref = a.cpu().double() @ w.cpu().double().t()
    assert float((c.cpu().double() - ref).abs().max()) < 1e-4          # TF32 would be off by 1e-1 here
    one = torch.empty(1, 96, device=DEV)
    ops().linear(a[7:8].contiguous(), w, None, one)
    assert torch.equal(one[0], c[7])                                   # bit for bit, alone or in a batch of 50


def paged_cache(k, v, seq_lens, page_size, n_pages, dtype, seed=0):
    """Scatters dense keys and values [sum(seq_lens), kv_heads, d] into shuffled pages.
    Returns k_cache, v_cache [pages, kv_heads, page_size, d] and the block table."""
    rng = random.Random(seed)
    kv_heads, d = k.shape[1], k.shape[2]
    kc = torch.full((n_pages, kv_heads, page_size, d), float("nan"), device=DEV).to(dtype)
    vc = torch.full_like(kc, float("nan"))
    free = list(range(n_pages))
    rng.shuffle(free)
    max_pages = max(-(-n // page_size) for n in seq_lens)
    table = torch.full((len(seq_lens), max_pages), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(seq_lens):
        for p in range(-(-n // page_size)):
            page = free.pop()
            table[s, p] = page
            cnt = min(page_size, n - p * page_size)
            kc[page, :, :cnt] = k[at + p * page_size: at + p * page_size + cnt].transpose(0, 1).to(dtype)
            vc[page, :, :cnt] = v[at + p * page_size: at + p * page_size + cnt].transpose(0, 1).to(dtype)
        at += n
    return kc, vc, table.to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,page_size,window", [(6, 2, 80, 32, None), (5, 5, 16, 16, 7), (8, 1, 128, 64, 50),
                                                               (3, 3, 256, 16, None), (28, 4, 128, 16, None), (14, 2, 64, 16, 90),
                                                               (7, 7, 112, 16, None), (9, 3, 96, 48, 33)])
def test_attention_over_pages(dtype, heads, kv_heads, d, page_size, window):
    """Three sequences in shuffled pages: whole ones and a tail of queries of a longer one."""
    torch.manual_seed(5)
    seq_lens = [70, 33, 150]
    q_lens = [70, 1, 9]                       # the queries are the last q_len positions of each sequence
    total = sum(seq_lens)
    k = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    v = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    kc, vc, table = paged_cache(k, v, seq_lens, page_size, 12 * 64 // page_size, dtype)
    T = sum(q_lens)
    q = (torch.randn(T, heads, d, device=DEV) * 2).to(dtype)
    qkv = torch.cat([q.view(T, -1), torch.zeros(T, 2 * kv_heads * d, device=DEV, dtype=dtype)], dim=1).contiguous()
    import helpers
    ctx = helpers.step_context(q_lens, [n - ql for n, ql in zip(seq_lens, q_lens)], DEV)
    out = torch.empty(T, heads * d, device=DEV, dtype=dtype)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    ops().paged_attention(qkv, out, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d), status=status)
    assert status.tolist() == [0, 0]
    at_q = at_k = 0
    for n, ql in zip(seq_lens, q_lens):
        qq = torch.zeros(n, heads, d, dtype=torch.float64)
        qq[n - ql:] = q[at_q:at_q + ql].cpu().double()
        ref = plain.attention(qq, k[at_k:at_k + n].cpu().double(), v[at_k:at_k + n].cpu().double(), window)[n - ql:]
        close(out[at_q:at_q + ql].view(ql, heads, d), ref, dtype, 4)
        at_q, at_k = at_q + ql, at_k + n


@pytest.mark.parametrize("heads,kv_heads,d,page_size,window", [(28, 4, 128, 16, None), (8, 1, 128, 64, 200), (3, 3, 128, 16, None),
                                                               (12, 2, 128, 32, 129), (32, 1, 128, 16, None), (4, 2, 128, 128, None),
                                                               (14, 2, 64, 16, None), (8, 8, 64, 64, 100), (6, 1, 64, 32, None)])
def test_prompt_portions_on_tcgen05(heads, kv_heads, d, page_size, window):
    """Portions long enough for tiles of 128 rows run the tcgen05 kernel: many blocks of 128 keys, a portion
    that starts in the middle of a sequence and of a page, ends that are no multiple of 16, a window's edge
    inside a block.  The pages' unused rows hold NaN.  Compared with the plain implementation and with the
    mma.sync kernel."""
    import helpers
    from vt_transformer_b200 import ops as o
    dtype = torch.bfloat16
    torch.manual_seed(21)
    seq_lens = [700, 333, 1501, 130]
    q_lens = [700, 45, 261, 129]
    total = sum(seq_lens)
    k = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    v = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    kc, vc, table = paged_cache(k, v, seq_lens, page_size, 2800 // page_size + 8, dtype, seed=4)
    T = sum(q_lens)
    q = (torch.randn(T, heads, d, device=DEV) * 2).to(dtype)
    qkv = torch.cat([q.view(T, -1), torch.zeros(T, 2 * kv_heads * d, device=DEV, dtype=dtype)], dim=1).contiguous()
    ctx = helpers.step_context(q_lens, [n - ql for n, ql in zip(seq_lens, q_lens)], DEV)
    assert o.backend().attention_tc_supports(d, heads, kv_heads)
    out = torch.full((T, heads * d), float("nan"), device=DEV, dtype=dtype)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    o.paged_attention(qkv, out, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d), status=status)
    assert status.tolist() == [0, 0]
    other = torch.empty_like(out)
    o.ATTENTION_KERNEL = "mma"
    try:
        o.paged_attention(qkv, other, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d), status=status)
    finally:
        o.ATTENTION_KERNEL = "auto"
    at_q = at_k = 0
    for n, ql in zip(seq_lens, q_lens):
        qq = torch.zeros(n, heads, d, dtype=torch.float64)
        qq[n - ql:] = q[at_q:at_q + ql].cpu().double()
        ref = plain.attention(qq, k[at_k:at_k + n].cpu().double(), v[at_k:at_k + n].cpu().double(), window)[n - ql:]
        close(out[at_q:at_q + ql].view(ql, heads, d), ref, dtype, 4)
        close(other[at_q:at_q + ql].view(ql, heads, d), ref, dtype, 4)
        at_q, at_k = at_q + ql, at_k + n


@pytest.mark.parametrize("heads,kv_heads,d,page_size,window", [(28, 4, 128, 16, None), (6, 2, 80, 32, None), (4, 4, 16, 16, 40),
                                                               (16, 1, 64, 64, 100), (14, 2, 64, 16, None), (40, 2, 32, 16, None),
                                                               (8, 2, 128, 48, None), (14, 2, 128, 32, 90)])
def test_single_token_steps_split_the_keys(heads, kv_heads, d, page_size, window, key_fetch):
    """Every sequence brings one token (a decode step): the tensor-core kernel splits the keys of a
    sequence over several CTAs and merges the parts.  Sequences of very different lengths, one of a
    single token."""
    import helpers
    from vt_transformer_b200 import ops as o
    dtype = torch.bfloat16
    torch.manual_seed(9)
    seq_lens = [1, 700, 64, 65, 333, 16]
    total = sum(seq_lens)
    k = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    v = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    kc, vc, table = paged_cache(k, v, seq_lens, page_size, 1300 // page_size + 8, dtype, seed=3)
    T = len(seq_lens)
    q = (torch.randn(T, heads, d, device=DEV) * 2).to(dtype)
    qkv = torch.cat([q.view(T, -1), torch.zeros(T, 2 * kv_heads * d, device=DEV, dtype=dtype)], dim=1).contiguous()
    ctx = helpers.step_context([1] * T, [n - 1 for n in seq_lens], DEV)
    out = torch.empty(T, heads * d, device=DEV, dtype=dtype)
    o.paged_attention(qkv, out, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d))
    plain_out = torch.empty_like(out)
    o.ATTENTION_KERNEL = "simt"
    try:
        o.paged_attention(qkv, plain_out, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d))
    finally:
        o.ATTENTION_KERNEL = "auto"
    at = 0
    for i, n in enumerate(seq_lens):
        qq = torch.zeros(n, heads, d, dtype=torch.float64)
        qq[n - 1] = q[i].cpu().double()
        ref = plain.attention(qq, k[at:at + n].cpu().double(), v[at:at + n].cpu().double(), window)[n - 1]
        close(out[i].view(heads, d), ref, dtype, 4)
        close(plain_out[i].view(heads, d), ref, dtype, 4)
        at += n


def last_row_attention(q, k, v, window):
    """The plain attention's last row, q [heads, d] against all n keys: the plain function itself for short
    sequences; for long ones (whose n x n scores would take it seconds a head) its formula for that one row."""
    n, heads = k.shape[0], q.shape[0]
    if n <= 800:
        qq = torch.zeros(n, heads, q.shape[1], dtype=torch.float64)
        qq[n - 1] = q
        return plain.attention(qq, k, v, window)[n - 1]
    g = heads // k.shape[1]
    lo = max(0, n - window) if window else 0
    out = torch.empty_like(q)
    for h in range(heads):
        p = torch.softmax((k[lo:, h // g] @ q[h]) / math.sqrt(q.shape[1]), dim=0)
        out[h] = p @ v[lo:, h // g]
    return out


@pytest.mark.parametrize("heads,kv_heads,d,page_size,window", [(28, 4, 128, 64, None), (12, 2, 128, 16, None), (14, 2, 64, 32, None),
                                                               (6, 2, 80, 16, None), (8, 1, 128, 48, 3000)])
def test_single_token_steps_of_very_different_lengths_meet_in_scratch_memory(heads, kv_heads, d, page_size, window, key_fetch):
    """A step whose sequences hold from one key to thousands: under a long bound the keys are cut into runs of a
    fixed number of blocks, so the long sequences take many CTAs (whose results meet in scratch memory and are merged
    by the CTA that arrives last), the short ones one (which stores its result itself), and CTAs without keys leave
    at once.  Run twice: the arrival counters are left at zero."""
    import helpers
    from vt_transformer_b200 import ops as o
    dtype = torch.bfloat16
    torch.manual_seed(31)
    seq_lens = [5000, 64, 1, 4097, 700, 17, 2300, 129]
    total = sum(seq_lens)
    k = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    v = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    kc, vc, table = paged_cache(k, v, seq_lens, page_size, sum(-(-n // page_size) for n in seq_lens) + 5, dtype, seed=6)
    T = len(seq_lens)
    q = (torch.randn(T, heads, d, device=DEV) * 2).to(dtype)
    qkv = torch.cat([q.view(T, -1), torch.zeros(T, 2 * kv_heads * d, device=DEV, dtype=dtype)], dim=1).contiguous()
    ctx = helpers.step_context([1] * T, [n - 1 for n in seq_lens], DEV)
    splits, run, scratch = o._decode_plan(T * kv_heads, min(max(seq_lens), window + 31) if window else max(seq_lens), torch.device(DEV))
    assert scratch == (window is None) and splits > 1 and run > 0
    for _ in range(2):
        out = torch.full((T, heads * d), float("nan"), device=DEV, dtype=dtype)
        o.paged_attention(qkv, out, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d))
        at = 0
        for i, n in enumerate(seq_lens):
            ref = last_row_attention(q[i].cpu().double(), k[at:at + n].cpu().double(), v[at:at + n].cpu().double(), window)
            close(out[i].view(heads, d), ref, dtype, 4)
            at += n
    counters = o._counters.get(torch.device(DEV))
    assert counters is None or int(counters.abs().sum()) == 0


@pytest.mark.parametrize("heads,kv_heads,d,page_size,n_seqs,longest", [(28, 4, 128, 16, 50, 300), (8, 2, 64, 32, 90, 200),
                                                                        (14, 2, 128, 64, 40, 1500), (6, 2, 80, 16, 80, 100)])
def test_single_token_steps_with_more_ctas_than_sms(heads, kv_heads, d, page_size, n_seqs, longest, key_fetch):
    """Many sequences: more CTAs than SMs, so the kernel runs with three warps a CTA and two CTAs an SM
    (head sizes 64 and 128), alone or with the keys of a sequence cut into runs."""
    import helpers
    from vt_transformer_b200 import ops as o
    dtype = torch.bfloat16
    torch.manual_seed(13)
    rng = random.Random(5)
    seq_lens = [rng.randrange(1, longest) for _ in range(n_seqs - 1)] + [longest]
    total = sum(seq_lens)
    k = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    v = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    kc, vc, table = paged_cache(k, v, seq_lens, page_size, sum(-(-n // page_size) for n in seq_lens) + 3, dtype, seed=6)
    T = len(seq_lens)
    q = (torch.randn(T, heads, d, device=DEV) * 2).to(dtype)
    qkv = torch.cat([q.view(T, -1), torch.zeros(T, 2 * kv_heads * d, device=DEV, dtype=dtype)], dim=1).contiguous()
    ctx = helpers.step_context([1] * T, [n - 1 for n in seq_lens], DEV)
    out = torch.full((T, heads * d), float("nan"), device=DEV, dtype=dtype)
    o.paged_attention(qkv, out, kc, vc, ctx, table, heads, kv_heads, d, None, 1 / math.sqrt(d))
    at = 0
    for i, n in enumerate(seq_lens):
        if i % 7 == 0 or n == longest:            # the plain implementation is slow: a sample of the sequences
            qq = torch.zeros(n, heads, d, dtype=torch.float64)
            qq[n - 1] = q[i].cpu().double()
            ref = plain.attention(qq, k[at:at + n].cpu().double(), v[at:at + n].cpu().double(), None)[n - 1]
            close(out[i].view(heads, d), ref, dtype, 4)
        at += n
    assert not bool(torch.isnan(out.float()).any())


@pytest.mark.parametrize("heads,kv_heads,d,page_size,window", [(28, 4, 128, 64, None), (12, 2, 128, 16, 700), (14, 2, 64, 32, None)])
def test_keys_fetched_as_boxes_give_the_same_bits_as_copies(heads, kv_heads, d, page_size, window):
    """The two ways of bringing a decode step's keys and values into shared memory feed the same arithmetic:
    their outputs are equal bit for bit, with pages in a shuffled order and contexts that end anywhere in a page."""
    import helpers
    from vt_transformer_b200 import ops as o
    dtype = torch.bfloat16
    torch.manual_seed(21)
    rng = random.Random(8)
    seq_lens = [rng.randrange(900, 2300) for _ in range(47)] + [1, 33, 2304]
    total = sum(seq_lens)
    k = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    v = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    kc, vc, table = paged_cache(k, v, seq_lens, page_size, sum(-(-n // page_size) for n in seq_lens) + 5, dtype, seed=2)
    T = len(seq_lens)
    qkv = torch.randn(T, (heads + 2 * kv_heads) * d, device=DEV).to(dtype)
    ctx = helpers.step_context([1] * T, [n - 1 for n in seq_lens], DEV)
    outs = {}
    old = o.DECODE_BOXES
    try:
        for mode in ("never", "always"):
            o.DECODE_BOXES = mode
            out = torch.full((T, heads * d), float("nan"), device=DEV, dtype=dtype)
            o.paged_attention(qkv, out, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d))
            outs[mode] = out
    finally:
        o.DECODE_BOXES = old
    assert not bool(torch.isnan(outs["never"].float()).any())
    assert torch.equal(outs["never"], outs["always"])
    # the automatic choice takes boxes where a warp streams many blocks of a typical sequence (a bound of 8,192 keys)
    splits, run, _ = o._decode_plan(T * kv_heads, 8192, torch.device(DEV))
    assert o._decode_long_runs(T * kv_heads, 8192, splits, run, d, torch.device(DEV))


@pytest.mark.parametrize("heads,kv_heads,d,page_size,window,rotate", [(28, 4, 128, 16, None, True), (6, 2, 48, 32, 40, True),
                                                                      (4, 4, 16, 16, None, True), (8, 1, 64, 16, None, False),
                                                                      (24, 2, 64, 16, None, True), (9, 1, 128, 64, 70, True),
                                                                      (14, 2, 128, 64, 200, True)])
def test_single_token_step_rotates_and_stores_inside_the_attention_kernel(heads, kv_heads, d, page_size, window, rotate,
                                                                          key_fetch):
    """A decode step's rotation, cache store and attention as one kernel against the same as two kernels:
    the same output, the same page contents, for a run that writes the cache and for one that only reads."""
    import helpers
    from vt_transformer_b200 import ops as o
    from vt_transformer_b200.parts.rope import rotation_table
    dtype = torch.bfloat16
    torch.manual_seed(14)
    seq_lens = [1, 300, 64, 65, 33, 17]                   # the new token is the last of each
    total = sum(seq_lens)
    k = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    v = torch.randn(total, kv_heads, d, device=DEV).to(dtype)
    kc0, vc0, table = paged_cache(k, v, seq_lens, page_size, 700 // page_size + 8, dtype, seed=4)
    kc0, vc0 = torch.nan_to_num(kc0), torch.nan_to_num(vc0)
    T = len(seq_lens)
    qkv0 = torch.randn(T, (heads + 2 * kv_heads) * d, device=DEV).to(dtype)
    cs = rotation_table(400, d, 10000.0).to(DEV) if rotate else None
    ctx = helpers.step_context([1] * T, [n - 1 for n in seq_lens], DEV)
    results = {}
    for store in (True, False):
        for fused in (True, False):
            o.FUSE_ROPE = fused
            try:
                qkv, kc, vc = qkv0.clone(), kc0.clone(), vc0.clone()
                out = torch.empty(T, heads * d, device=DEV, dtype=dtype)
                status = torch.zeros(2, dtype=torch.int32, device=DEV)
                o.rope_attention(qkv, out, cs, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d), store=store,
                                 status=status)
                assert status.tolist() == [0, 0]
                results[(store, fused)] = (out, kc, vc)
            finally:
                o.FUSE_ROPE = True
        a, b = results[(store, True)], results[(store, False)]
        close(a[0], b[0].double().cpu(), dtype, 2)
        assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])          # the pages hold the same bits
        assert torch.equal(a[1], kc0) != store                               # and were written iff the run stores
    assert float((results[(True, True)][0].float() - results[(False, True)][0].float()).abs().max()) > 0.01
    # q, k and v as three unadded 32-bit shares that sum (in bfloat16) to the same values: the same output and pages
    parts = torch.randn(3, *qkv0.shape, device=DEV)
    parts[0] = qkv0.float() - parts[1] - parts[2]
    parts[0] += qkv0.float() - (parts[0] + parts[1] + parts[2])          # what rounding took
    assert torch.equal((parts[0] + parts[1] + parts[2]).to(dtype), qkv0)
    kc, vc = kc0.clone(), vc0.clone()
    out = torch.empty(T, heads * d, device=DEV, dtype=dtype)
    o.rope_attention(o.SplitSum(parts), out, cs, kc, vc, ctx, table, heads, kv_heads, d, window, 1 / math.sqrt(d), store=True)
    ref = results[(True, True)]
    assert torch.equal(out, ref[0]) and torch.equal(kc, ref[1]) and torch.equal(vc, ref[2])


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("n,k", [(40, 64), (301, 72), (1000, 344), (4608, 3584), (100, 18944)])
def test_weight_streaming_product(m, n, k):
    torch.manual_seed(10)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    ref = plain.linear(x.cpu().double(), w.cpu().double(), bias.cpu().double())
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(m, n, device=DEV, dtype=out_dtype)
        ops().backend().gemm_skinny(x, w, bias, out)
        close(out, ref, out_dtype, 2 if out_dtype == torch.bfloat16 else 40)
    out = torch.empty(m, n, device=DEV, dtype=torch.float32)
    ops().backend().gemm_skinny(x, w, None, out)
    close(out, ref - bias.cpu().double(), torch.float32, 40)


@pytest.mark.parametrize("m", [1, 8, 16, 17, 33, 64, 65, 128, 129, 300, 1000])
@pytest.mark.parametrize("n,k", [(40, 64), (301, 72), (344, 136), (1000, 344), (4608, 3584), (520, 18944), (3584, 3584)])
def test_tcgen05_product(m, n, k):
    """The tcgen05 kernel alone, in both orientations (w as the 128-row operand for up to 64 rows of x,
    x beyond), with tiles that hang over every edge, k that is no multiple of 64, and k cut over a cluster."""
    torch.manual_seed(11)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    ref = plain.linear(x.cpu().double(), w.cpu().double(), bias.cpu().double())
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    scratch, counters = ops()._split_workspace(torch.device(DEV))
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), float("nan"), device=DEV, dtype=out_dtype)
        ops().backend().gemm_tc(x, w, bias, out, status)                       # k in one piece
        close(out, ref, out_dtype, 2 if out_dtype == torch.bfloat16 else 40)
        for _ in range(2):                                                     # k cut over CTAs where that pays; twice:
            out.fill_(float("nan"))                                            # the counters must be back at zero
            ops().backend().gemm_tc(x, w, bias, out, status, scratch, counters)
            close(out, ref, out_dtype, 2 if out_dtype == torch.bfloat16 else 40)
    out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.float32)
    ops().backend().gemm_tc(x, w, None, out, status, scratch, counters)
    close(out, ref - bias.cpu().double(), torch.float32, 40)
    assert status.tolist() == [0, 0] and int(counters.abs().sum()) == 0


@pytest.mark.parametrize("m", [1, 8, 40, 64, 65, 300])
@pytest.mark.parametrize("inter,k", [(8, 64), (136, 72), (344, 128), (18944 // 8, 3584)])
def test_gate_up_product_with_the_activation_in_its_epilogue(m, inter, k):
    """silu(x Wg^T) * (x Wu^T) from one product over the interleaved rows, fused (tcgen05 epilogue) and
    in two kernels (product, then the elementwise kernel on the interleaved layout), in both dtypes of
    the elementwise kernel."""
    torch.manual_seed(13)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    wg = (torch.randn(inter, k, device=DEV) / math.sqrt(k) * 2).to(torch.bfloat16)
    wu = (torch.randn(inter, k, device=DEV) / math.sqrt(k) * 2).to(torch.bfloat16)
    g, u = x.cpu().double() @ wg.cpu().double().t(), x.cpu().double() @ wu.cpu().double().t()
    ref = g / (1 + torch.exp(-g)) * u
    o = ops()
    packed = o.interleave_gate_up(wg, wu)
    assert torch.equal(packed[:8], wg[:8]) and torch.equal(packed[8:16], wu[:8])
    fused = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    o.linear_silu_mul(x, packed, fused)
    close(fused, ref, torch.bfloat16, 2)
    o.FUSE_SILU = False
    try:
        two = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
        o.linear_silu_mul(x, packed, two)
    finally:
        o.FUSE_SILU = True
    close(two, ref, torch.bfloat16, 3)                       # gate and up are rounded to bfloat16 on the way
    xf, pf = x.float(), packed.float()
    out32 = torch.empty(m, inter, device=DEV)
    o.linear_silu_mul(xf, pf, out32)
    close(out32, ref, torch.float32, 40)


@pytest.mark.parametrize("m", [1, 8, 33, 64, 200])
@pytest.mark.parametrize("n,k", [(301, 72), (3584, 3584), (520, 18944)])
def test_asking_for_the_next_products_weights_changes_no_bit(m, n, k):
    """A product that is told which matrix streams next asks for its first boxes into L2 while it ends: the same
    bits with and without, whatever the next matrix is (smaller than a box, with edges that hang over, of another
    epilogue, far larger than what is asked for), and no status."""
    o = ops()
    be = o.backend()
    torch.manual_seed(23)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    scratch, counters = o._split_workspace(torch.device(DEV))
    nexts = [(torch.zeros(8, 8, device=DEV, dtype=torch.bfloat16), 0), (torch.zeros(130, 72, device=DEV, dtype=torch.bfloat16), 2),
             (torch.zeros(2 * 1000, 3584, device=DEV, dtype=torch.bfloat16), 1), (torch.zeros(3584, 18944, device=DEV, dtype=torch.bfloat16), 2)]
    ref = torch.empty(m, n, device=DEV, dtype=torch.float32)
    be.gemm_tc(x, w, bias, ref, status, scratch, counters)
    n_shares = be.gemm_tc_shares(m, n, k) if m <= 256 else 0
    ref_shares = torch.empty(n_shares, m, n, device=DEV, dtype=torch.float32)
    if n_shares:
        be.gemm_tc(x, w, bias, ref_shares, status, None, None, 2)
    for next_w, next_epilogue in nexts:
        for n_bytes in (16 << 10, 8 << 20, 1 << 30):
            out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.float32)
            be.gemm_tc(x, w, bias, out, status, scratch, counters, 0, next_w, next_epilogue, n_bytes)
            assert torch.equal(out, ref)
            if n_shares:
                shares = torch.full((n_shares, m, n), float("nan"), device=DEV, dtype=torch.float32)
                be.gemm_tc(x, w, bias, shares, status, None, None, 2, next_w, next_epilogue, n_bytes)
                assert torch.equal(shares, ref_shares)
    # through ops, with the hint as the parts pass it; a matrix the kernel does not take gives no hint
    assert o.product_hint(w.float(), "linear") is None and o.product_hint(None, "stream") is None
    hint = o.product_hint(nexts[2][0], "silu_mul")
    assert hint[0] is nexts[2][0] and hint[1] == 1
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    o.linear(x, w, bias, out, status, then=hint)
    plain_out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    o.linear(x, w, bias, plain_out, status)
    assert torch.equal(out, plain_out)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0] and int(counters.abs().sum()) == 0


@pytest.mark.parametrize("m", [1, 8, 17, 64, 100, 256])
@pytest.mark.parametrize("n,k", [(40, 64), (301, 72), (3584, 3584), (520, 18944)])
def test_tcgen05_product_leaves_its_shares_unadded_and_the_norm_adds_them(m, n, k):
    """Small batches on the way into the residual stream: the product's kernel writes the sums of each share
    of k as 32-bit [shares, m, n] (the bias with share 0) and the norm adds them, in order, to the stream."""
    o = ops()
    torch.manual_seed(15)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    ref = plain.linear(x.cpu().double(), w.cpu().double(), bias.cpu().double())
    got = o.linear_to_stream(x, w, bias)
    if m > 128 and n * k * 2 <= o.STREAM_SMALL_WEIGHT_BYTES:
        # a small matrix under a wide batch: an ordinary tensor from the kernel with x as the 128-row operand
        assert isinstance(got, torch.Tensor) and got.dtype == torch.bfloat16 and tuple(got.shape) == (m, n)
        close(got, ref, torch.bfloat16, 2)
        forced, o.STREAM_SMALL_WEIGHT_BYTES = o.STREAM_SMALL_WEIGHT_BYTES, 0          # and the shares, as for the other sizes
        try:
            got = o.linear_to_stream(x, w, bias)
        finally:
            o.STREAM_SMALL_WEIGHT_BYTES = forced
    assert isinstance(got, o.SplitSum) and got.shares.dtype == torch.float32
    assert got.shares.shape == (o.backend().gemm_tc_shares(m, n, k), m, n) and tuple(got.shape) == (m, n)
    close(o.dense(got), ref, torch.float32, 40)
    if k >= 3584:
        assert got.shares.shape[0] > 1, "a long inner dimension on few tiles should have been cut"
    if n % 8 == 0:
        stream = torch.randn(m, n, device=DEV)
        g = 1 + 0.1 * torch.randn(n, device=DEV)
        total = stream.cpu().double() + o.dense(got).cpu().double()
        rows = torch.tensor([m - 1, 0], dtype=torch.int32, device=DEV)
        for r in (None, rows):
            s1 = stream.clone()
            out = torch.empty(m if r is None else 2, n, device=DEV, dtype=torch.bfloat16)
            o.rmsnorm(s1, g, 1e-6, out, delta=got, rows=r)
            idx = torch.arange(m) if r is None else r.cpu().long()
            assert float((s1.cpu().double()[idx] - total[idx]).abs().max()) <= 1e-5
            close(out, plain.rms_norm(total[idx], g.cpu().double(), 1e-6), torch.bfloat16, 2)
    # the same numbers as the kernel that adds the shares itself, to the last bit of its bfloat16 result's rounding
    merged = torch.empty(m, n, device=DEV, dtype=torch.float32)
    o.backend().gemm_tc(x, w, bias, merged, None, *o._split_workspace(torch.device(DEV)))
    close(o.dense(got), merged.cpu().double(), torch.float32, 2)


def test_tcgen05_product_takes_each_element_once():
    """x and w of small integers: every product and sum is exact in bfloat16 and float, so a tile read
    from the wrong place, a k-block counted twice or dropped, shows as a wrong integer."""
    torch.manual_seed(12)
    # the sizes of 2,048 (and 1,990) rows make the kernel choose tiles of 208, 224, 240, 192 and again 208 features
    # (the width whose rounds of one tile an SM come out best), the last with tiles that hang over both edges
    for m, n, k in ((200, 300, 1096), (40, 700, 2056), (2048, 3584, 520), (2048, 2016, 264), (2048, 2160, 264),
                    (2048, 1728, 264), (1990, 3500, 264)):
        x = torch.randint(-3, 4, (m, k), device=DEV).to(torch.bfloat16)
        w = torch.randint(-3, 4, (n, k), device=DEV).to(torch.bfloat16)
        ref = x.cpu().float() @ w.cpu().float().t()          # exact: the sums stay far below 2^24
        for out_dtype in (torch.float32, torch.bfloat16):
            out = torch.full((m, n), float("nan"), device=DEV, dtype=out_dtype)
            ops().backend().gemm_tc(x, w, None, out, None, *ops()._split_workspace(torch.device(DEV)))
            assert torch.equal(out.cpu().float(), ref.to(out_dtype).float())
    # and with the activation in the epilogue at a width of 208 (gate and up interleaved in runs of 8)
    m, inter, k = 2048, 1792, 264
    x = torch.randint(-2, 3, (m, k), device=DEV).to(torch.bfloat16)
    wg = torch.randint(-2, 3, (inter, k), device=DEV).to(torch.bfloat16)
    wu = torch.randint(-2, 3, (inter, k), device=DEV).to(torch.bfloat16)
    act = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops().backend().gemm_tc(x, ops().interleave_gate_up(wg, wu), None, act, None, *ops()._split_workspace(torch.device(DEV)), 1)
    g, u = x.cpu().double() @ wg.cpu().double().t(), x.cpu().double() @ wu.cpu().double().t()
    close(act, g / (1 + torch.exp(-g)) * u, torch.bfloat16, 2)


@pytest.mark.parametrize("bn", [256, 224, 192])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 520, 200), (777, 3000, 136), (1000, 1160, 72), (1990, 3500, 264),
                                   (512, 768, 3592)])
def test_tcgen05_product_of_a_pair_of_ctas(m, n, k, bn):
    """A tile of 256 rows of x to two CTAs (tcgen05.mma.cta_group::2), alone: every width of tile, tiles that hang over
    every edge (the second CTA's rows of x or of w may lie wholly outside), k that is no multiple of 64, more tiles
    than pairs and fewer; small integers first, so that a k-block or a half of w read from the wrong place shows as a
    wrong integer, then random numbers against the plain product with bias."""
    be = ops().backend()
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    torch.manual_seed(16)
    x = torch.randint(-3, 4, (m, k), device=DEV).to(torch.bfloat16)
    w = torch.randint(-3, 4, (n, k), device=DEV).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
    be.gemm_tc_pair(x, w, None, out, 0, bn, status)
    assert torch.equal(out.cpu().float(), (x.cpu().float() @ w.cpu().float().t()).to(torch.bfloat16).float())
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    for _ in range(2):                                        # twice: the barriers' phases start over every launch
        out.fill_(float("nan"))
        be.gemm_tc_pair(x, w, bias, out, 0, bn, status)
        close(out, plain.linear(x.cpu().double(), w.cpu().double(), bias.cpu().double()), torch.bfloat16, 2)
    assert status.tolist() == [0, 0]


@pytest.mark.parametrize("m,inter,k,bn", [(600, 752, 200, 224), (512, 18944 // 4, 1544, 0), (1100, 344, 72, 256), (300, 96, 64, 192)])
def test_gate_up_product_of_a_pair_of_ctas(m, inter, k, bn):
    """silu(x Wg^T) * (x Wu^T) in the epilogue of the kernel of two CTAs a tile; and the same bits as the kernel of one
    CTA a tile gives, which adds a tile's k-blocks in the same order."""
    o = ops()
    torch.manual_seed(17)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    wg = (torch.randn(inter, k, device=DEV) / math.sqrt(k) * 2).to(torch.bfloat16)
    wu = (torch.randn(inter, k, device=DEV) / math.sqrt(k) * 2).to(torch.bfloat16)
    g, u = x.cpu().double() @ wg.cpu().double().t(), x.cpu().double() @ wu.cpu().double().t()
    packed = o.interleave_gate_up(wg, wu)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    out = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    o.backend().gemm_tc_pair(x, packed, None, out, 1, bn, status)
    close(out, g / (1 + torch.exp(-g)) * u, torch.bfloat16, 2)
    assert status.tolist() == [0, 0]
    if k < 1536:                                              # below that the dispatch keeps the kernel of one CTA a tile
        one = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
        o.backend().gemm_tc(x, packed, None, one, None, *o._split_workspace(torch.device(DEV)), 1)
        assert torch.equal(one, out)


@pytest.mark.parametrize("m,n,k,epi", [(300, 520, 8200, 0), (512, 3584, 18944, 0), (272, 1000, 8264, 0), (400, 1504, 8192, 1)])
def test_pairs_of_ctas_with_k_in_two_shares(m, n, k, epi):
    """Few tiles and a long inner dimension: the kernel of two CTAs a tile cuts k into two shares for twice the pairs;
    the shares meet in scratch memory and the pair that arrives last adds them.  Twice: the counters must be back at
    zero; against the plain product, and close to the same kernel without shares (which adds in another order)."""
    o = ops()
    torch.manual_seed(19)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k) * (2 if epi else 1)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV) if epi == 0 else None
    if epi == 0:
        ref = plain.linear(x.cpu().double(), w.cpu().double(), bias.cpu().double())
        packed = w
    else:
        inter = n // 2
        g, u = x.cpu().double() @ w[:inter].cpu().double().t(), x.cpu().double() @ w[inter:].cpu().double().t()
        ref = g / (1 + torch.exp(-g)) * u
        packed = o.interleave_gate_up(w[:inter], w[inter:])
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    scratch, counters = o._split_workspace(torch.device(DEV))
    cols = n if epi == 0 else n // 2
    whole = torch.full((m, cols), float("nan"), device=DEV, dtype=torch.bfloat16)
    o.backend().gemm_tc_pair(x, packed, bias, whole, epi, 0, status)
    for _ in range(2):
        out = torch.full((m, cols), float("nan"), device=DEV, dtype=torch.bfloat16)
        o.backend().gemm_tc_pair(x, packed, bias, out, epi, 0, status, scratch, counters)
        close(out, ref, torch.bfloat16, 2)
        assert int(counters.abs().sum()) == 0 and status.tolist() == [0, 0]
    # two orders of adding the same 32-bit products: a last bit of bfloat16 here and there, no more
    assert float((out.float() - whole.float()).abs().max()) <= float(ref.abs().max()) / 128
    assert float((out.float() != whole.float()).float().mean()) < 0.2


@pytest.mark.parametrize("m,n,k", [(2560, 2048, 8192), (1536, 3584, 8200), (4200, 3584, 8192)])
def test_pairs_of_ctas_cut_the_tiles_of_a_last_partial_round(m, n, k):
    """More tiles than pairs of SMs and a last round of few tiles (80 = 74 + 6, 84 = 74 + 10, 238 = 3 * 74 + 16): with
    scratch memory those tiles' k-blocks are cut into shares for the pairs that would stand idle; the other tiles are
    as without.  The last case's x is larger than half of L2: its tiles are taken across the rows of w first."""
    o = ops()
    torch.manual_seed(20)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    ref = (x.double() @ w.double().t() + bias.double()).cpu()            # a plain 64-bit product (on the device: 40 GFLOP)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    scratch, counters = o._split_workspace(torch.device(DEV))
    whole = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
    o.backend().gemm_tc_pair(x, w, bias, whole, 0, 256, status)
    close(whole, ref, torch.bfloat16, 2)
    for _ in range(2):
        out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
        o.backend().gemm_tc_pair(x, w, bias, out, 0, 256, status, scratch, counters)
        close(out, ref, torch.bfloat16, 2)
        assert int(counters.abs().sum()) == 0 and status.tolist() == [0, 0]
    changed = (out.float() != whole.float()).float().mean()
    assert 0 < float(changed) < 0.1                       # only the cut tiles add in another order
    assert float((out.float() - whole.float()).abs().max()) <= float(ref.abs().max()) / 128


def test_products_of_many_rows_go_to_pairs_of_ctas_and_give_the_same_numbers():
    """What the dispatch sends to the kernel of two CTAs a tile (many rows, a long k, a tile for every pair) equals,
    bit for bit, what that kernel gives when called by name; with 32-bit results and for fewer rows the dispatch
    keeps the kernel of one CTA a tile."""
    o = ops()
    torch.manual_seed(18)
    m, n, k = 1536, 4608, 1536
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn(n, device=DEV)
    ref = plain.linear(x.cpu().double(), w.cpu().double(), bias.cpu().double())
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    by_name = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    o.backend().gemm_tc_pair(x, w, bias, by_name, 0, 0, status)
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    o.linear(x, w, bias, out)
    close(out, ref, torch.bfloat16, 2)
    assert torch.equal(out, by_name) and status.tolist() == [0, 0]
    out32 = torch.empty(m, n, device=DEV, dtype=torch.float32)
    o.linear(x, w, bias, out32)
    close(out32, ref, torch.float32, 40)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,page_size", [(6, 2, 48, 16), (4, 4, 128, 32)])
def test_rotation_and_cache_store(dtype, heads, kv_heads, d, page_size):
    from vt_transformer_b200.parts.rope import rotation_table
    torch.manual_seed(6)
    table = rotation_table(300, d, 50000.0).to(DEV)
    cos, sin = plain.rotation_table(300, d, 50000.0)
    positions = [0, 1, 15, 16, 17, 250, 299, 3]
    token_seq = [0, 0, 0, 0, 0, 1, 1, -1]                       # the last token is padding
    T = len(positions)
    qkv = torch.randn(T, (heads + 2 * kv_heads) * d, device=DEV).to(dtype)
    before = qkv.clone()
    n_pages = 30
    kc = torch.zeros(n_pages, kv_heads, page_size, d, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    bt = torch.full((2, 300 // page_size + 1), -1, dtype=torch.int32)
    bt[0, 0], bt[0, 1], bt[1, 250 // page_size], bt[1, 299 // page_size] = 7, 3, 11, 29
    bt = bt.to(DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    ops().rope_store(qkv, torch.tensor(positions, dtype=torch.int32, device=DEV), table, kc, vc,
                     torch.tensor(token_seq, dtype=torch.int32, device=DEV), bt, heads, kv_heads, d, status=status)
    assert status.tolist() == [0, 0]
    qd, kd = heads * d, kv_heads * d
    live = list(range(T - 1))
    q_ref = plain.rotate(before[:, :qd].view(T, heads, d).cpu().double(), positions, cos, sin)
    k_ref = plain.rotate(before[:, qd:qd + kd].view(T, kv_heads, d).cpu().double(), positions, cos, sin)
    got_q = qkv[:, :qd].view(T, heads, d).cpu().double()
    assert float((got_q[live] - q_ref[live]).abs().max()) <= tol(dtype, 8)
    assert torch.equal(qkv[T - 1], before[T - 1])                       # padding is left alone
    assert torch.equal(qkv[:, qd:], before[:, qd:])                     # k and v rows stay as they were
    for t in live:
        page = int(bt[token_seq[t], positions[t] // page_size])
        slot = positions[t] % page_size
        assert float((kc[page, :, slot].cpu().double() - k_ref[t]).abs().max()) <= tol(dtype, 8)
        assert torch.equal(vc[page, :, slot], before[t, qd + kd:].view(kv_heads, d))
    assert int((kc != 0).any(dim=-1).sum()) == len(live) * kv_heads     # nothing else was written
    # a run that only reads another's cache rotates q and stores nothing
    kc.zero_()
    qkv2 = before.clone()
    ops().rope_store(qkv2, torch.tensor(positions, dtype=torch.int32, device=DEV), table, kc, vc,
                     torch.tensor(token_seq, dtype=torch.int32, device=DEV), bt, heads, kv_heads, d, store=False)
    assert torch.equal(qkv2, qkv) and float(kc.abs().sum()) == 0.0
    # a position beyond the table is reported, not followed
    ops().rope_store(qkv2[:1], torch.tensor([300], dtype=torch.int32, device=DEV), table, kc, vc,
                     torch.tensor([0], dtype=torch.int32, device=DEV), bt, heads, kv_heads, d, status=status)
    assert status.tolist() == [2, 300]


def test_argmax_takes_the_lowest_of_equals():
    torch.manual_seed(7)
    logits = torch.randn(5, 50257, device=DEV)
    logits[1, 40000] = logits[1, 123] = 50.0
    logits[2, 50256] = 60.0
    logits[3, 0] = 70.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops().argmax(logits, out)
    assert out.tolist() == [plain.sample_greedy(logits[r].cpu()) for r in range(5)]
    assert out.tolist()[1:4] == [123, 50256, 0]


@pytest.mark.parametrize("vocab", [1000, 50257])
def test_sampling_kernel_draws_what_the_plain_sampler_draws(vocab):
    from vt_transformer_b200.sampling import uniform
    torch.manual_seed(8)
    cases = [(0.0, -1, 1.0), (0.7, -1, 1.0), (1.3, -1, 1.0), (0.8, 3, 1.0), (1.0, 40, 1.0), (1.0, -1, 0.9),
             (0.6, 50, 0.5), (1.0, 1, 1.0), (2.0, vocab, 0.999)]
    rows = len(cases) * 8
    logits = torch.randn(rows, vocab, device=DEV) * 3
    params = [cases[r % len(cases)] for r in range(rows)]
    us = [uniform(5, r) for r in range(rows)]
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample(logits, torch.tensor([p[0] for p in params], device=DEV),
                 torch.tensor([p[1] for p in params], dtype=torch.int32, device=DEV),
                 torch.tensor([p[2] for p in params], device=DEV), torch.tensor(us, device=DEV), out)
    host = logits.cpu()
    want = [plain.sample(host[r], params[r][0], float(torch.tensor(us[r], dtype=torch.float32)), params[r][1], params[r][2])
            for r in range(rows)]
    assert out.tolist() == want
    assert len(set(out.tolist())) > rows // 2


@pytest.mark.parametrize("vocab", [152064, 151937])
def test_sampling_kernel_on_peaked_flat_and_tied_rows(vocab):
    """The sampling kernel's ways through a row, each against the plain sampler: a peaked row (few tokens hold the
    mass: thresholds and draw finished among a few gathered candidates), a flat row (top_p keeps tens of thousands:
    further passes over the row), top_k beyond what is gathered, thousands of values equal to the k-th (all kept),
    top_p of 0 (the largest alone) and a row whose length is no multiple of four (its start is on no 16-byte
    boundary)."""
    from vt_transformer_b200.sampling import uniform
    torch.manual_seed(9)
    peaked = torch.randn(vocab) * 2
    peaked[torch.randperm(vocab)[:40]] += 12.0
    flat = torch.randn(vocab) * 0.5
    tied = torch.randn(vocab)
    tied[torch.randperm(vocab)[:3000]] = 2.5                    # thousands of equals at the edge of top_k
    tied[torch.randperm(vocab)[:10]] += 6.0
    rows, params = [], []
    for base in (peaked, flat, tied):
        for (t, k, p) in [(0.7, 20, 0.8), (1.0, -1, 0.9), (0.8, 50, 1.0), (1.0, 5000, 0.95), (1.2, -1, 0.0), (0.9, 300, 0.999),
                          (1.0, -1, 1.0), (0.5, 2000, 1.0)]:
            rows.append(base)
            params.append((t, k, p))
    logits = torch.stack(rows).to(DEV)
    n = len(rows)
    for trial in range(3):
        us = [uniform(11 + trial, r) for r in range(n)]
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        ops().sample(logits, torch.tensor([q[0] for q in params], device=DEV),
                     torch.tensor([q[1] for q in params], dtype=torch.int32, device=DEV),
                     torch.tensor([q[2] for q in params], device=DEV), torch.tensor(us, device=DEV), out)
        host = logits.cpu()
        want = [plain.sample(host[r], params[r][0], float(torch.tensor(us[r], dtype=torch.float32)), params[r][1], params[r][2])
                for r in range(n)]
        assert out.tolist() == want, [(r, params[r]) for r in range(n) if out.tolist()[r] != want[r]]
    # the ends of the kept sets: u = 0 draws the first kept index, u just below 1 one of the last
    for uval in (0.0, 0.99999994):
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        ops().sample(logits, torch.tensor([q[0] for q in params], device=DEV),
                     torch.tensor([q[1] for q in params], dtype=torch.int32, device=DEV),
                     torch.tensor([q[2] for q in params], device=DEV), torch.full((n,), uval, device=DEV), out)
        uu = float(torch.tensor(uval, dtype=torch.float32))
        for r in range(n):
            kept = torch.nonzero(plain.kept_probabilities(logits[r].cpu(), *params[r])).flatten()
            assert int(out[r]) == plain.sample(logits[r].cpu(), params[r][0], uu, params[r][1], params[r][2]), (r, params[r])
            assert int(out[r]) in kept.tolist() and (uval > 0 or int(out[r]) == int(kept[0]))


def test_sampling_kernel_follows_the_distribution():
    logits = torch.tensor([0.0, math.log(2.0), math.log(5.0), -40.0] + [-60.0] * 96, device=DEV).repeat(4000, 1)
    n = logits.shape[0]
    u = (torch.arange(n, device=DEV, dtype=torch.float32) + 0.5) / n
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops().sample(logits, torch.ones(n, device=DEV), torch.full((n,), -1, dtype=torch.int32, device=DEV),
                 torch.ones(n, device=DEV), u, out)
    freq = torch.bincount(out.long().cpu(), minlength=100)[:4].double() / n
    assert float((freq - torch.tensor([1 / 8, 2 / 8, 5 / 8, 0.0], dtype=torch.float64)).abs().max()) < 1e-3
