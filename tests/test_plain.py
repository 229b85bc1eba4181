"""The plain implementation itself (no GPU): properties that follow from vt-transformer's
formulas, and the one piece of the reference that runs on a CPU (its rotation table)."""
import math
import os

import numpy as np
import torch

import helpers
from plain import qwen2_plain as plain


def test_rotation_table_equals_the_reference_function():
    """tests/golden/rotary_table.npz was made by compiling v1/tensortype/common.cpp:6-24."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "rotary_table.npz"))
    for n in range(4):
        length, dims, base = g[f"case{n}_args"]
        ref = g[f"case{n}"]                                   # [len, dims, (cos, sin)]
        cos, sin = plain.rotation_table(int(length), int(dims), float(base))
        half = int(dims) // 2
        assert np.array_equal(ref[:, :half], ref[:, half:])   # both halves carry the same angles
        # The reference calls cos(float) and sin(float), libm's single-precision routines, which
        # are not always correctly rounded; the plain table rounds the double result.  So the
        # tables agree to one unit in the last place, and in nearly all entries exactly.
        from vt_transformer_b200.parts.rope import rotation_table
        ours = rotation_table(int(length), int(dims), float(base)).numpy()
        for col, mine in ((0, cos), (1, sin)):
            mine = mine.to(torch.float32).numpy()
            want = np.ascontiguousarray(ref[:, :half, col])
            ulps = np.abs(mine.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
            assert ulps.max() <= 1 and (ulps == 0).mean() > 0.98
            assert np.array_equal(ours[..., col], mine)      # the engine's table is the plain one's numbers


def test_rms_norm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64)
    out = plain.rms_norm(x, w, 0.0)
    assert torch.allclose(out, torch.tensor([[3.0, 8.0, 0.0, 0.0]], dtype=torch.float64) / math.sqrt(25 / 4))
    wg = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    wu = torch.tensor([[0.0, 2.0]], dtype=torch.float64)
    wd = torch.tensor([[1.0], [-1.0]], dtype=torch.float64)
    y = plain.swiglu(torch.tensor([[0.5, 3.0]], dtype=torch.float64), wg, wu, wd)
    silu = 0.5 / (1 + math.exp(-0.5))
    assert torch.allclose(y, torch.tensor([[silu * 6.0, -silu * 6.0]], dtype=torch.float64))


def test_rotation_pairs_and_relative_positions():
    cos, sin = plain.rotation_table(64, 16, 10000.0)
    x = torch.randn(1, 1, 16, dtype=torch.float64)
    r = plain.rotate(x, [5], cos, sin)
    i = 3                                                    # pair (3, 3 + 8)
    assert math.isclose(float(r[0, 0, i]), float(x[0, 0, i] * cos[5, i] - x[0, 0, i + 8] * sin[5, i]))
    assert math.isclose(float(r[0, 0, i + 8]), float(x[0, 0, i + 8] * cos[5, i] + x[0, 0, i] * sin[5, i]))
    # q.k depends on the distance of the positions only
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    d1 = (plain.rotate(q, [9], cos, sin) * plain.rotate(k, [4], cos, sin)).sum()
    d2 = (plain.rotate(q, [25], cos, sin) * plain.rotate(k, [20], cos, sin)).sum()
    assert abs(float(d1 - d2)) < 1e-6      # the angles are float32 products, so not to the last bit


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, nh, nkv, d = 12, 4, 2, 16
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nh, nkv, nkv))
    o = plain.attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[7:], v2[7:] = 0, 99                                   # the future does not reach rows 0..6
    assert torch.allclose(plain.attention(q, k2, v2)[:7], o[:7])
    assert torch.allclose(o[0], v[0].repeat_interleave(2, dim=0))        # one key: the value itself, by group
    # a window of 3: row t sees t-2..t
    ow = plain.attention(q, k, v, window=3)
    s = (q[9, 1] @ k[7:10, 0].t()) / math.sqrt(d)
    assert torch.allclose(ow[9, 1], torch.softmax(s, 0) @ v[7:10, 0])
    assert torch.allclose(ow[:3], o[:3])


def test_forward_prefix_property_and_orders(folders):
    folder = folders("A")
    cfg, w = plain.read_config(folder), plain.read_weights(folder)
    ids = helpers.prompts_for("A")[2]
    full = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:9]), full[:9], atol=1e-12)   # causal as a whole
    assert full.shape == (len(ids), cfg.vocab) and torch.isfinite(full).all()
    # naming every layer once in order is the default; another order gives other logits
    assert torch.equal(plain.forward(cfg, w, ids, order=[0, 1]), full)
    assert not torch.allclose(plain.forward(cfg, w, ids, order=[0, 1, 1]), full)
    assert not torch.allclose(plain.forward(cfg, w, ids, order=[0, (1, 0)]), full)


def test_window_config_changes_only_late_positions(folders):
    folder = folders("C")
    cfg, w = plain.read_config(folder), plain.read_weights(folder)
    assert cfg.window == [None, None, 20, 20]
    ids = helpers.prompts_for("C")[3]
    with_window = plain.forward(cfg, w, ids)
    cfg.window = [None] * 4
    without = plain.forward(cfg, w, ids)
    assert torch.allclose(with_window[:20], without[:20], atol=1e-12)     # the window is not full yet
    assert not torch.allclose(with_window[40:], without[40:], atol=1e-6)


def test_samplers():
    torch.manual_seed(1)
    logits = torch.randn(50)
    logits[17] = logits[33] = 9.0                            # a tie: the lowest index wins
    assert plain.sample_greedy(logits) == 17
    assert plain.sample(logits, 0.0, 0.3) == 17 and plain.sample(logits, 1.0, 0.3, top_k=1) == 17
    logits = torch.tensor([0.0, math.log(2.0), math.log(5.0), -50.0])   # p = 1/8, 2/8, 5/8, ~0
    assert [plain.sample(logits, 1.0, u) for u in (0.0, 0.12, 0.13, 0.37, 0.38, 0.999)] == [0, 0, 1, 1, 2, 2]
    p = plain.kept_probabilities(logits, 1.0, top_k=2)
    assert torch.allclose(p, torch.tensor([0.0, 2 / 7, 5 / 7, 0.0], dtype=torch.float64))
    p = plain.kept_probabilities(logits, 1.0, top_p=0.7)     # 5/8 < 0.7 <= 7/8: two tokens
    assert torch.allclose(p, torch.tensor([0.0, 2 / 7, 5 / 7, 0.0], dtype=torch.float64))
    p = plain.kept_probabilities(logits, 1.0, top_p=0.5)
    assert torch.allclose(p, torch.tensor([0.0, 0.0, 1.0, 0.0], dtype=torch.float64))
    # temperature sharpens
    assert plain.kept_probabilities(logits, 0.5)[2] > plain.kept_probabilities(logits, 1.0)[2]
    # the reference's top-3 walk draws from the distribution of top_k = 3
    torch.manual_seed(2)
    logits = torch.randn(40)
    us = [(i + 0.5) / 4000 for i in range(4000)]
    ours = np.bincount([plain.sample(logits, 0.8, u, top_k=3) for u in us], minlength=40) / 4000
    theirs = np.bincount([plain.sample_top3_reference(logits, 0.8, u) for u in us], minlength=40) / 4000
    assert np.abs(ours - theirs).max() < 2e-3 and (ours > 0).sum() == 3
    assert np.abs(ours - plain.kept_probabilities(logits, 0.8, top_k=3).numpy()).max() < 1e-3
    # the counter random numbers are uniform and differ by request and index
    u = [plain.uniform_from_counter(7, r, i) for r in range(20) for i in range(50)]
    assert 0.45 < float(np.mean(u)) < 0.55 and len(set(u)) > 990 and all(0 <= x < 1 for x in u)


# ----------------------------------------------------------------------------- the reference's own kernels
# tests/golden/reference_kernels.npz holds inputs and outputs of vt-transformer's CUDA kernels, compiled unchanged
# and run on a B200 (tests/golden/make_kernel_golden.py).  They are float kernels: the plain functions run in
# float64 and must agree to float rounding.


def _kernels():
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz"))


def test_rms_norm_equals_the_reference_kernel():
    """v1/tensortype/cuda_kernels/rmsnorm.cu:10-49: out = w * x * rsqrt(mean(x^2) + eps), and norm2 is that rsqrt."""
    g = _kernels()
    for n in range(2):
        x, w = torch.from_numpy(g[f"rms{n}_x"]).double(), torch.from_numpy(g[f"rms{n}_w"]).double()
        eps = float(g[f"rms{n}_eps"])
        got = plain.rms_norm(x, w, eps)
        want = torch.from_numpy(g[f"rms{n}_out"]).double()
        assert float((got - want).abs().max()) <= 2e-6 * float(want.abs().max())
        r = torch.rsqrt((x * x).mean(dim=-1) + eps)
        assert float((r - torch.from_numpy(g[f"rms{n}_norm2"]).double()).abs().max()) <= 1e-6
        # the weight multiplies as it is: with 1 + w the result would differ by the size of the result itself
        assert float((plain.rms_norm(x, 1.0 + w, eps) - want).abs().max()) > 0.5


def test_rotation_equals_the_reference_kernel():
    """v1/tensortype/cuda_kernels/rotary_embed.cu:9-30 with the table of fill_rotary_cache: pairs (i, i + d/2), the
    row at index l of sequence b rotated by position pos[b] + l."""
    g = _kernels()
    x, want = torch.from_numpy(g["rot_x"]).double(), torch.from_numpy(g["rot_out"]).double()
    table, pos = g["rot_table"], g["rot_pos"]
    bs, length, hnum, dims = x.shape
    cos, sin = plain.rotation_table(table.shape[0], dims, 1000000.0)          # the table's case: 24 positions, base 1e6
    assert np.abs(cos.float().numpy() - table[:, :dims // 2, 0]).max() <= 1e-7
    for b in range(bs):
        got = plain.rotate(x[b], range(int(pos[b]), int(pos[b]) + length), cos, sin)
        assert float((got - want[b]).abs().max()) <= 5e-6, b
    # another pairing (neighbours 2i, 2i + 1) is another function
    a, c = x[1, :, :, 0::2], x[1, :, :, 1::2]
    p = torch.arange(int(pos[1]), int(pos[1]) + length)
    co, si = cos[p][:, None, :], sin[p][:, None, :]
    other = torch.stack([a * co - c * si, c * co + a * si], dim=-1).reshape(length, hnum, dims)
    assert float((other - want[1]).abs().max()) > 0.1


def test_the_activation_of_swiglu_equals_the_reference_kernel():
    """v1/tensortype/cuda_kernels/silu_product.cu:9-18: out = act / (1 + exp(-act)) * in, the activation on the first
    argument, which the graph gives the product with w1, the gate (inference_fp16.dag:333-335)."""
    g = _kernels()
    act, inp = torch.from_numpy(g["silu_act"]).double(), torch.from_numpy(g["silu_in"]).double()
    n = act.numel()
    eye, zero = torch.eye(n, dtype=torch.float64), torch.zeros(n, n, dtype=torch.float64)
    x = torch.cat([act, inp])[None, :]
    got = plain.swiglu(x, torch.cat([eye, zero], dim=1), torch.cat([zero, eye], dim=1), eye)[0]   # gate picks act, up picks in
    want = torch.from_numpy(g["silu_out"]).double()
    assert float((got - want).abs().max()) <= 2e-6 * max(1.0, float(want.abs().max()))
    swapped = plain.swiglu(x, torch.cat([zero, eye], dim=1), torch.cat([eye, zero], dim=1), eye)[0]
    assert float((swapped - want).abs().max()) > 0.5


def test_the_mask_rule_of_attention_equals_the_reference_kernel():
    """v1/tensortype/cuda_kernels/causal_mask.cu:12-57: new row t of `new` rows after `full - new` cached ones sees
    key j if j <= full - new + t (and the key is not masked out).  The plain attention's rule is read off its
    output: with all scores equal and one-hot values, out[t, j] > 0 exactly where row t sees key j."""
    g = _kernels()
    m, want = g["mask_in"], g["mask_out"]
    batch, new, full = want.shape
    q = torch.zeros(full, 1, full, dtype=torch.float64)
    k = torch.zeros(full, 1, full, dtype=torch.float64)
    v = torch.eye(full, dtype=torch.float64)[:, None, :]
    seen = (plain.attention(q, k, v)[:, 0, :] > 0).numpy()[full - new:]        # the last `new` rows of the whole sequence
    assert np.array_equal(want[0] == 0.0, seen)
    assert (want[0][~seen] < -1e30).all()
    # the second sequence has key 2 masked out (a padding key of the reference's rectangular batch; the engine has
    # no padding keys): everything else follows the same rule
    expect = seen.copy()
    expect[:, 2] = False
    assert np.array_equal(want[1] == 0.0, expect) and int(m[1, 2]) == 0


def test_the_samplers_equal_the_reference_kernels():
    """v1/tensortype/cuda_kernels/easy_sampling.cu:141-169 (the largest logit) and :32-104 (the three largest,
    softmax over them at a temperature, walked from the third to the first against one uniform number)."""
    g = _kernels()
    logits = torch.from_numpy(g["top_logits"])
    for b in range(logits.shape[0]):
        assert plain.sample_greedy(logits[b]) == int(g["top1_ids"][b])
    temp = float(g["top3_temperature"])
    for n, u in enumerate(g["top3_draws"]):
        for b in range(logits.shape[0]):
            assert plain.sample_top3_reference(logits[b], temp, float(u)) == int(g["top3_ids"][n, b]), (n, b)
    assert len({int(i) for i in g["top3_ids"].flatten()}) > logits.shape[0]   # the draws did pick different ranks
