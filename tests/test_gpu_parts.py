"""Each part alone on the GPU, built from its spec and fed its own tensors, against the plain
implementation's function for it, at sizes of its own."""
import pytest
import torch

from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def runtime(dtype):
    from vt_transformer_b200 import ops
    from vt_transformer_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype, ops)


def ops_module():
    from vt_transformer_b200 import ops
    return ops


def tensors_for(part, sigma=0.1, seed=0):
    from vt_transformer_b200.weights.loader import random_tensor
    return {name: random_tensor(name, spec, seed, sigma) for name, spec in part.param_specs().items()}


@pytest.fixture(autouse=True)
def _same_numbers_whatever_ran_before():
    torch.manual_seed(1234)


def tol(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


def close(got, ref, dtype, factor=1.0):
    """Within the dtype's tolerance at the scale of the reference (bfloat16 rounds every part's
    output to 8 bits of mantissa, so its error grows with the size of the numbers)."""
    err = float((got.double().cpu() - ref).abs().max())
    bound = tol(dtype) * factor * max(1.0, float(ref.abs().max()))
    assert err <= bound, f"error {err:.3e} above {bound:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from vt_transformer_b200.parts import NormSpec, build_part
    part = build_part("norm", NormSpec(size=264, eps=2e-4), "n", runtime(dtype))
    w = tensors_for(part)
    assert list(w) == ["n.weight"] and abs(float(w["n.weight"].float().mean()) - 1) < 0.05
    part.load(w.__getitem__)
    x = torch.randn(9, 264, device=DEV)
    out = part(x)
    ref = plain.rms_norm(x.cpu().double(), w["n.weight"].double(), 2e-4)
    assert out.dtype == dtype
    close(out, ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from vt_transformer_b200.parts import GatedMLPSpec, build_part
    part = build_part("feed_forward", GatedMLPSpec(hidden=136, inter=200), "mlp.", runtime(dtype))
    w = tensors_for(part, sigma=0.15)
    assert set(w) == {"mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"}
    part.load(w.__getitem__)
    h = torch.randn(21, 136, device=DEV).to(dtype)
    out = ops_module().dense(part.forward(h, None))     # a small bfloat16 batch leaves unadded shares
    ref = plain.swiglu(h.cpu().double(), *(w[f"mlp.{n}_proj.weight"].double() for n in ("gate", "up", "down")))
    close(out, ref, dtype)
    with pytest.raises(ValueError, match="gelu"):
        build_part("feed_forward", GatedMLPSpec(hidden=8, inter=8, activation="gelu"), "m.", runtime(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 11])
def test_attention_part_in_two_portions(dtype, window):
    """The mixer alone, with a cache view made by hand: a sequence in two steps."""
    from vt_transformer_b200.parts import AttentionSpec, CacheView, PositionSpec, build_part
    spec = AttentionSpec(hidden=96, heads=6, kv_heads=2, head_dim=32, qkv_bias=True, window=window,
                         position=PositionSpec(kind="rotary", dim=32, base=7777.0, max_positions=64))
    part = build_part("mixer", spec, "att.", runtime(dtype))
    assert part.cache_spec().kv_heads == 2 and part.cache_spec().window == window
    w = tensors_for(part, sigma=0.2)
    part.load(w.__getitem__)
    T = 40
    h = torch.randn(T, 96, device=DEV).to(dtype)
    kc = torch.zeros(5, 2, 16, 32, device=DEV, dtype=dtype)
    view = CacheView(spec=part.cache_spec(), k=kc, v=torch.zeros_like(kc),
                     block_table=torch.tensor([[4, 0, 2]], dtype=torch.int32, device=DEV), page_size=16)
    outs = []
    for a, b in ((0, 27), (27, 40)):
        import helpers
        ctx = helpers.step_context([b - a], [a], DEV, status=torch.zeros(2, dtype=torch.int32, device=DEV))
        outs.append(ops_module().dense(part.forward(h[a:b].contiguous(), ctx, view), dtype))
        assert ctx.status.tolist() == [0, 0]
    hd = h.cpu().double()
    cos, sin = plain.rotation_table(64, 32, 7777.0)
    q = plain.linear(hd, w["att.q_proj.weight"].double(), w["att.q_proj.bias"].double()).view(T, 6, 32)
    k = plain.linear(hd, w["att.k_proj.weight"].double(), w["att.k_proj.bias"].double()).view(T, 2, 32)
    v = plain.linear(hd, w["att.v_proj.weight"].double(), w["att.v_proj.bias"].double()).view(T, 2, 32)
    o = plain.attention(plain.rotate(q, range(T), cos, sin), plain.rotate(k, range(T), cos, sin), v, window)
    ref = plain.linear(o.reshape(T, 192), w["att.o_proj.weight"].double())
    close(torch.cat(outs), ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part_and_the_residual_stream(dtype):
    """A whole block; the stream is 32-bit and the sums are formed inside the norms."""
    from vt_transformer_b200.parts import (AttentionSpec, BlockSpec, CacheView, GatedMLPSpec, NormSpec, PositionSpec,
                                           ResidualStream, build_part)
    spec = BlockSpec(mixer=AttentionSpec(hidden=64, heads=2, kv_heads=1, head_dim=16, qkv_bias=True,
                                         position=PositionSpec(kind="none")),
                     ffn=GatedMLPSpec(hidden=64, inter=72), norm1=NormSpec(64, 1e-6), norm2=NormSpec(64, 1e-6), prefix="b.")
    part = build_part("block", spec, "b.", runtime(dtype))
    w = tensors_for(part, sigma=0.2)
    part.load(w.__getitem__)
    T = 20
    x0 = torch.randn(T, 64, device=DEV)
    stream = ResidualStream(x0.clone())
    kc = torch.zeros(2, 1, 16, 16, device=DEV, dtype=dtype)
    view = CacheView(spec=part.cache_spec(), k=kc, v=torch.zeros_like(kc),
                     block_table=torch.tensor([[1, 0]], dtype=torch.int32, device=DEV), page_size=16)
    import helpers
    part.forward(stream, helpers.step_context([T], [0], DEV), view)
    assert stream.x.dtype == torch.float32 and stream.pending is not None
    got = stream.x.cpu().double() + ops_module().dense(stream.pending).cpu().double()
    x = x0.cpu().double()
    wd = {k: v.double() for k, v in w.items()}
    h = plain.rms_norm(x, wd["b.input_layernorm.weight"], 1e-6)
    q = plain.linear(h, wd["b.self_attn.q_proj.weight"], wd["b.self_attn.q_proj.bias"]).view(T, 2, 16)
    k = plain.linear(h, wd["b.self_attn.k_proj.weight"], wd["b.self_attn.k_proj.bias"]).view(T, 1, 16)
    v = plain.linear(h, wd["b.self_attn.v_proj.weight"], wd["b.self_attn.v_proj.bias"]).view(T, 1, 16)
    x = x + plain.linear(plain.attention(q, k, v).reshape(T, 32), wd["b.self_attn.o_proj.weight"])   # no rotation
    h = plain.rms_norm(x, wd["b.post_attention_layernorm.weight"], 1e-6)
    x = x + plain.swiglu(h, wd["b.mlp.gate_proj.weight"], wd["b.mlp.up_proj.weight"], wd["b.mlp.down_proj.weight"])
    close(got, x, dtype)


def test_a_matrix_stored_in_32_bit_stays_32_bit_on_the_bfloat16_path():
    from vt_transformer_b200.parts import GatedMLPSpec, build_part
    part = build_part("feed_forward", GatedMLPSpec(hidden=64, inter=80), "m.", runtime(torch.bfloat16))
    w = {n: t.float() + 1e-4 * torch.randn(t.shape) for n, t in tensors_for(part, sigma=0.2).items()}   # not bfloat16 values
    part.load(w.__getitem__)
    assert part.w_down.dtype == torch.float32 and part.w_gate_up.dtype == torch.float32
    h = torch.randn(5, 64, device=DEV).to(torch.bfloat16)
    out = ops_module().dense(part.forward(h, None))
    ref = plain.swiglu(h.cpu().double(), *(w[f"m.{n}_proj.weight"].double() for n in ("gate", "up", "down")))
    close(out, ref, torch.bfloat16)          # the bound of every other part here: at the scale of the reference
