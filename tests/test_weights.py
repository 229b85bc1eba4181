"""Safetensors reading and writing, the check against the model, random weights (no GPU)."""
import json
import os
import struct

import pytest
import torch

import helpers
from vt_transformer_b200.weights import (DictSource, SafetensorsError, SafetensorsSource, WeightError, check_against,
                                         write_random_model)
from vt_transformer_b200.weights import safetensors_io as st
from vt_transformer_b200.weights.random_init import parameter_table


def test_random_folder_reads_back_and_matches_the_library_reader(tmp_path):
    from safetensors import safe_open
    folder = helpers.make_folder("A", str(tmp_path / "A"))
    src = SafetensorsSource(folder)
    table = parameter_table(helpers.make_config("A"))
    check_against(src, table)
    assert "lm_head.weight" not in src.entries()          # tied: the head is not written
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        assert set(f.keys()) == set(src.entries())
        for name in f.keys():
            ours, theirs = src.get(name), f.get_tensor(name)
            assert ours.dtype == theirs.dtype == torch.bfloat16
            assert torch.equal(ours, theirs)
    # norm weights are 1 + N(0, sigma), the rest N(0, sigma)
    n = src.get("model.norm.weight").float()
    assert abs(float(n.mean()) - 1.0) < 0.05
    q = src.get("model.layers.0.self_attn.q_proj.weight").float()
    assert abs(float(q.mean())) < 0.01 and 0.5 * helpers.SIGMA["A"] < float(q.std()) < 1.5 * helpers.SIGMA["A"]


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    cfg = helpers.make_config("B")
    a = SafetensorsSource(write_random_model(cfg, str(tmp_path / "a"), seed=5, sigma=0.05))
    b = SafetensorsSource(write_random_model(cfg, str(tmp_path / "b"), seed=5, sigma=0.05))
    c = SafetensorsSource(write_random_model(cfg, str(tmp_path / "c"), seed=6, sigma=0.05))
    name = "model.layers.2.mlp.down_proj.weight"
    assert torch.equal(a.get(name), b.get(name)) and not torch.equal(a.get(name), c.get(name))
    assert not torch.equal(a.get(name), a.get("model.layers.1.mlp.down_proj.weight"))
    assert "lm_head.weight" in a.entries()                # untied


def test_reads_a_file_the_library_wrote_and_keeps_32_bit(tmp_path):
    from safetensors.torch import save_file
    t = {"a": torch.randn(3, 8), "b": torch.randn(4, 8).to(torch.bfloat16), "c": torch.randn(2, 8).to(torch.float16),
         "i": torch.arange(6, dtype=torch.int64).view(2, 3)}
    os.makedirs(tmp_path / "m")
    save_file(t, str(tmp_path / "m" / "model.safetensors"))
    src = SafetensorsSource(str(tmp_path / "m"))
    assert src.get("a").dtype == torch.float32 and torch.equal(src.get("a"), t["a"])      # 32-bit stays
    assert src.get("b").dtype == torch.bfloat16 and torch.equal(src.get("b"), t["b"])
    assert src.get("c").dtype == torch.bfloat16                                               # float16 -> bfloat16
    assert src.get("i").dtype == torch.int32 and torch.equal(src.get("i").long(), t["i"])    # tables -> int32


def test_sharded_folder_and_duplicate(tmp_path):
    from safetensors.torch import save_file
    d = tmp_path / "s"
    os.makedirs(d)
    save_file({"x": torch.ones(2, 8)}, str(d / "p1.safetensors"))
    save_file({"y": torch.zeros(2, 8)}, str(d / "p2.safetensors"))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "p1.safetensors", "y": "p2.safetensors"}}))
    src = SafetensorsSource(str(d))
    assert set(src.entries()) == {"x", "y"} and float(src.get("x").sum()) == 16.0
    save_file({"x": torch.ones(2, 8)}, str(d / "p2.safetensors"))
    with pytest.raises(SafetensorsError, match="two shards"):
        SafetensorsSource(str(d))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = helpers.make_folder("A", str(tmp_path / "A"))
    src = SafetensorsSource(folder)
    tensors = {n: src.get(n).clone() for n in src.entries()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(48)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 64, dtype=torch.int32)
    table = parameter_table(helpers.make_config("A"))
    with pytest.raises(WeightError) as e:
        check_against(DictSource(tensors, "a test folder"), table)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert err.wrong_shape == {"model.layers.0.self_attn.k_proj.bias": ((32,), (48,))}
    assert list(err.wrong_dtype) == ["model.layers.0.self_attn.q_proj.weight"]
    text = str(err)
    for word in ("a test folder", "missing (2)", "unexpected (1)", "expected [32], found [48]", "up_proj", "inv_freq"):
        assert word in text


def test_untied_model_misses_its_head(tmp_path):
    folder = helpers.make_folder("B", str(tmp_path / "B"))
    src = SafetensorsSource(folder)
    tensors = {n: src.get(n) for n in src.entries() if n != "lm_head.weight"}
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_against(DictSource(tensors), parameter_table(helpers.make_config("B")))


def test_broken_files(tmp_path):
    d = tmp_path / "x"
    os.makedirs(d)
    with pytest.raises(SafetensorsError, match="neither"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="not plausible"):
        SafetensorsSource(str(d))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    (d / "model.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsSource(str(d))
    hdr = b"{not json"
    (d / "model.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr)
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsSource(str(d))


def test_writer_checks_its_layout(tmp_path):
    layout = [("a", torch.bfloat16, (2, 8))]
    with pytest.raises(SafetensorsError, match="layout"):
        st.write_file(str(tmp_path / "f.safetensors"), iter([("a", torch.zeros(2, 4, dtype=torch.bfloat16))]), layout)
    with pytest.raises(SafetensorsError, match="fewer"):
        st.write_file(str(tmp_path / "f.safetensors"), iter([]), layout)


def _rewrite(src_folder, dst_folder, change, extra=None):
    """A copy of a model folder whose tensors went through ``change(name, tensor)``, plus ``extra`` tensors."""
    src = SafetensorsSource(src_folder)
    tensors = {n: change(n, src.get(n).clone()) for n in src.entries()}
    tensors.update(extra or {})
    os.makedirs(dst_folder, exist_ok=True)
    with open(os.path.join(src_folder, "config.json")) as f, open(os.path.join(dst_folder, "config.json"), "w") as g:
        g.write(f.read())
    st.write_file(os.path.join(dst_folder, "model.safetensors"), iter(tensors.items()),
                  [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()])
    return dst_folder


def wide_and_rounded_folders(tmp):
    """A folder stored in float32 whose values bfloat16 cannot hold exactly, and one that stores its matrices
    rounded to bfloat16 (vectors, that is norm weights and biases, are read in 32-bit in both modes and stay)."""
    g = torch.Generator().manual_seed(3)
    base = helpers.make_folder("B", os.path.join(tmp, "bf16"))
    wide = _rewrite(base, os.path.join(tmp, "f32"), lambda n, t: t.float() + 1e-4 * torch.randn(t.shape, generator=g))
    rounded = _rewrite(wide, os.path.join(tmp, "rounded"), lambda n, t: t.to(torch.bfloat16) if t.dim() == 2 else t)
    return wide, rounded


def test_matrices_stored_in_32_bit_are_kept_with_a_warning_or_rounded_with_a_report(fake_backend, tmp_path, capsys):
    """In bfloat16 mode matrices stored in float32 stay 32-bit by default and a warning says what that costs; with
    fp32_weights="round" they become bfloat16 and a line reports it; in 32-bit mode nothing is said.  (What the
    logits then are is compared on the GPU: tests/test_gpu_engine.py.)"""
    import warnings
    from vt_transformer_b200.engine import ModelRunner
    wide, rounded = wide_and_rounded_folders(str(tmp_path))
    kw = dict(device="cpu", page_size=16, num_pages=8, max_requests=1)
    with pytest.warns(UserWarning, match="stored in float32 and stay so.*fp32_weights='round'"):
        kept = ModelRunner.from_folder(wide, dtype="bfloat16", **kw)
    assert kept.model.blocks[0].mixer.w_qkv.dtype == torch.float32
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        capsys.readouterr()
        cut = ModelRunner.from_folder(wide, dtype="bfloat16", fp32_weights="round", **kw)
        assert "rounded to bfloat16 (to nearest even): 0 values became infinite, 0 became zero" in capsys.readouterr().err
        ref = ModelRunner.from_folder(rounded, dtype="bfloat16", **kw)
        full = ModelRunner.from_folder(wide, dtype="float32", **kw)
        assert capsys.readouterr().err == ""
    assert cut.model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16 and cut.model.blocks[2].ffn.w_down.dtype == torch.bfloat16
    assert cut.model.head.weight.dtype == torch.bfloat16 and full.model.head.weight.dtype == torch.float32
    for a, b in ((cut.model.blocks[1].mixer.w_qkv, ref.model.blocks[1].mixer.w_qkv), (cut.model.head.weight, ref.model.head.weight)):
        assert torch.equal(a, b)                            # rounded at load = rounded in the file
    with pytest.raises(ValueError, match="fp32_weights"):
        ModelRunner.from_folder(wide, dtype="bfloat16", fp32_weights="maybe", **kw)


def test_rounding_counts_the_values_that_change_class():
    from vt_transformer_b200.parts import Runtime
    rt = Runtime(torch.device("cpu"), torch.bfloat16, None, fp32_weights="round")
    t = torch.tensor([[1.0, 3.4e38, -3.4e38, 1e-44], [0.0, 2.5, 1e-40, -7.0]], dtype=torch.float32)
    out = rt.param(t)
    assert out.dtype == torch.bfloat16 and rt.notes == {"rounded": 1, "rounded_values": 8, "to_inf": 2, "to_zero": 1}
    assert torch.equal(out, t.to(torch.bfloat16))
    assert rt.param(t, "vector").dtype == torch.float32 and rt.notes["rounded"] == 1     # vectors are read in 32-bit anyway


def test_float16_is_rounded_with_a_report_and_known_extras_are_left_aside_with_a_warning(fake_backend, tmp_path, capsys):
    from vt_transformer_b200.engine import ModelRunner
    base = helpers.make_folder("A", str(tmp_path / "bf16"))
    extra = {f"model.layers.{i}.self_attn.rotary_emb.inv_freq": torch.ones(8) for i in range(2)}
    half = _rewrite(base, str(tmp_path / "f16"), lambda n, t: t.to(torch.float16), extra)
    with pytest.warns(UserWarning, match="2 tensors that the model does not read were left aside: .*rotary_emb.inv_freq"):
        runner = ModelRunner.from_folder(half, dtype="bfloat16", device="cpu", page_size=16, num_pages=2, max_requests=1)
    err = capsys.readouterr().err
    assert "tensors stored in float16 were rounded to bfloat16" in err
    assert runner.model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    # a tensor that is no known extra is still a difference
    odd = _rewrite(base, str(tmp_path / "odd"), lambda n, t: t, {"model.layers.0.self_attn.rotary_emb.other": torch.ones(8)})
    with pytest.raises(WeightError, match="unexpected"):
        ModelRunner.from_folder(odd, dtype="bfloat16", device="cpu", page_size=16, num_pages=2, max_requests=1)


def test_a_part_may_bring_an_initialiser_of_its_own():
    """The random-weights mode fills a tensor by the function its ParamSpec names; a new one is registered, not
    edited in."""
    from vt_transformer_b200.parts import ParamSpec
    from vt_transformer_b200.weights import random_tensor, register_initialiser, unregister_initialiser
    spec = ParamSpec((4, 6), init="toy_ramp")
    with pytest.raises(ValueError, match="unknown initialiser 'toy_ramp'.*known: normal, one_plus_normal, zeros"):
        random_tensor("x", spec, 0, 0.02)
    register_initialiser("toy_ramp", lambda shape, g, sigma, device: torch.arange(shape[0] * shape[1], dtype=torch.float32).view(shape) * sigma)
    try:
        t = random_tensor("x", spec, 0, 0.5)
        assert t.dtype == torch.bfloat16 and torch.equal(t.float(), (torch.arange(24.0) * 0.5).view(4, 6))
        with pytest.raises(ValueError, match="registered already"):
            register_initialiser("toy_ramp", lambda *a: None)
    finally:
        unregister_initialiser("toy_ramp")
    assert float(random_tensor("b", ParamSpec((8,), role="vector", init="zeros"), 1, 0.3).abs().sum()) == 0.0
