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
