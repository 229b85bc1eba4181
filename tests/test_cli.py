"""The command line: the random-weights mode (no GPU) and generation (GPU)."""
import json
import os
import subprocess
import sys

import pytest

import helpers

ROOT = helpers.ROOT


def run_cli(*args, stdin=None):
    env = dict(os.environ, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, "-m", "vt_transformer_b200", *args], input=stdin, capture_output=True,
                          text=True, timeout=600, env=env, cwd=ROOT)


def test_random_weights_mode_writes_a_folder_that_loads(tmp_path):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(helpers.CONFIGS["B"]))
    out = tmp_path / "model"
    res = run_cli("random-weights", "--config", str(cfg), "--out", str(out), "--seed", "5", "--sigma", "0.05")
    assert res.returncode == 0, res.stderr
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    from vt_transformer_b200.config import load_config
    from vt_transformer_b200.weights import SafetensorsSource, check_against
    from vt_transformer_b200.weights.random_init import parameter_table
    config = load_config(str(out))
    assert config == helpers.make_config("B")
    check_against(SafetensorsSource(str(out)), parameter_table(config))


def test_cli_errors_are_plain(tmp_path):
    assert run_cli("generate", "--model", str(tmp_path)).returncode != 0
    bad = tmp_path / "cfg.json"
    bad.write_text(json.dumps({"architectures": ["Nope"]}))
    res = run_cli("random-weights", "--config", str(bad), "--out", str(tmp_path / "m"))
    assert res.returncode != 0 and "not registered" in res.stderr


def test_defaults_follow_the_front_end():
    from vt_transformer_b200.cli import build_parser
    args = build_parser().parse_args(["generate", "--model", "x"])
    assert (args.max_tokens, args.temperature, args.top_k, args.top_p) == (2048, 0.6, -1, 1.0)
    assert (args.max_running_reqs, args.max_seq_len, args.max_extend_tokens) == (128, 4096, 8192)


@pytest.mark.gpu
def test_generate_from_the_command_line(folders):
    import scenarios
    folder = folders("A")
    prompts = helpers.prompts_for("A")[:2]
    args = ["generate", "--model", folder, "--dtype", "float32", "--temperature", "0", "--max-tokens", "8", "--ignore-eos",
            "--num-pages", "16", "--max-seq-len", "128", "--stats"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(str(t) for t in p)]
    res = run_cli(*args, "--shell-mode", stdin=" ".join(str(t) for t in prompts[0]) + "\n")
    assert res.returncode == 0, res.stderr[-3000:]
    lines = [[int(t) for t in l.split()] for l in res.stdout.splitlines() if l.strip()]
    want = [scenarios.plain_generate(folder, p, 8) for p in prompts]
    assert lines == want + [want[0]]
    assert res.stderr.count("Generated") == 2 and '"finished": 3' in res.stderr
