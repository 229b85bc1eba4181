"""Tiny configurations, traces and comparisons shared by the tests."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Three tiny configurations that differ in every size and option.  A and B are the two of the
# task's description; C adds a window on the later layers, a head size that is no power of two,
# a head_dim that is not hidden / heads, and a vocabulary and width that are no powers of two.
CONFIGS: Dict[str, dict] = {
    "A": dict(architectures=["Qwen2ForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=176,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6,
              rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=True),
    "B": dict(architectures=["Qwen2ForCausalLM"], vocab_size=512, hidden_size=128, intermediate_size=344,
              num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-5,
              rope_theta=1000000.0, max_position_embeddings=512, tie_word_embeddings=False),
    "C": dict(architectures=["Qwen2ForCausalLM"], vocab_size=301, hidden_size=72, intermediate_size=136,
              num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3, head_dim=48, rms_norm_eps=3e-5,
              rope_theta=500000.0, max_position_embeddings=192, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=20, max_window_layers=2),
    # the head size of the tcgen05 attention kernel, prompts long enough for its tiles of 128 rows and
    # blocks of 128 keys, a window on the second layer that cuts through them
    "D": dict(architectures=["Qwen2ForCausalLM"], vocab_size=400, hidden_size=96, intermediate_size=200,
              num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
              rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=150, max_window_layers=1),
}
# Two layers of real layer widths: those of Qwen2-7B (v1/models/qwen2-7b/inference_fp16.dag:1-14: hidden 3584,
# intermediate 18944, 28 heads over 4 KV heads of 128, vocabulary 152064, separate output head) and those of the
# 0.5B model of the family (896 / 4864, 14 heads over 2 of 64, tied head).  The products then take the tiles, the
# cuts of the inner dimension and the CTA counts that a served model takes; the plain implementation on the CPU
# still answers in seconds because there are two layers and a few hundred tokens.
CONFIGS["W7"] = dict(architectures=["Qwen2ForCausalLM"], vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                     num_hidden_layers=2, num_attention_heads=28, num_key_value_heads=4, rms_norm_eps=1e-6,
                     rope_theta=1000000.0, max_position_embeddings=4096, tie_word_embeddings=False,
                     sliding_window=131072, use_sliding_window=False, max_window_layers=28)
CONFIGS["W05"] = dict(architectures=["Qwen2ForCausalLM"], vocab_size=151936, hidden_size=896, intermediate_size=4864,
                      num_hidden_layers=2, num_attention_heads=14, num_key_value_heads=2, rms_norm_eps=1e-6,
                      rope_theta=1000000.0, max_position_embeddings=4096, tie_word_embeddings=True)
SIGMA = {"A": 0.02, "B": 0.05, "C": 0.08, "D": 0.06, "W7": 0.02, "W05": 0.02}
SEED = {"A": 11, "B": 22, "C": 33, "D": 44, "W7": 55, "W05": 66}
# request lengths of the replay tests: a single token, page edges (16, 32), beyond 32 for the
# one-by-one tail, several pages
LENGTHS = {"A": [5, 17, 33, 70, 100], "B": [1, 8, 31, 70, 129], "C": [3, 16, 48, 81, 120], "D": [44, 150, 333, 64],
           "W7": [40, 129, 300, 64, 77, 200, 50, 100], "W05": [40, 129, 300, 64, 77, 200, 50, 100]}

# Tolerances on |logit - plain logit|, measured and pinned.  The 32-bit path differs from the plain implementation
# (float64) by the rounding and the order of its sums only.  The bfloat16 path rounds activations to 8 bits of
# mantissa at every part, so its error goes with the spread of a model's logits (config A's have a standard
# deviation of 0.17, B to D's of 0.6, the real widths' of 1.2) and with the square root of the depth.
# Worst difference over the four ways of cutting and the wide decode steps, measured on a B200:
#              A        B        C        D        W05 (0.5B widths)   W7 (7B widths)
#   bfloat16   2.2e-3   1.74e-2  1.47e-2  1.61e-2  2.44e-2             8.82e-2
#   float32    4.2e-7   2.2e-6   1.8e-6   2.0e-6   7.7e-6              4.26e-5   (sums of 18,944 terms at W7)
# The bfloat16 bound of a named configuration is three times its measured worst; that of any other model (a
# test's own weights) is three times the largest ratio to the spread of the plain logits measured on the tiny
# configurations (0.030, B).  The 32-bit bound is 2e-5 for the tiny configurations (ten times the worst measured,
# so that another order of the same sums still passes) and three times the measured worst at the real widths.
MEASURED = {"bfloat16": {"A": 2.2e-3, "B": 1.74e-2, "C": 1.47e-2, "D": 1.61e-2, "W05": 2.44e-2, "W7": 8.82e-2},
            "float32": {"W05": 7.7e-6, "W7": 4.26e-5}}
BF16_OF_SPREAD = 0.09
F32_ABS = 2e-5


def tol(dtype: str, name: str = None, ref=None) -> float:
    """The bound on |logit - plain logit| for a model: of the named configuration, or of the model whose plain
    logits are ``ref``."""
    if name is not None and name in MEASURED[dtype]:
        return 3.0 * MEASURED[dtype][name]
    if dtype == "float32":
        return F32_ABS if ref is None else F32_ABS * max(1.0, float(ref.double().std()))
    if ref is None:
        raise ValueError("a bfloat16 bound needs the configuration's name or the model's plain logits")
    return BF16_OF_SPREAD * float(ref.double().std())


def make_config(name: str):
    from vt_transformer_b200.config import config_from_dict
    return config_from_dict(CONFIGS[name])


def make_folder(name: str, folder: str) -> str:
    from vt_transformer_b200.weights import write_random_model
    return write_random_model(make_config(name), folder, seed=SEED[name], sigma=SIGMA[name])


def prompts_for(name: str, seed: int = 0) -> List[List[int]]:
    rng = random.Random(1000 + seed)
    vocab = CONFIGS[name]["vocab_size"]
    return [[rng.randrange(vocab) for _ in range(n)] for n in LENGTHS[name]]


_plain_cache: Dict[Tuple[str, Tuple[int, ...]], torch.Tensor] = {}


def plain_logits(folder: str, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] (float64) of the plain implementation for the whole sequence."""
    from plain import qwen2_plain as plain
    key = (folder, tuple(tokens))
    if key not in _plain_cache:
        cfg, w = plain.read_config(folder), _plain_weights(folder)
        _plain_cache[key] = plain.forward(cfg, w, list(tokens))
    return _plain_cache[key]


_weights_cache: Dict[str, dict] = {}


def _plain_weights(folder: str):
    from plain import qwen2_plain as plain
    if folder not in _weights_cache:
        _weights_cache[folder] = plain.read_weights(folder)
    return _weights_cache[folder]


# ----------------------------------------------------------------------------- traces
# A trace is a list of steps {"step", "entries": [{"id", "tokens", "want"}], "end"}; `expect`
# lists for each step the (request, position) of every wanted row, in order.


class Trace:
    def __init__(self):
        self.steps: List[dict] = []
        self.expect: Dict[int, List[Tuple[int, int]]] = {}

    def add(self, entries: List[Tuple[int, int, int]], prompts, end=(), want_all=True, tag=""):
        """entries: (request index, first position, n tokens); wants every position."""
        n = len(self.steps)
        recs, exp = [], []
        for r, a, k in entries:
            want = list(range(k)) if want_all else [k - 1]
            recs.append({"id": f"{tag}r{r}", "tokens": prompts[r][a:a + k], "want": want})
            exp += [(r, a + w) for w in want]
        self.steps.append({"step": n, "entries": recs, "end": [f"{tag}r{r}" for r in end]})
        if exp:
            self.expect[n] = exp

    def extend(self, other: "Trace"):
        base = len(self.steps)
        for s in other.steps:
            s = dict(s)
            s["step"] += base
            self.steps.append(s)
        for k, v in other.expect.items():
            self.expect[k + base] = v


def trace_whole(prompts, tag="w") -> Trace:
    t = Trace()
    for r, p in enumerate(prompts):
        t.add([(r, 0, len(p))], prompts, end=[r], tag=tag)
    return t


def trace_tail(prompts, tail=32, tag="t") -> Trace:
    """Most of each request in one step, its last `tail` tokens one by one."""
    t = Trace()
    for r, p in enumerate(prompts):
        head = max(1, len(p) - tail)
        t.add([(r, 0, head)], prompts, tag=tag, end=[r] if head == len(p) else [])
        for a in range(head, len(p)):
            t.add([(r, a, 1)], prompts, end=[r] if a == len(p) - 1 else [], tag=tag)
    return t


def trace_portions(prompts, sizes=(2, 3, 5, 8, 13, 2, 21, 4), tag="p") -> Trace:
    """Each request alone in portions of changing size, down to two tokens."""
    t = Trace()
    for r, p in enumerate(prompts):
        a, i = 0, r
        while a < len(p):
            k = min(sizes[i % len(sizes)], len(p) - a)
            t.add([(r, a, k)], prompts, end=[r] if a + k == len(p) else [], tag=tag)
            a, i = a + k, i + 1
    return t


def trace_mixed(prompts, max_live=4, seed=0, tag="m", decode_tail=6) -> Trace:
    """Up to `max_live` live requests: portions of some beside single tokens of others; a
    request skips a step now and then; finished requests make room for the next."""
    rng = random.Random(seed)
    t = Trace()
    order = list(range(len(prompts)))
    rng.shuffle(order)
    done = {r: 0 for r in order}
    live: List[int] = []
    while order or live:
        while order and len(live) < max_live:
            live.append(order.pop(0))
        entries = []
        for r in live:
            left = len(prompts[r]) - done[r]
            if len(live) > 1 and rng.random() < 0.2:
                continue   # sits this step out
            k = 1 if left <= decode_tail else min(left - decode_tail, rng.choice([2, 3, 7, 16, 25]))
            entries.append((r, done[r], k))
        if not entries:
            r = live[0]
            entries.append((r, done[r], 1))
        ends = []
        for r, a, k in entries:
            done[r] += k
            if done[r] == len(prompts[r]):
                ends.append(r)
                live.remove(r)
        t.add(entries, prompts, end=ends, tag=tag)
    return t


def tokens_needed(trace: Trace, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to `round_to`."""
    held: Dict[str, int] = {}
    most = 0
    for s in trace.steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most


def run_trace_cli(folder: str, trace: Trace, dtype: str, out_dir: str, max_tokens: int, extra=()) -> Dict[int, np.ndarray]:
    """Replays the trace with bin/trace_run in a process of its own and reads the logits back."""
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), *extra]
    res = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, f"trace_run failed ({res.returncode}):\n{res.stdout[-2000:]}\n{res.stderr[-4000:]}"
    done = [l for l in res.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in trace.steps], "a `done` line is missing"
    vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
    out = {}
    for n in trace.expect:
        arr = np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4")
        out[n] = arr.reshape(-1, vocab)
    return out


def run_trace_inproc(runner, trace: Trace) -> Dict[int, np.ndarray]:
    """Replays the trace on a ModelRunner in this process (the code path of bin/trace_run)."""
    from vt_transformer_b200.engine.batch import StepEntry
    rows, out = {}, {}
    for s in trace.steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in rows:
                rows[e["id"]] = runner.admit()
            entries.append(StepEntry(rows[e["id"]], e["tokens"], e["want"]))
        logits = runner.step(entries)
        runner.check_status()
        if logits.shape[0]:
            out[s["step"]] = logits.float().cpu().numpy()
        for rid in s["end"]:
            runner.release(rows.pop(rid))
        runner.cache.check()
    return out


def compare_trace(folder: str, prompts, trace: Trace, got: Dict[int, np.ndarray], tol: float) -> float:
    """Every wanted row against the plain implementation; returns the largest difference and
    fails at the first row beyond `tol`, saying where it lies."""
    worst = 0.0
    for n in sorted(trace.expect):
        exp = trace.expect[n]
        assert got[n].shape[0] == len(exp), f"step {n}: {got[n].shape[0]} rows, {len(exp)} wanted"
        for i, (r, pos) in enumerate(exp):
            ref = plain_logits(folder, prompts[r])[pos].numpy()
            d = float(np.abs(got[n][i].astype(np.float64) - ref).max())
            assert np.isfinite(d) and d <= tol, (
                f"step {n}, request {r} (length {len(prompts[r])}), position {pos}: |dlogit| {d:.3e} > {tol:.1e} "
                f"(entries {[(e['id'], len(e['tokens'])) for e in trace.steps[n]['entries']]})")
            worst = max(worst, d)
    return worst


def step_context(q_lens, starts, device, status=None):
    """A StepContext for sequences whose new tokens are `q_lens` long and start at positions
    `starts` (no block tables: tests of parts pass theirs in the cache view)."""
    from vt_transformer_b200.engine.batch import SeqSlice, StepContext
    seqs, off, pos, tseq = [], 0, [], []
    for i, (n, s) in enumerate(zip(q_lens, starts)):
        seqs.append(SeqSlice(i, s, n, off))
        pos += list(range(s, s + n))
        tseq += [i] * n
        off += n
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return StepContext(n_tokens=off, n_seqs=len(q_lens), seqs=seqs, token_ids=t([0] * off), positions=t(pos),
                       token_seq=t(tseq), cu_q=t([s.offset for s in seqs] + [off]), q_start=t(list(starts)),
                       kv_len=t([s + n for s, n in zip(starts, q_lens)]), rows=t(list(range(len(q_lens)))),
                       want_rows=t([]), block_tables={}, max_q_len=max(q_lens), max_kv_len=max(s + n for s, n in zip(starts, q_lens)),
                       status=status)
