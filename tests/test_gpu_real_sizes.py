"""The engine at real layer widths, and decode steps of many requests, against the plain implementation.

Two layers of Qwen2-7B's widths (hidden 3584, intermediate 18944, 28 heads over 4 KV heads of 128, vocabulary
152064, separate head: v1/models/qwen2-7b/inference_fp16.dag:1-14) and of the 0.5B model's (896 / 4864, 14 heads
over 2 of 64, tied head), random weights written as a folder.  At these widths the bfloat16 products run the tiles,
the cuts of the inner dimension over CTAs, the shares left for the norm and the fused single-token attention that
a served model runs; the tiny configurations of the other tests are too narrow for most of them.

Decode steps of 7 to 70 live requests run at the tiny widths (the plain implementation answers for 70 requests
in seconds there) and, at batch 8, at the 7B widths: CUDA graphs of the batch buckets 8, 48 and 96 with padding
rows, a context that grows across a context bucket while it decodes, and a step whose keys are cut into more runs
than a thread-block cluster holds.
"""
import random

import pytest
import torch

import helpers
import scenarios

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
WIDTHS = ["W05", "W7"]


@pytest.fixture(scope="module", autouse=True)
def _free_the_shared_models():
    yield
    scenarios.forget_shared_models()
    helpers._weights_cache.clear()
    helpers._plain_cache.clear()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", WIDTHS)
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_at_real_widths(folders, name, family, dtype):
    """Whole (a prompt of 300 tokens: the products with x as the 128-row operand, the tcgen05 attention), the
    last 32 one by one, portions down to two tokens with one of 260, and mixed with pages used again."""
    sizes = (2, 3, 260, 5, 8, 13, 2, 21, 4) if family == "portions" else None
    worst = scenarios.replay_family_shared(folders(name), name, family, DEV, dtype, sizes=sizes)
    print(f"\n{name} {dtype} {family}: worst |dlogit| {worst:.3e}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", WIDTHS)
def test_decode_steps_of_eight_at_real_widths(folders, name, dtype):
    """Eight requests of 40 to 300 tokens decode their last six tokens together: the step that the benchmark times
    (graph bucket 8, products with the weights as the 128-row operand and k cut over CTAs, their shares added by the
    norm or by the attention kernel)."""
    folder = folders(name)
    seqs = helpers.prompts_for(name)
    worst, keys = scenarios.wide_decode_case(folder, name, DEV, dtype, seqs, decode_steps=6, page_size=64)
    print(f"\n{name} {dtype} decode of 8: worst |dlogit| {worst:.3e}, graphs {keys}")
    assert (8, 512) in keys and (8, 256) not in keys       # the longest request holds 294 to 300 tokens


def _sequences(name, n, seed, shortest=3, longest=200):
    rng = random.Random(seed)
    vocab = helpers.CONFIGS[name]["vocab_size"]
    return [[rng.randrange(vocab) for _ in range(rng.randint(shortest, longest))] for _ in range(n)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_live", [7, 8, 40, 70])
def test_decode_steps_of_many_requests(folders, n_live, dtype):
    """7, 8, 40 and 70 live requests of different lengths (config B, one of them growing from 250 to 262 tokens
    while it decodes: the context bucket changes from 256 to 512 under live requests) decode 12 tokens each in one
    step a token: graph buckets 8 (with and without a padding row), 48 and 96."""
    folder = folders("B")
    seqs = _sequences("B", n_live - 1, seed=n_live, longest=180)
    seqs.insert(n_live // 2, _sequences("B", 1, seed=100 + n_live, shortest=262, longest=262)[0])
    worst, keys = scenarios.wide_decode_case(folder, "B", DEV, dtype, seqs, decode_steps=12, page_size=16)
    print(f"\nB {dtype} decode of {n_live}: worst |dlogit| {worst:.3e}, graphs {keys}")
    from vt_transformer_b200.engine.graphs import batch_bucket
    assert keys == [(batch_bucket(n_live), 256), (batch_bucket(n_live), 512)]


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_with_keys_cut_into_more_runs_than_a_cluster_holds(tmp_path, dtype, request):
    """One request of 2,100 tokens decodes alone (head size 128, two KV heads): its keys are cut into more than
    eight runs, which meet in scratch memory and are merged by the CTA that arrives last; beside it, the same
    request in a step of three (fewer runs, merged inside a cluster)."""
    import copy
    from vt_transformer_b200 import ops
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.weights import write_random_model
    d = copy.deepcopy(helpers.CONFIGS["D"])
    d.update(max_position_embeddings=4096, use_sliding_window=False)
    folder = write_random_model(config_from_dict(d), str(tmp_path / "long"), seed=45, sigma=0.06)
    seqs = _sequences("D", 1, seed=7, shortest=2100, longest=2100)
    ref = helpers.plain_logits(folder, seqs[0])
    bound = helpers.tol(dtype, ref=ref)
    # (runs as short as a cluster's, so that this sequence is cut into more of them than a cluster holds)
    shortest, ops.DECODE_MIN_RUN_LONG = ops.DECODE_MIN_RUN_LONG, 8
    request.addfinalizer(lambda: setattr(ops, "DECODE_MIN_RUN_LONG", shortest))
    assert ops._decode_plan(2, 4096, torch.device(DEV))[0] > 8 and ops._decode_plan(2, 4096, torch.device(DEV))[2]
    for others in (0, 2):
        batch = seqs + _sequences("D", others, seed=8, longest=90)
        runner = scenarios.shared_runner(folder, DEV, dtype, num_pages=sum(-(-len(s) // 16) for s in batch),
                                         max_requests=len(batch), page_size=16)
        worst, keys = scenarios.wide_decode_case(folder, None, DEV, dtype, batch, decode_steps=8, runner=runner, bound=bound)
        print(f"\nlong context, {dtype}, {others} other requests: worst |dlogit| {worst:.3e}, graphs {keys}")
        assert keys[-1][1] == 4096


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_of_like_long_sequences_keeps_the_cluster(tmp_path, dtype):
    """Eight requests of 2,050 to 2,200 tokens (head size 128, two KV heads) decode together under a bound of 4,096
    keys: their lengths are alike (all above a quarter of the bound), so the runs of a sequence stay the CTAs of a
    cluster and do not meet in scratch memory, as they would for lengths that differ by thousands of keys."""
    import copy
    from vt_transformer_b200 import ops
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.weights import write_random_model
    d = copy.deepcopy(helpers.CONFIGS["D"])
    d.update(max_position_embeddings=4096, use_sliding_window=False)
    folder = write_random_model(config_from_dict(d), str(tmp_path / "alike"), seed=46, sigma=0.06)
    rng = random.Random(11)
    vocab = d["vocab_size"]
    seqs = [[rng.randrange(vocab) for _ in range(rng.randint(2050, 2200))] for _ in range(8)]
    bound = helpers.tol(dtype, ref=helpers.plain_logits(folder, seqs[0]))
    dev = torch.device(DEV)
    assert ops._decode_plan(16, 4096, dev, 1024)[2] is False and ops._decode_plan(16, 4096, dev, 0)[2] is True
    runner = scenarios.shared_runner(folder, DEV, dtype, num_pages=sum(-(-len(s) // 16) for s in seqs) + 8, max_requests=8, page_size=16)
    worst, keys = scenarios.wide_decode_case(folder, None, DEV, dtype, seqs, decode_steps=6, runner=runner, bound=bound)
    print(f"\nlike lengths, {dtype}: worst |dlogit| {worst:.3e}, graphs {keys}")
    assert keys[-1] == (8, 4096) and any(k == (8, 4096, True) for k in runner._graphs)


def test_all_layers_of_the_benchmark_model_in_bfloat16_against_32_bit():
    """Qwen2-7B's sizes with all 28 layers and random weights, as the benchmark runs them, built twice on the
    device: bfloat16 and 32-bit (whose kernels the tests above compare with the plain implementation at the same
    widths).  A prompt of 2,048 tokens in one step (the benchmark's prefill), a prompt of 300, and decode steps of
    eight requests through the captured graph (the benchmark's step).  The bound is that of a model of two layers
    (a share of the logits' spread) grown with the square root of the depth; measured on a B200: 0.284 at a spread
    of 1.197 (0.227 at the prefill's row), against a bound of 0.403."""
    import bench
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.engine import ModelRunner, StepEntry
    cfg = config_from_dict(dict(bench.MODEL))
    runners = {}
    for dtype in ("bfloat16", "float32"):
        runners[dtype] = ModelRunner.from_random(cfg, seed=0, sigma=0.02, dtype=dtype, device=DEV, page_size=64,
                                                 num_pages=96, max_requests=8, max_seq_len=4096)
    rng = random.Random(5)
    seqs = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (2048, 300, 40, 129, 64, 77, 200, 50)]
    got = {}
    for dtype, runner in runners.items():
        rows = [runner.admit() for _ in seqs]
        out = [runner.step([StepEntry(rows[0], seqs[0], [2047])]).double().cpu()]
        out.append(runner.step([StepEntry(rows[1], seqs[1][:-4], [295])]).double().cpu())
        runner.step([StepEntry(r, s[:-4], []) for r, s in zip(rows[2:], seqs[2:])])
        for t in range(-4, 0):
            entries = [StepEntry(r, [s[t]], [0]) for r, s in zip(rows[1:], seqs[1:])]
            entries.insert(3, StepEntry(rows[0], [seqs[0][t]], [0]))                # a step of eight single tokens
            out.append(runner.step(entries).double().cpu())
        runner.check_status()
        assert any(k[:2] == (8, 4096) for k in runner._graphs)
        got[dtype] = torch.cat(out)
    ref = got["float32"]
    err = (got["bfloat16"] - ref).abs().max(dim=1).values
    bound = helpers.BF16_OF_SPREAD * float(ref.std()) * (cfg.num_hidden_layers / 2) ** 0.5
    print(f"\n28 layers: worst |dlogit| {float(err.max()):.3e} of a spread {float(ref.std()):.3f} (bound {bound:.3e}); "
          f"prefill row {float(err[0]):.3e}, decode rows {float(err[2:].max()):.3e}")
    assert torch.isfinite(got["bfloat16"]).all() and float(err.max()) <= bound
