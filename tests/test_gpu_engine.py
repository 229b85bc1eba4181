"""The engine on the GPU with the real kernels, in 32-bit and in bfloat16, against the plain
implementation: every way of cutting, run orders, a toy mixer, generation."""
import pytest
import torch

import helpers
import scenarios

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(folders, name, family, dtype):
    scenarios.replay_family(folders(name), name, family, DEV, dtype)


@pytest.mark.parametrize("family", ["tail", "mixed"])
def test_decoding_with_keys_and_values_fetched_as_tensor_map_boxes(folders, family):
    """Head size 128 (one layer with a window): the engine fetches a decode step's keys as boxes only for long
    contexts; here it is made to do so for these short ones, pages of 16, used again."""
    from vt_transformer_b200 import ops as o
    old = o.DECODE_BOXES
    o.DECODE_BOXES = "always"
    try:
        scenarios.replay_family(folders("D"), "D", family, DEV, "bfloat16")
    finally:
        o.DECODE_BOXES = old


@pytest.mark.parametrize("dtype", DTYPES)
def test_run_order_is_data(tmp_path, dtype):
    scenarios.run_order_case(str(tmp_path), DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    scenarios.toy_state_case(str(tmp_path), DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_feed_forward_with_routing_and_another_position_encoding(tmp_path, dtype):
    scenarios.toy_routed_case(str(tmp_path), DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_norm_cache_kind_and_the_models_two_ends(tmp_path, dtype):
    scenarios.toy_seams_case(str(tmp_path), DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    scenarios.greedy_generation_case(folders(name), name, DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_temperature_generation_survives_recutting_and_preemption(folders, dtype):
    scenarios.temperature_generation_case(folders("B"), "B", DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_next_step_enqueued_early_changes_no_token(folders, dtype):
    scenarios.overlap_generation_case(folders("B"), "B", DEV, dtype)


def test_each_part_knows_which_matrix_streams_next_and_the_hint_changes_no_logit(folders):
    """Once the weights are loaded the model tells every run's block what the step streams after it: the mixer's
    last product is followed by the feed-forward's first, the feed-forward's by the next run's first, the last run's
    by the head's.  With the hints off, a prompt and single-token steps give the same bits."""
    from vt_transformer_b200 import ops as o
    from vt_transformer_b200.engine import StepEntry
    folder = folders("A")
    ids = helpers.prompts_for("A")[2]
    logits = {}
    for n_bytes in (o.LOOK_AHEAD_BYTES or (8 << 20), 0):
        old, o.LOOK_AHEAD_BYTES = o.LOOK_AHEAD_BYTES, n_bytes
        try:
            runner = scenarios.runner_for(folder, DEV, "bfloat16", num_pages=8, max_requests=2)
            model = runner.model
            order = model.spec.order
            for n, run in enumerate(order):
                block = model.blocks[run.block]
                after = model.blocks[order[n + 1].block].mixer.w_qkv if n + 1 < len(order) else model.head.weight
                assert block.mixer.then[0] is block.ffn.w_gate_up and block.mixer.then[1] == 1
                assert block.ffn.then[0] is after and block.ffn.then[1] == (2 if n + 1 < len(order) else 0)
            row = runner.admit()
            got = [runner.step([StepEntry(row, ids[:9], [8])]).clone()]
            for t in range(9, 14):
                got.append(runner.step([StepEntry(row, ids[t:t + 1], [0])]).clone())
            runner.check_status()
            logits[n_bytes] = torch.cat(got)
        finally:
            o.LOOK_AHEAD_BYTES = old
    with_hints, without = logits.values()
    assert torch.equal(with_hints, without)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(folders, dtype):
    """One token, two tokens, three: the first positions, where the cache is empty and a
    portion is shorter than any tile."""
    from vt_transformer_b200.engine import StepEntry
    folder = folders("B")
    ids = helpers.prompts_for("B")[3]
    ref = helpers.plain_logits(folder, ids)
    runner = scenarios.runner_for(folder, DEV, dtype, num_pages=4, max_requests=4)
    for n in (1, 2, 3):
        row = runner.admit()
        got = runner.step([StepEntry(row, ids[:n], list(range(n)))]).double().cpu()
        assert float((got - ref[:n]).abs().max()) <= helpers.tol(dtype, "B")
        for t in range(n, n + 3):                            # and three single tokens after them
            got = runner.step([StepEntry(row, ids[t:t + 1], [0])]).double().cpu()
            assert float((got[0] - ref[t]).abs().max()) <= helpers.tol(dtype, "B"), (n, t)
        runner.release(row)
    runner.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    """A short prompt and then 230 tokens one by one, beside a second request that joins late:
    the cache grows over many pages, one token at a time."""
    from vt_transformer_b200.engine import StepEntry
    folder = folders("A")
    rng_ids = helpers.prompts_for("A", seed=5)
    ids = (rng_ids[4] + rng_ids[3] + rng_ids[2] + rng_ids[1] + rng_ids[0] + rng_ids[4])[:240]
    other = rng_ids[3]
    ref, ref_other = helpers.plain_logits(folder, ids), helpers.plain_logits(folder, other)
    runner = scenarios.runner_for(folder, DEV, dtype, num_pages=21, max_requests=2)
    a = runner.admit()
    worst = float((runner.step([StepEntry(a, ids[:10], [9])]).double().cpu()[0] - ref[9]).abs().max())
    b, done_b = None, 0
    for t in range(10, 240):
        entries = [StepEntry(a, ids[t:t + 1], [0])]
        if t == 100:
            b = runner.admit()
        if b is not None and done_b < len(other):
            k = min(7, len(other) - done_b)
            entries.append(StepEntry(b, other[done_b:done_b + k], [k - 1]))
        got = runner.step(entries).double().cpu()
        worst = max(worst, float((got[0] - ref[t]).abs().max()))
        if len(entries) == 2:
            done_b += k
            worst = max(worst, float((got[1] - ref_other[done_b - 1]).abs().max()))
    runner.check_status()
    assert worst <= helpers.tol(dtype, "A"), worst


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_is_found(tmp_path, dtype):
    """Random weights give flat attention, which hides a key that is read from the wrong place.
    Here the queries and keys of layer 0 are scaled up so that the scores are sharp and every
    token attends to a few keys that differ from token to token: a key missed at a page's
    edge, in a page that was used before, or far back, changes the logits by far more than
    the tolerance."""
    from vt_transformer_b200.engine import StepEntry
    from vt_transformer_b200.weights import SafetensorsSource, write_random_model
    from vt_transformer_b200.weights import safetensors_io as st
    import os
    # bfloat16 rounds q and k to 8 bits, and a score of size s is then off by s / 256: sharper
    # scores than these would turn that rounding itself into a large change of the weights
    sharp = 6.0 if dtype == "float32" else 3.0
    src_folder = write_random_model(helpers.make_config("B"), str(tmp_path / "src"), seed=41, sigma=0.05)
    src = SafetensorsSource(src_folder)
    tensors = {n: src.get(n).clone() for n in src.entries()}
    for proj in ("q_proj", "k_proj"):
        for kind in ("weight", "bias"):
            name = f"model.layers.0.self_attn.{proj}.{kind}"
            tensors[name] = (tensors[name].float() * sharp).to(torch.bfloat16)
    folder = str(tmp_path / "sharp")
    os.makedirs(folder)
    helpers.make_config("B").save(folder)
    st.write_file(os.path.join(folder, "model.safetensors"), iter(tensors.items()),
                  [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()])
    ids = (helpers.prompts_for("B", seed=8)[4] * 3)[:380]
    ref = helpers.plain_logits(folder, ids)
    flat = helpers.plain_logits(src_folder, ids)
    assert float((ref - flat).abs().max()) > 5 * helpers.tol(dtype, ref=ref)        # the scaling matters
    runner = scenarios.runner_for(folder, DEV, dtype, num_pages=26, max_requests=2)
    # a first request fills and frees pages, so the long one lives in pages that were used before
    warm = runner.admit()
    runner.step([StepEntry(warm, ids[:200][::-1], [])])
    runner.release(warm)
    row = runner.admit()
    got, a = [], 0
    for k in (300, 17, 1, 1, 1, 30, 2, 28):
        got.append(runner.step([StepEntry(row, ids[a:a + k], list(range(k)))]).double().cpu())
        a += k
    runner.check_status()
    err = float((torch.cat(got) - ref).abs().max())
    assert err <= helpers.tol(dtype, ref=ref), (err, float((ref - flat).abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(folders, dtype):
    """Config C's late layers see 20 keys.  Positions around the edge (19, 20, 21), around the
    pages' edges, and with the window cutting through a portion are compared one by one."""
    from vt_transformer_b200.engine import StepEntry
    folder = folders("C")
    ids = helpers.prompts_for("C")[4]
    ref = helpers.plain_logits(folder, ids)
    runner = scenarios.runner_for(folder, DEV, dtype, num_pages=8, max_requests=2)
    row = runner.admit()
    got, a = [], 0
    for k in (19, 1, 1, 1, 10, 16, 1, 31, 2, 38):
        got.append(runner.step([StepEntry(row, ids[a:a + k], list(range(k)))]).double().cpu())
        a += k
        runner.cache.check()
    assert a == len(ids)
    win = [g for g in runner.cache.groups if g.spec.window][0]
    assert win.pool.free >= win.pool.num_pages - 3               # pages behind the window went back
    runner.check_status()
    err = (torch.cat(got) - ref).abs().max(dim=1).values
    assert float(err.max()) <= helpers.tol(dtype, "C"), (int(err.argmax()), float(err.max()))


def test_a_folder_stored_in_32_bit_rounded_at_load_runs_the_bfloat16_kernels(tmp_path):
    """A model stored in float32, loaded in bfloat16 mode: with fp32_weights="round" its matrices are bfloat16 (the
    tcgen05 products run) and the logits are those of a folder that stores the rounded values, bit for bit; kept in
    32-bit (the default, with a warning) the products run the 32-bit kernel and the logits are within the bound."""
    from test_weights import wide_and_rounded_folders
    from vt_transformer_b200.engine import ModelRunner, StepEntry
    wide, rounded = wide_and_rounded_folders(str(tmp_path))
    ids = helpers.prompts_for("B")[4]
    kw = dict(dtype="bfloat16", device=DEV, page_size=16, num_pages=10, max_requests=1)

    def logits(runner):
        out = runner.step([StepEntry(runner.admit(), ids, list(range(len(ids))))])
        runner.check_status()
        return out

    cut = ModelRunner.from_folder(wide, fp32_weights="round", **kw)
    ref = ModelRunner.from_folder(rounded, **kw)
    assert cut.model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16 and cut.model.blocks[0].ffn.w_gate_up.dtype == torch.bfloat16
    got, want = logits(cut), logits(ref)
    assert torch.equal(got, want)
    with pytest.warns(UserWarning, match="stay so"):
        kept = ModelRunner.from_folder(wide, **kw)
    assert kept.model.blocks[0].mixer.w_qkv.dtype == torch.float32
    plain_ref = helpers.plain_logits(rounded, ids)
    assert float((logits(kept).double().cpu() - plain_ref).abs().max()) <= helpers.tol("bfloat16", ref=plain_ref)
    assert float((want.double().cpu() - plain_ref).abs().max()) <= helpers.tol("bfloat16", ref=plain_ref)


def test_mixed_step_with_decoding_requests_first(folders):
    """A step as a scheduler makes it: five decoding requests first (one token each, contexts of 43 to 332 tokens),
    then portions of two prompts.  At head size 128 the portions run the tcgen05 kernel and the single tokens at the
    head of the batch a launch of the single-token kernel of their own; a second such step has a single token behind
    a portion as well (that one runs with the portions).  Every row against the plain implementation."""
    from vt_transformer_b200 import ops
    from vt_transformer_b200.engine import StepEntry
    folder = folders("D")
    prompts = helpers.prompts_for("D") + helpers.prompts_for("D", seed=3)[:3]      # 44, 150, 333, 64, 44, 150, 333 tokens
    runner = scenarios.runner_for(folder, DEV, "bfloat16", num_pages=80, max_requests=7, page_size=16)
    rows = [runner.admit() for _ in prompts]
    for r, p in zip(rows[:5], prompts[:5]):
        runner.step([StepEntry(r, p[:-2], [])])
    before = ops.launches
    entries = [StepEntry(r, [p[-2]], [0]) for r, p in zip(rows[:5], prompts[:5])]
    entries += [StepEntry(rows[5], prompts[5][:100], list(range(100))), StepEntry(rows[6], prompts[6][:60], list(range(60)))]
    got = runner.step(entries).double().cpu()
    layers = len(runner.model.blocks)
    assert ops._leading_single_tokens(scenarios.helpers.step_context([1] * 5 + [100, 60], [0] * 7, "cpu")) == 5
    entries2 = [StepEntry(r, [p[-1]], [0]) for r, p in zip(rows[:4], prompts[:4])]
    entries2 += [StepEntry(rows[5], prompts[5][100:], [len(prompts[5]) - 101]), StepEntry(rows[4], [prompts[4][-1]], [0])]
    got2 = runner.step(entries2).double().cpu()
    runner.check_status()
    bound = helpers.tol("bfloat16", "D")
    at = 0
    for i, p in enumerate(prompts[:5]):
        assert float((got[at] - helpers.plain_logits(folder, p)[len(p) - 2]).abs().max()) <= bound, i
        at += 1
    for i, n in ((5, 100), (6, 60)):
        assert float((got[at:at + n] - helpers.plain_logits(folder, prompts[i])[:n]).abs().max()) <= bound, i
        at += n
    for j, i in enumerate((0, 1, 2, 3)):
        assert float((got2[j] - helpers.plain_logits(folder, prompts[i])[-1]).abs().max()) <= bound, i
    assert float((got2[4] - helpers.plain_logits(folder, prompts[5])[-1]).abs().max()) <= bound
    assert float((got2[5] - helpers.plain_logits(folder, prompts[4])[-1]).abs().max()) <= bound


def test_status_word_reports_a_bad_token_id(folders):
    from vt_transformer_b200.engine import DeviceStatusError, StepEntry
    runner = scenarios.runner_for(folders("A"), DEV, "float32", num_pages=2, max_requests=1)
    row = runner.admit()
    runner.step([StepEntry(row, [1, 2, 100000], [2])])
    with pytest.raises(DeviceStatusError, match="token id"):
        runner.check_status()
    runner.check_status()                                        # the word was cleared
