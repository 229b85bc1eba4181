"""The engine's host-side logic on the CPU: the step function, the cache manager and the
scheduler drive stand-in kernels (tests/fake_ops.py) and are compared with the plain
implementation.  The same scenarios run on the GPU with the real kernels in
test_gpu_engine.py."""
import pytest
import torch

import helpers
import scenarios

DEV, DT = "cpu", "float32"


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(fake_backend, folders, name, family):
    scenarios.replay_family(folders(name), name, family, DEV, DT)


def test_run_order_is_data(fake_backend, tmp_path):
    scenarios.run_order_case(str(tmp_path), DEV, DT)


def test_bad_run_orders_are_refused(fake_backend):
    from dataclasses import replace
    from vt_transformer_b200.models import DecoderModel
    from vt_transformer_b200.models.qwen2 import qwen2_model_spec
    from vt_transformer_b200.parts import RunSpec, Runtime
    spec = qwen2_model_spec(helpers.make_config("A"))
    rt = Runtime(torch.device("cpu"), torch.float32, None)
    for order, word in (((RunSpec(0, 0), RunSpec(1, 0)), "written by an earlier run"),
                        ((RunSpec(0, 0, writes=False),), "before any run wrote"),
                        ((RunSpec(5, 0),), "names block 5"),
                        ((RunSpec(0, None),), "names no slot")):
        with pytest.raises(ValueError, match=word):
            DecoderModel(replace(spec, order=order), rt)


def test_the_model_tells_each_part_which_matrix_streams_next(fake_backend, folders, monkeypatch):
    """After loading, every run's block knows the first product of what runs after it (the next run's block, the
    head after the last); the mixer's last product is followed by the feed-forward's first.  A matrix that the
    tcgen05 kernel does not take (here: 32-bit on the CPU) gives no hint at all."""
    from vt_transformer_b200 import ops
    runner = scenarios.runner_for(folders("A"), DEV, DT, num_pages=4, max_requests=1)
    for block in runner.model.blocks:
        assert block.mixer.then is None and block.ffn.then is None and block.first_product() is None
    monkeypatch.setattr(ops, "product_hint", lambda w, kind: (w, kind))
    model = runner.model
    model._link_runs()
    order = model.spec.order
    assert len(order) >= 2
    for n, run in enumerate(order):
        block = model.blocks[run.block]
        assert block.mixer.then[0] is block.ffn.w_gate_up and block.mixer.then[1] == "silu_mul"
        if n + 1 < len(order):
            assert block.ffn.then[0] is model.blocks[order[n + 1].block].mixer.w_qkv and block.ffn.then[1] == "stream"
        else:
            assert block.ffn.then[0] is model.head.weight and block.ffn.then[1] == "linear"


def test_toy_mixer_with_state_is_registered_built_and_stepped(fake_backend, tmp_path):
    scenarios.toy_state_case(str(tmp_path), DEV, DT)


def test_toy_feed_forward_with_routing_and_another_position_encoding(fake_backend, tmp_path):
    scenarios.toy_routed_case(str(tmp_path), DEV, DT)


def test_toy_norm_cache_kind_and_the_models_two_ends(fake_backend, tmp_path):
    scenarios.toy_seams_case(str(tmp_path), DEV, DT)


def test_end_tokens_and_position_limit_come_from_the_model_spec(fake_backend, tmp_path):
    """An architecture whose configuration names things its own way: the engine reads the positions a model can
    hold and the tokens that end a request from the ModelSpec, not from a configuration key."""
    import copy
    from dataclasses import replace
    from vt_transformer_b200 import LLM
    from vt_transformer_b200.config import Qwen2Config, config_from_dict, register_architecture, unregister_architecture
    from vt_transformer_b200.models.qwen2 import qwen2_model_spec
    from vt_transformer_b200.weights import write_random_model

    def spec(cfg):
        return replace(qwen2_model_spec(cfg), max_positions=48, eos_token_ids=(7, 9))

    register_architecture("ToyLimitsLM", Qwen2Config, spec, replace=True)
    try:
        d = copy.deepcopy(helpers.CONFIGS["A"])
        d["architectures"] = ["ToyLimitsLM"]
        folder = write_random_model(config_from_dict(d), str(tmp_path / "limits"), seed=2, sigma=0.05)
        llm = LLM(folder, dtype=DT, device=DEV, max_running_reqs=2, page_size=16)
        assert llm.scheduler.eos == (7, 9) and llm.runner.cache.max_seq_len == 48
    finally:
        unregister_architecture("ToyLimitsLM")


def test_an_unknown_kind_of_cache_spec_is_refused_by_name():
    from vt_transformer_b200.cache import CacheManager
    with pytest.raises(TypeError, match="cache slot 3: unknown kind of cache spec.*register_cache_kind"):
        CacheManager({3: object()}, page_size=16, num_pages=2, max_requests=1, max_seq_len=32, dtype=torch.float32,
                     device="cpu", allocate=False)


def test_attention_refuses_a_rotation_of_part_of_the_head():
    from vt_transformer_b200.parts import AttentionSpec, PositionSpec, Runtime, build_part
    rt = Runtime(torch.device("cpu"), torch.float32, None)
    spec = AttentionSpec(hidden=64, heads=4, kv_heads=2, head_dim=16, position=PositionSpec(dim=8, base=1e4, max_positions=32))
    with pytest.raises(ValueError, match="covers 8 of the head's 16"):
        build_part("mixer", spec, "x.", rt)


def test_step_refuses_bad_entries_and_leaves_the_cache_alone(fake_backend, folders):
    from vt_transformer_b200.cache import OutOfPages
    from vt_transformer_b200.engine import StepEntry
    runner = scenarios.runner_for(folders("A"), DEV, DT, num_pages=2, max_requests=2, max_seq_len=64)
    a, b = runner.admit(), runner.admit()
    with pytest.raises(ValueError, match="twice"):
        runner.step([StepEntry(a, [1, 2]), StepEntry(a, [3])])
    with pytest.raises(ValueError, match="outside"):
        runner.step([StepEntry(a, [1, 2], [2])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry(a, [1] * 20, [0]), StepEntry(b, [2] * 20, [0])])
    assert runner.cache.free_pages() == [2] and runner.cache.length(a) == 0
    out = runner.step([StepEntry(a, [1] * 20, [19, 0, 19])])      # a place may be wanted twice
    assert out.shape == (3, 256) and torch.equal(out[0], out[2]) and not torch.equal(out[0], out[1])
    assert runner.step([]).shape == (0, 256)
    assert runner.step([StepEntry(a, [5], [])]).shape == (0, 256) and runner.cache.length(a) == 21


def test_greedy_generation(fake_backend, folders):
    scenarios.greedy_generation_case(folders("A"), "A", DEV, DT)


def test_temperature_generation_survives_recutting_and_preemption(fake_backend, folders):
    out, pre = scenarios.temperature_generation_case(folders("B"), "B", DEV, DT)
    assert pre[0] == 0


def test_the_next_step_enqueued_early_changes_no_token(fake_backend, folders):
    scenarios.overlap_generation_case(folders("B"), "B", DEV, DT)


def test_missing_extension_fails_loudly():
    from vt_transformer_b200 import ops
    ops.use_backend(None)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU path"):
            ops.backend()


def test_single_token_steps_cut_their_keys_by_the_work_and_fetch_by_boxes_where_that_pays():
    """How a decode step's keys are cut over CTAs, and the choice between cp.async copies and tensor-map boxes for
    them, are made on the host (148 SMs assumed where there is no device)."""
    import torch
    from vt_transformer_b200 import ops as o
    dev = torch.device("cpu")
    o._sm_counts[dev] = 148
    try:
        # batch 8 of 4 KV heads under a bound of 2,048 keys: a typical sequence (64 blocks) is cut into a cluster of
        # three runs of 22 blocks; a sequence of 1,040 keys (65 blocks) takes all three, one at the bound longer runs
        assert o._decode_plan(32, 2048, dev) == (3, 22, False)
        # batch 64: a CTA a (sequence, KV head) already fills the SMs: no cut
        assert o._decode_plan(256, 2048, dev) == (1, 0, False)
        # one sequence of up to 4,096 keys: runs of 32 blocks (not shorter: a run has its fixed cost), met in scratch memory
        assert o._decode_plan(2, 4096, dev) == (8, 32, True)
        # one sequence of 4 KV heads of up to 32,768 keys: no more runs than give every SM one CTA of eight warps
        assert o._decode_plan(4, 32768, dev) == (37, 32, True)
        # 32 sequences of 2 KV heads under a bound of 16,384 keys: their lengths may differ by thousands of keys, so
        # up to 7 runs of 148 blocks meet in scratch memory and a short sequence takes one CTA
        assert o._decode_plan(64, 16384, dev) == (7, 148, True)
        # the same 64 (sequence, KV head) under that bound with lengths alike (all of 4,096 keys or more): the runs stay
        # the CTAs of a cluster, sized for a typical sequence; one or two sequences of like lengths still meet in scratch
        assert o._decode_plan(64, 16384, dev, 4096) == (2, 341, False)
        assert o._decode_plan(4, 32768, dev, 8192) == (37, 32, True)
        # a short bound is not cut
        assert o._decode_plan(8, 200, dev) == (1, 0, False)
        # boxes: where a warp streams 16 blocks or more (batch 64 at 4,096 keys), not where it has few, however many CTAs
        assert not o._decode_long_runs(256, 1040, 1, 0, 128, dev) and o._decode_long_runs(256, 1040, 1, 0, 64, dev)
        assert o._decode_long_runs(256, 4096, 2, 128, 128, dev) and o._decode_long_runs(256, 2048, 1, 0, 64, dev)
        assert not o._decode_long_runs(32, 2048, 3, 22, 128, dev)
        assert o._decode_long_runs(8, 32768, 1, 0, 128, dev)
        assert not o._decode_long_runs(256, 4096, 2, 128, 80, dev)        # other head sizes have no boxes
        old = o.DECODE_BOXES
        try:
            o.DECODE_BOXES = "never"
            assert not o._decode_long_runs(256, 4096, 2, 128, 128, dev)
            o.DECODE_BOXES = "always"
            assert o._decode_long_runs(32, 2048, 3, 22, 128, dev) and not o._decode_long_runs(32, 2048, 3, 22, 96, dev)
        finally:
            o.DECODE_BOXES = old
    finally:
        del o._sm_counts[dev]
