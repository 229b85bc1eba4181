"""bin/trace_run as a user runs it: a process of its own, steps on standard input, logits in
files.  One process for each configuration and dtype replays all four families one after the
other in a pool that is only as large as the live requests need, so pages are used again."""
import pytest

import helpers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_trace_run_replays_every_family(folders, tmp_path, name, dtype):
    folder = folders(name)
    prompts = helpers.prompts_for(name)
    trace = helpers.Trace()
    for t in (helpers.trace_whole(prompts), helpers.trace_tail(prompts), helpers.trace_portions(prompts),
              helpers.trace_mixed(prompts, max_live=4, seed=9), helpers.trace_mixed(prompts, max_live=2, seed=10, tag="n")):
        trace.extend(t)
    if name == "D":
        # portions long enough for the tcgen05 attention kernel that start in the middle of a sequence
        trace.extend(helpers.trace_portions(prompts, sizes=(60, 2, 45, 100, 3, 70), tag="q"))
    # the engine's own page size (64) for A and D, smaller pages for B and C
    extra = {"B": ("--page-size", "16"), "C": ("--page-size", "32")}.get(name, ())
    got = helpers.run_trace_cli(folder, trace, dtype, str(tmp_path / "out"), helpers.tokens_needed(trace, 64), extra)
    helpers.compare_trace(folder, prompts, trace, got, helpers.tol(dtype, name))


def test_trace_run_skips_files_for_steps_that_want_nothing(folders, tmp_path):
    import os
    folder = folders("A")
    prompts = helpers.prompts_for("A")
    trace = helpers.Trace()
    trace.steps = [{"step": 0, "entries": [{"id": "a", "tokens": prompts[1][:9], "want": []}], "end": []},
                   {"step": 1, "entries": [{"id": "a", "tokens": prompts[1][9:], "want": [7]}], "end": ["a"]}]
    trace.expect = {1: [(1, 16)]}
    got = helpers.run_trace_cli(folder, trace, "float32", str(tmp_path / "o"), 64)
    helpers.compare_trace(folder, prompts, trace, got, helpers.tol("float32", "A"))
    assert sorted(os.listdir(tmp_path / "o")) == ["1.f32"]
