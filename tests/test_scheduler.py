"""The scheduler's decisions, with a fake model (no GPU)."""
import random

import pytest
import torch

from vt_transformer_b200.cache import CacheManager
from vt_transformer_b200.engine.scheduler import Scheduler, SchedulerConfig
from vt_transformer_b200.parts import KVCacheSpec
from vt_transformer_b200.sampling import SamplingParams


class FakeModel:
    """Stands where the engine binds ``ModelRunner.step`` + sampler: it allocates and commits
    pages as the real step does, records the batches, and 'samples' a token that is a function
    of the request's tokens so far (so that a request's output shows if its history changed)."""

    def __init__(self, cache):
        self.cache = cache
        self.batches = []
        self.history = {}

    def __call__(self, entries, wanting):
        self.cache.extend([(e.row, self.cache.length(e.row) + len(e.tokens)) for e in entries])
        self.batches.append([(e.row, self.cache.length(e.row), len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            self.history.setdefault(e.row, [])
            if self.cache.length(e.row) == 0:
                self.history[e.row] = []
            self.history[e.row] += list(e.tokens)
            self.cache.commit(e.row, self.cache.length(e.row) + len(e.tokens))
        out = []
        for req in wanting:
            seen = self.history[req.row]
            assert seen == req.prompt + req.output, "the model saw other tokens than the request holds"
            out.append((sum(seen) * 31 + len(seen)) % 97 + 3)
        return out


def make(num_pages=16, max_running=4, budget=64, chunk=None, max_seq_len=256, eos=()):
    cache = CacheManager({0: KVCacheSpec(1, 16)}, page_size=16, num_pages=num_pages, max_requests=max_running,
                         max_seq_len=max_seq_len, dtype=torch.float32, device="cpu", allocate=False)
    cfg = SchedulerConfig(max_running_reqs=max_running, num_pages=num_pages, max_seq_len=max_seq_len, page_size=16,
                          max_extend_tokens=budget, chunk_size=chunk)
    model = FakeModel(cache)
    return Scheduler(cache, cfg, model, eos_token_ids=eos), model, cache


def run_all(s, limit=10000):
    results = {}
    for _ in range(limit):
        if not s.has_work():
            break
        for r in s.step().results:
            results.setdefault(r.uid, []).append(r)
    assert not s.has_work()
    return results


def expected_output(prompt, n):
    seen, out = list(prompt), []
    for _ in range(n):
        out.append((sum(seen) * 31 + len(seen)) % 97 + 3)
        seen.append(out[-1])
    return out


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    s, model, cache = make(budget=24, chunk=16)
    a = s.add_request(list(range(1, 41)), SamplingParams(max_tokens=3))
    s.step()                                            # 16 of 40 (the chunk)
    assert model.batches[-1] == [(0, 0, 16, [])]
    b = s.add_request([5, 6, 7], SamplingParams(max_tokens=2))
    s.step()                                            # a: next 16; b admitted with what is left of 24
    assert model.batches[-1] == [(0, 16, 16, []), (1, 0, 3, [2])]
    res = s.step()                                      # b decodes (first), a ends its prompt
    assert model.batches[-1] == [(1, 3, 1, [0]), (0, 32, 8, [7])]
    assert {r.uid for r in res.results} == {a, b}
    out = run_all(s)
    assert [r.next_token for r in out[a]][-1] == expected_output(list(range(1, 41)), 3)[-1]
    assert s.finished[a].output == expected_output(list(range(1, 41)), 3)
    assert s.finished[b].output == expected_output([5, 6, 7], 2)
    assert s.finished[a].finish_reason == "length"
    cache.check()
    assert cache.free_pages() == [16] and cache.free_rows == 4


def test_fifo_and_row_limit():
    s, model, cache = make(max_running=2, budget=100)
    ids = [s.add_request([i + 1] * 4, SamplingParams(max_tokens=2)) for i in range(4)]
    s.step()
    assert [r.uid for r in s.running] == ids[:2] and [r.uid for r in s.waiting] == ids[2:]
    run_all(s)
    order = [uid for uid in s.finished]
    assert order[:2] == ids[:2] and set(order) == set(ids)


def test_eos_max_tokens_and_max_seq_len():
    s, model, cache = make(eos=(expected_output([9, 9], 2)[1],), max_seq_len=12)
    a = s.add_request([9, 9], SamplingParams(max_tokens=50))
    b = s.add_request([9, 9], SamplingParams(max_tokens=50, ignore_eos=True))
    c = s.add_request([9, 9], SamplingParams(max_tokens=4, ignore_eos=True))
    out = run_all(s)
    assert s.finished[a].finish_reason == "stop" and len(s.finished[a].output) == 2
    assert s.finished[b].finish_reason == "length" and len(s.finished[b].prompt) + len(s.finished[b].output) == 12
    assert s.finished[c].finish_reason == "length" and len(s.finished[c].output) == 4
    assert out[a][-1].finished and not out[a][0].finished
    with pytest.raises(ValueError, match="max_seq_len"):
        s.add_request([1] * 12)
    with pytest.raises(ValueError, match="at least one"):
        s.add_request([])


def test_pages_run_out_the_youngest_is_preempted_and_resumes_with_the_same_tokens():
    # 6 pages of 16: three requests of 30 tokens (2 pages each) fill the pool; their third page does not fit
    s, model, cache = make(num_pages=6, max_running=3, budget=200)
    prompts = [[i + 1] * 30 for i in range(3)]
    ids = [s.add_request(p, SamplingParams(max_tokens=20, ignore_eos=True)) for p in prompts]
    preempted = 0
    for _ in range(500):
        if not s.has_work():
            break
        res = s.step()
        preempted += res.n_preempted
        cache.check()
    assert not s.has_work() and preempted > 0
    assert s.finished[ids[0]].preemptions == 0          # the oldest always goes on
    assert sum(s.finished[u].preemptions for u in ids[1:]) == preempted
    for uid, p in zip(ids, prompts):
        assert s.finished[uid].output == expected_output(p, 20)
    assert cache.free_pages() == [6] and cache.free_rows == 3


def test_a_request_too_large_for_the_pool_is_finished_not_stalled():
    s, model, cache = make(num_pages=2, max_running=2, budget=200)
    a = s.add_request([1] * 40, SamplingParams(max_tokens=4))    # needs 3 pages to end its prompt
    b = s.add_request([2] * 8, SamplingParams(max_tokens=4, ignore_eos=True))
    run_all(s, limit=100)
    assert s.finished[a].finish_reason == "out_of_pages"
    assert s.finished[b].output == expected_output([2] * 8, 4)
    cache.check()
    assert cache.free_pages() == [2]


def test_abort_gives_everything_back():
    s, model, cache = make()
    a = s.add_request([1] * 20, SamplingParams(max_tokens=50, ignore_eos=True))
    b = s.add_request([2] * 20, SamplingParams(max_tokens=50, ignore_eos=True))
    s.step(), s.step()
    assert s.abort(a) and not s.abort(12345)
    assert s.finished[a].finish_reason == "abort" and cache.free_rows == 3
    c = s.add_request([3] * 5, SamplingParams(max_tokens=2))
    assert s.abort(c)                                   # still waiting
    run_all(s)
    assert s.finished[b].output == expected_output([2] * 20, 50)
    cache.check()
    assert cache.free_pages() == [16]


@pytest.mark.parametrize("seed", range(4))
def test_random_load_every_request_gets_its_own_tokens(seed):
    rng = random.Random(seed)
    s, model, cache = make(num_pages=rng.choice([6, 9, 14]), max_running=rng.choice([2, 3, 4]),
                           budget=rng.choice([8, 24, 64]), chunk=rng.choice([None, 4, 16]))
    want = {}
    pending = [[rng.randrange(1, 90) for _ in range(rng.choice([1, 3, 17, 33, 50]))] for _ in range(10)]
    steps = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.4:
            p = pending.pop()
            n = rng.choice([1, 5, 12])
            want[s.add_request(p, SamplingParams(max_tokens=n, ignore_eos=True))] = expected_output(p, n)
        if s.has_work():
            s.step()
            cache.check()
            assert sum(m for _, _, m, _ in model.batches[-1]) <= s.config.max_extend_tokens if model.batches else True
        steps += 1
        assert steps < 5000
    for uid, out in want.items():
        assert s.finished[uid].output == out, (uid, s.finished[uid].finish_reason)
    assert cache.free_pages() == [cache.groups[0].pool.num_pages]


# ---- overlap: the next step enqueued before the tokens of the one in flight are read --------------------------

class FakeAsyncModel(FakeModel):
    """The same fake behind the two hooks of the overlap mode.  A step that is enqueued behind another takes its
    input tokens from that step's tokens, as the device does; the host's entries hold placeholders then."""

    def __init__(self, cache):
        super().__init__(cache)
        self.early = 0
        self.open_handles = 0

    def launch(self, entries, wanting, indices, before=None):
        if before is not None:
            assert len(entries) == len(before["tokens"]) and all(len(e.tokens) == 1 for e in entries)
            assert [r.uid for r in wanting] == before["uids"], "carried tokens must come in the order of the entries"
            for e, tok in zip(entries, before["tokens"]):
                e.tokens = [tok]
            self.early += 1
        self.cache.extend([(e.row, self.cache.length(e.row) + len(e.tokens)) for e in entries])
        self.batches.append([(e.row, self.cache.length(e.row), len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            if self.cache.length(e.row) == 0:
                self.history[e.row] = []
            self.history.setdefault(e.row, [])
            self.history[e.row] += list(e.tokens)
            self.cache.commit(e.row, self.cache.length(e.row) + len(e.tokens))
        out = []
        for req, index in zip(wanting, indices):
            seen = self.history[req.row]
            known = req.prompt + req.output
            assert seen[:len(known)] == known and len(seen) == len(req.prompt) + index
            out.append((sum(seen) * 31 + len(seen)) % 97 + 3)
        self.open_handles += 1
        assert self.open_handles <= 2, "more than one step ahead"
        return {"tokens": out, "uids": [r.uid for r in wanting]}

    def collect(self, handle):
        self.open_handles -= 1
        return handle["tokens"]


def make_overlap(num_pages=16, max_running=4, budget=64, chunk=None, max_seq_len=256, eos=()):
    cache = CacheManager({0: KVCacheSpec(1, 16)}, page_size=16, num_pages=num_pages, max_requests=max_running,
                         max_seq_len=max_seq_len, dtype=torch.float32, device="cpu", allocate=False)
    cfg = SchedulerConfig(max_running_reqs=max_running, num_pages=num_pages, max_seq_len=max_seq_len, page_size=16,
                          max_extend_tokens=budget, chunk_size=chunk)
    model = FakeAsyncModel(cache)
    s = Scheduler(cache, cfg, None, eos_token_ids=eos, launch_step=model.launch, collect_step=model.collect, overlap=True)
    return s, model, cache


def test_overlap_reports_every_token_once_and_stops_where_the_plain_loop_stops():
    s, model, cache = make_overlap(num_pages=24)
    # b's end token is the 7th it generates: it is found when that step lands, with the next step already enqueued
    pb = [2] * 20
    eos = expected_output(pb, 7)[6]
    stop_b = expected_output(pb, 50).index(eos) + 1
    a = s.add_request([1] * 20, SamplingParams(max_tokens=30, ignore_eos=True))
    b = s.add_request(pb, SamplingParams(max_tokens=50, eos_token_ids=(eos,)))
    c = s.add_request([3] * 9, SamplingParams(max_tokens=12, ignore_eos=True))
    results = run_all(s)
    assert s.finished[a].output == expected_output([1] * 20, 30) and s.finished[a].finish_reason == "length"
    assert s.finished[b].output == expected_output(pb, stop_b) and s.finished[b].finish_reason == "stop"
    assert s.finished[c].output == expected_output([3] * 9, 12)
    for uid in (a, b, c):
        assert [r.next_token for r in results[uid]] == s.finished[uid].output
        assert [r.finished for r in results[uid]] == [False] * (len(results[uid]) - 1) + [True]
    assert model.early > 20 and model.open_handles == 0 and not s.has_inflight()
    cache.check()
    assert cache.free_pages() == [24]


def test_overlap_abort_while_a_step_is_in_flight():
    s, model, cache = make_overlap()
    a = s.add_request([1] * 20, SamplingParams(max_tokens=50, ignore_eos=True))
    b = s.add_request([2] * 20, SamplingParams(max_tokens=50, ignore_eos=True))
    for _ in range(4):
        s.step()
    assert s.has_inflight()
    n = len(s.running[0].output)
    assert s.abort(a)
    assert s.finished[a].finish_reason == "abort" and len(s.finished[a].output) == n
    res = s.step()                                      # lands the step that still held a: its token is dropped
    assert [r.uid for r in res.results] == [b] and len(s.finished[a].output) == n
    run_all(s)
    assert s.finished[b].output == expected_output([2] * 20, 50)
    cache.check()
    assert cache.free_pages() == [16] and model.open_handles == 0


@pytest.mark.parametrize("seed", range(4))
def test_overlap_random_load_every_request_gets_its_own_tokens(seed):
    rng = random.Random(100 + seed)
    s, model, cache = make_overlap(num_pages=rng.choice([6, 9, 14]), max_running=rng.choice([2, 3, 4]),
                                   budget=rng.choice([8, 24, 64]), chunk=rng.choice([None, 4, 16]))
    want = {}
    pending = [[rng.randrange(1, 90) for _ in range(rng.choice([1, 3, 17, 33, 50]))] for _ in range(10)]
    steps = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.25:
            p = pending.pop()
            n = rng.choice([1, 5, 12, 30])
            full = expected_output(p, n)
            if rng.random() < 0.5:
                eos = full[rng.randrange(len(full))]
                want[s.add_request(p, SamplingParams(max_tokens=n, eos_token_ids=(eos,)))] = full[:full.index(eos) + 1]
            else:
                want[s.add_request(p, SamplingParams(max_tokens=n, ignore_eos=True))] = full
        if s.has_work():
            s.step()
            cache.check()
        steps += 1
        assert steps < 5000
    for uid, out in want.items():
        assert s.finished[uid].output == out, (uid, s.finished[uid].finish_reason)
    assert cache.free_pages() == [cache.groups[0].pool.num_pages] and model.open_handles == 0
