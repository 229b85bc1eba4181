"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

After vt-transformer's ``FullScheduler`` (vt-transformer/core/vt_scheduler.cpp): two queues,
waiting and running (``pending_``/``running_``, vt_scheduler.hpp:132-141); FIFO admission
(:251-302); a token budget for a step (``max_extend_tokens``); a result for every request that
produced a token, ``ReqResult{uid, next_token, finished}`` (vt_scheduler.hpp:94-98).  What is
decided differently, because the reference leaves it open:

* a step is mixed: every running request takes part, those that decode with one token,
  those still in their prompt with a portion of it (the reference runs prompts or decodes,
  never both, vt_scheduler.cpp:102-110, and never cuts a prompt, :277,:292-294);
* admission reserves nothing for the future; when pages run out, the youngest running
  request is pre-empted: its pages and row are given back, its tokens (prompt and what it
  has generated) are kept, and it goes to the head of the waiting queue; when it is
  admitted again its tokens are run again in portions and it goes on where it stopped,
  with the same random numbers.  (The reference rolls a prompt batch back and otherwise
  stalls, vt_scheduler.cpp:386-402, and never evicts.)  The oldest request always goes on;
  a request that cannot fit the pool even alone is finished with reason "out_of_pages".

With ``overlap`` (the reference's ``step_overlap``, vt_scheduler.cpp:148-226: it counts the tokens of the
step in flight as cached, starts the next forward pass and takes the results of the one before at the next
call) a step is enqueued and its tokens are read one call later.  While every running request decodes and
none can be foreseen to finish (by its length), the next step is enqueued before the tokens of the step in
flight have been read: its input tokens are that step's sampled tokens, which it finds on the device.  A
request that then turns out to have ended (an end token) has run one token too far; that token is dropped
when its step lands.  Everything else (prompts, admission, pre-emption, a foreseen end) happens with nothing
in flight, as without overlap.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import DEFAULT_PAGE_SIZE, OutOfPages
from ..sampling.params import SamplingParams
from .batch import StepEntry


@dataclass
class SchedulerConfig:
    """Names and defaults of vt-transformer/core/vt_scheduler.hpp:33-38, except
    ``page_size`` (64 here: the attention kernels read keys in runs of 16 and bring a page with one TMA box) and
    ``chunk_size`` (the longest portion of one prompt in a step; the reference has none)."""
    max_running_reqs: int = 128
    num_pages: int = 1024
    max_seq_len: int = 4096
    page_size: int = DEFAULT_PAGE_SIZE
    max_extend_tokens: int = 8192
    default_max_output: int = 1024
    chunk_size: Optional[int] = None


WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    uid: int
    prompt: List[int]
    params: SamplingParams
    arrival: int
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    row: Optional[int] = None
    cached: int = 0              # tokens whose keys and values are in the cache
    preemptions: int = 0
    finish_reason: Optional[str] = None

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def pending(self) -> int:
        """Tokens that still have to run: the rest of the prompt, or the last sampled token."""
        return self.n_tokens - self.cached

    def token_slice(self, a: int, b: int) -> List[int]:
        n = len(self.prompt)
        if b <= n:
            return self.prompt[a:b]
        if a >= n:
            return self.output[a - n:b - n]
        return self.prompt[a:] + self.output[:b - n]


@dataclass
class ReqResult:
    uid: int
    next_token: int
    finished: bool
    finish_reason: Optional[str] = None


@dataclass
class StepResult:
    ran_batch: bool
    results: List[ReqResult]
    n_tokens: int = 0
    n_preempted: int = 0


@dataclass
class _Flight:
    """A step that has been enqueued and whose tokens have not been read."""
    plan: List[Tuple[Request, int]]
    wanting: List[Request]
    handle: object
    n_preempted: int = 0


class Scheduler:
    """``cache`` is the cache manager (pages and rows); ``run_step(entries)`` runs a batch and
    returns one sampled token for each entry that wants logits, in order (the engine binds it
    to ``ModelRunner.step`` plus the sampler; tests bind a fake)."""

    def __init__(self, cache, config: SchedulerConfig, run_step, eos_token_ids: Sequence[int] = (),
                 launch_step=None, collect_step=None, overlap: bool = False):
        """``launch_step(entries, wanting, indices, before) -> handle`` enqueues a step (``before``: the handle of
        the step whose sampled tokens are this step's input tokens, or None) and ``collect_step(handle)`` waits
        for it and returns its tokens; both are needed for ``overlap``."""
        self.cache = cache
        self.config = config
        self.run_step = run_step
        self.launch_step, self.collect_step = launch_step, collect_step
        self.overlap = bool(overlap) and launch_step is not None and collect_step is not None
        self._flight: Optional[_Flight] = None
        self.eos = tuple(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: Dict[int, Request] = {}
        self._next_uid = 0
        self._arrivals = 0
        self.stats = {"steps": 0, "tokens": 0, "preemptions": 0, "finished": 0}

    # ---- requests ----------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    uid: Optional[int] = None) -> int:
        params = params or SamplingParams(max_tokens=self.config.default_max_output)
        params.validate()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if len(prompt) >= self.config.max_seq_len:
            raise ValueError(f"the prompt has {len(prompt)} tokens; max_seq_len is {self.config.max_seq_len}")
        if uid is None:
            uid = self._next_uid
        self._next_uid = max(self._next_uid, uid) + 1
        req = Request(uid=uid, prompt=prompt, params=params, arrival=self._arrivals)
        self._arrivals += 1
        self.waiting.append(req)
        return uid

    def abort(self, uid: int) -> bool:
        """Drops a request wherever it is; what it holds is given back at once."""
        for req in list(self.waiting):
            if req.uid == uid:
                self.waiting.remove(req)
                self._finish(req, "abort")
                return True
        for req in self.running:
            if req.uid == uid:
                self.running.remove(req)
                self._finish(req, "abort")
                return True
        return False

    def has_inflight(self) -> bool:
        """A step has been enqueued whose tokens have not been read (vt_scheduler.hpp: ``has_inflight``)."""
        return self._flight is not None

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._flight is not None)

    def _finish(self, req: Request, reason: str) -> None:
        if req.row is not None:
            self.cache.release(req.row)
            req.row = None
        req.state, req.finish_reason = FINISHED, reason
        self.finished[req.uid] = req
        self.stats["finished"] += 1

    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        self.cache.release(req.row)
        req.row, req.cached, req.state = None, 0, WAITING
        req.preemptions += 1
        self.waiting.appendleft(req)
        self.stats["preemptions"] += 1

    # ---- planning ------------------------------------------------------------------------------
    def plan(self) -> Tuple[List[Tuple[Request, int]], int]:
        """Decides the step: which requests run how many tokens.  Pre-empts and admits as
        needed.  Returns the plan and the number of requests pre-empted.

        The decision itself is ``plan_step`` of ``csrc/host_runtime.cpp`` (decodes first, then prompt portions
        under ``max_extend_tokens`` and ``chunk_size``; the youngest running request is pre-empted while the
        running requests' next tokens need more pages than are free; admission in arrival order with a page
        of head-room for each running request); it releases and admits rows in the cache manager's book, and
        this method moves the request objects accordingly."""
        from ..csrc import build
        running, waiting = list(self.running), list(self.waiting)
        chunk = -1 if self.config.chunk_size is None else int(self.config.chunk_size)
        plan_idx, preempted, gone_running, gone_waiting, admitted = build.load_host().plan_step(
            self.cache.book, [(r.row, r.pending, r.cached, r.arrival) for r in running], [r.pending for r in waiting],
            int(self.config.max_running_reqs), int(self.config.max_extend_tokens), chunk)
        for i in gone_running:                      # alone and still too large for the pool (its row is released already)
            req = running[i]
            self.running.remove(req)
            req.row = None
            self._finish(req, "out_of_pages")
        for i in preempted:                         # back to the head of the queue, the one pre-empted last in front
            req = running[i]
            self.running.remove(req)
            req.row, req.cached, req.state = None, 0, WAITING
            req.preemptions += 1
            self.waiting.appendleft(req)
            self.stats["preemptions"] += 1
        for k in gone_waiting:
            req = waiting[k]
            self.waiting.remove(req)
            self._finish(req, "out_of_pages")
        for k, row in admitted:
            req = waiting[k]
            self.waiting.remove(req)
            self.cache.zero_state(row)
            req.row, req.state, req.cached = row, RUNNING, 0
            self.running.append(req)
        plan = [((running[i] if i >= 0 else waiting[-1 - i]), int(n)) for i, n in plan_idx]
        return plan, len(preempted)

    # ---- the step ----------------------------------------------------------------------------------
    def step(self) -> StepResult:
        """One step: plan, run the batch, sample, finish and free."""
        if not self.has_work():
            return StepResult(False, [])
        if self.overlap:
            return self._step_overlap()
        plan, n_preempted = self.plan()
        if not plan:
            return StepResult(False, [], n_preempted=n_preempted)
        entries, wanting = [], []
        for req, n in plan:
            last = (n == req.pending)
            entries.append(StepEntry(req.row, req.token_slice(req.cached, req.cached + n), [n - 1] if last else []))
            if last:
                wanting.append(req)
        try:
            tokens = self.run_step(entries, wanting)
        except OutOfPages:
            # the plan counted pages; a group can still be short when window groups hold pages of
            # portions in flight.  Pre-empt the youngest and let the next step plan again.
            if len(self.running) > 1:
                self._preempt(max(self.running, key=lambda r: r.arrival))
                return StepResult(False, [], n_preempted=n_preempted + 1)
            raise
        for req, n in plan:
            req.cached += n
        results = self._take_tokens(wanting, tokens)
        n_tok = sum(n for _, n in plan)
        self.stats["steps"] += 1
        self.stats["tokens"] += n_tok
        return StepResult(True, results, n_tokens=n_tok, n_preempted=n_preempted)

    def _take_tokens(self, wanting: List[Request], tokens) -> List[ReqResult]:
        """Appends a step's sampled tokens to their requests and finishes those that have ended.  A request
        that is no longer running (it ended or was aborted while the step was in flight) drops its token."""
        results = []
        for req, tok in zip(wanting, tokens):
            if req.state != RUNNING:
                continue
            tok = int(tok)
            req.output.append(tok)
            reason = None
            eos = req.params.eos_token_ids if req.params.eos_token_ids is not None else self.eos
            if not req.params.ignore_eos and tok in eos:
                reason = "stop"
            elif len(req.output) >= req.params.max_tokens:
                reason = "length"
            elif req.n_tokens >= self.config.max_seq_len:
                reason = "length"
            if reason is not None:
                self.running.remove(req)
                self._finish(req, reason)
            results.append(ReqResult(req.uid, tok, reason is not None, reason))
        return results

    # ---- the step, with the next one enqueued before this one's tokens are read ---------------------------
    def _step_overlap(self) -> StepResult:
        flight = self._flight
        self._flight = None
        if flight is None:
            plan, n_preempted = self.plan()
            if not plan:
                return StepResult(False, [], n_preempted=n_preempted)
            entries, wanting = [], []
            for req, n in plan:
                last = (n == req.pending)
                entries.append(StepEntry(req.row, req.token_slice(req.cached, req.cached + n), [n - 1] if last else []))
                if last:
                    wanting.append(req)
            try:
                handle = self.launch_step(entries, wanting, [len(r.output) for r in wanting], None)
            except OutOfPages:
                if len(self.running) > 1:
                    self._preempt(max(self.running, key=lambda r: r.arrival))
                    return StepResult(False, [], n_preempted=n_preempted + 1)
                raise
            for req, n in plan:
                req.cached += n             # as the reference does: counted as cached when the step is enqueued
            flight = _Flight(plan, wanting, handle, n_preempted)
        ahead = self._launch_ahead(flight)
        results = self._take_tokens(flight.wanting, self.collect_step(flight.handle))
        self._flight = ahead
        n_tok = sum(n for _, n in flight.plan)
        self.stats["steps"] += 1
        self.stats["tokens"] += n_tok
        return StepResult(True, results, n_tokens=n_tok, n_preempted=flight.n_preempted)

    def _launch_ahead(self, flight: "_Flight") -> Optional["_Flight"]:
        """Enqueues the step after ``flight`` if that needs no decision: nobody waits, the running requests are
        those that get a token from ``flight`` (each then has that one token to run), none of them ends by
        its length with that token, and the pages for one more token each are there."""
        wanting = flight.wanting
        if self.waiting or not wanting or len(flight.plan) != len(wanting) or len(self.running) != len(wanting):
            return None
        running = {id(r) for r in self.running}
        for r in wanting:
            if r.state != RUNNING or id(r) not in running:
                return None
            if len(r.output) + 1 >= r.params.max_tokens or r.n_tokens + 1 >= self.config.max_seq_len:
                return None
        entries = [StepEntry(r.row, [0], [0]) for r in wanting]      # the ids are on the device: flight's tokens
        try:
            handle = self.launch_step(entries, wanting, [len(r.output) + 1 for r in wanting], flight.handle)
        except OutOfPages:
            return None
        for r in wanting:
            r.cached += 1
        return _Flight([(r, 1) for r in wanting], list(wanting), handle, 0)
