"""The Python entry point: a model folder in, generated token ids out.

vt-transformer's own entry points are the C++ chat loop (v1/models/qwen2-7b/chat.cpp:54-123:
prompt ids in, one token a step, stop at the end token or after ``max_output``) and, in its
second generation, the back end driven by ``FullScheduler::step`` with the front end's
``SamplingParams`` (sglfront/sglfront/core.py:6-17).  ``LLM`` keeps those names:
``SchedulerConfig`` fields for the engine, ``SamplingParams`` for a request, ``step()``
returning ``ReqResult`` records.  Text is outside: prompts are token ids.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache.manager import DEFAULT_PAGE_SIZE
from ..config.registry import get_architecture, load_config
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .runner import ModelRunner
from .scheduler import Scheduler, SchedulerConfig, StepResult


class _InFlight:
    """A step that has been enqueued: its sampled tokens on the device, the pinned memory they are copied to,
    and the event after that copy."""
    __slots__ = ("tokens", "host", "event", "n")

    def __init__(self, tokens, host, event, n):
        self.tokens, self.host, self.event, self.n = tokens, host, event, n


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_running_reqs: int = 128, num_pages: Optional[int] = None, max_seq_len: int = 4096,
                 page_size: int = DEFAULT_PAGE_SIZE, max_extend_tokens: int = 8192, default_max_output: int = 1024,
                 chunk_size: Optional[int] = None, runner: Optional[ModelRunner] = None, overlap: bool = False,
                 fp32_weights: str = "keep"):
        """``model``: a folder with config.json and model.safetensors.  ``num_pages`` None
        sizes the pool for ``max_running_reqs`` requests of ``max_seq_len`` tokens, capped at
        half a million tokens.  ``overlap``: while all running requests decode, the next step is
        enqueued before the tokens of the one before have been read (``Scheduler`` says how);
        ``step()`` then reports a step's tokens one call later.  ``fp32_weights``: "keep" or "round", what becomes
        of matrices stored in 32-bit when ``dtype`` is bfloat16 (``ModelRunner.build``)."""
        if runner is None:
            # what the engine needs to know of a model beyond its parts is in its ModelSpec, whatever the
            # architecture's configuration calls it: the positions it can hold, the tokens that end a request
            config = load_config(model)
            limit = get_architecture(config.architecture).model_spec(config).max_positions
            if limit:
                max_seq_len = min(max_seq_len, limit)
            if num_pages is None:
                num_pages = -(-min(max_running_reqs * max_seq_len, 1 << 19) // page_size)
            runner = ModelRunner.from_folder(model, dtype=dtype, device=device, page_size=page_size,
                                             num_pages=num_pages, max_requests=max_running_reqs,
                                             max_seq_len=max_seq_len, fp32_weights=fp32_weights)
        self.runner = runner
        cache = runner.cache
        self.config = SchedulerConfig(max_running_reqs=cache.max_requests, num_pages=cache.groups[0].pool.num_pages
                                      if cache.groups else 0, max_seq_len=cache.max_seq_len,
                                      page_size=cache.page_size, max_extend_tokens=max_extend_tokens,
                                      default_max_output=default_max_output, chunk_size=chunk_size)
        self.sampler = Sampler(runner.rt.ops, runner.rt.device)
        self.h2d_bytes_last_step = 0
        self.d2h_bytes_last_step = 0
        eos = tuple(runner.model.spec.eos_token_ids)
        self.scheduler = Scheduler(cache, self.config, self._run_step, eos_token_ids=eos,
                                   launch_step=self._launch_step, collect_step=self._collect_step, overlap=overlap)
        self._landing = [None, None]     # two pinned buffers for the sampled tokens: one step may be read while the next runs
        self._turn = 0

    # The scheduler's hooks.  A step is enqueued (the batch, then one sampled token for each request that wants
    # one, then their copy to pinned memory) and collected (wait for that copy); ``_run_step`` does both.
    def _launch_step(self, entries, wanting, indices, before=None):
        """``indices[i]``: which output of its request the token of ``wanting[i]`` is.  ``before``: the handle of
        the step whose sampled tokens, in the same order, are this step's input tokens."""
        logits = self.runner.step(entries, carried=before.tokens if before is not None else None)
        self.h2d_bytes_last_step = self.runner.last_h2d_bytes
        self.d2h_bytes_last_step = 0
        if not wanting:
            return _InFlight(None, None, None, 0)
        params = [r.params for r in wanting]
        tokens = self.sampler.sample(logits, params, list(indices))
        if not all(p.is_greedy for p in params):
            self.h2d_bytes_last_step += 16 * len(wanting)
        self.runner.stage_status()
        n = len(wanting)
        slot, self._turn = self._turn, self._turn ^ 1
        if self._landing[slot] is None or self._landing[slot].numel() < n:
            self._landing[slot] = torch.empty(max(n, self.runner.cache.max_requests), dtype=torch.int32,
                                              pin_memory=tokens.is_cuda)
        host = self._landing[slot]
        host[:n].copy_(tokens, non_blocking=True)
        event = None
        if tokens.is_cuda:
            event = torch.cuda.Event()
            event.record()
        self.d2h_bytes_last_step = 4 * n + 8
        return _InFlight(tokens, host, event, n)

    def _collect_step(self, flight) -> List[int]:
        if flight.n == 0:
            return []
        if flight.event is not None:
            flight.event.synchronize()      # the step, the copy of the status word and the copy of the tokens are done
        self.runner.check_status(staged=True)
        return flight.host[:flight.n].tolist()

    def _run_step(self, entries, wanting) -> List[int]:
        return self._collect_step(self._launch_step(entries, wanting, [len(r.output) for r in wanting]))

    # ---- requests one by one ---------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None) -> int:
        return self.scheduler.add_request(prompt_token_ids, sampling_params)

    def abort(self, uid: int) -> bool:
        return self.scheduler.abort(uid)

    def step(self) -> StepResult:
        return self.scheduler.step()

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ---- whole batches ---------------------------------------------------------------------------
    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Generates for every prompt and returns the new token ids of each, in the order of
        the prompts.  One ``SamplingParams`` stands for all prompts; prompt i then draws with
        seed ``sampling_params.seed + i``."""
        n = len(prompt_token_ids)
        if sampling_params is None:
            sampling_params = SamplingParams(max_tokens=self.config.default_max_output)
        if isinstance(sampling_params, SamplingParams):
            params = [replace(sampling_params, seed=sampling_params.seed + i) for i in range(n)]
        else:
            params = list(sampling_params)
            if len(params) != n:
                raise ValueError(f"{n} prompts but {len(params)} sampling parameters")
        uids = [self.add_request(p, sp) for p, sp in zip(prompt_token_ids, params)]
        while self.scheduler.has_work():
            res = self.scheduler.step()
            if not res.ran_batch and not res.n_preempted and self.scheduler.has_work():
                raise RuntimeError("the scheduler can run nothing: the cache pool is too small for the waiting request")
        out = []
        for uid in uids:
            req = self.scheduler.finished.pop(uid)
            if req.finish_reason == "out_of_pages":
                raise RuntimeError(f"request {uid} does not fit the cache pool even alone")
            out.append(list(req.output))
        return out

    @property
    def stats(self) -> Dict[str, int]:
        s = dict(self.scheduler.stats)
        s["free_pages"] = self.runner.cache.free_pages()
        return s
