"""The step function: one batch of (request, its next tokens) in, logits at the wanted
places out.

It is the only way tokens go through the model: generation, the scheduler and the trace
replay all call ``ModelRunner.step``.  A step runs only the tokens it is given, as one
flat batch, against the keys and values that earlier steps left in the pages.  Like
vt-transformer's forward (vt-transformer/core/vt_request.hpp:18-33) it writes the cache
for exactly the new tokens; unlike it (vt-transformer/core/vt_engine.hpp:34-37) it returns
logits and leaves sampling to the caller.
"""
from __future__ import annotations

import sys
import warnings
from typing import Optional, Sequence

import torch

from .. import ops as _ops
from ..cache.manager import DEFAULT_PAGE_SIZE, CacheManager
from ..config.registry import get_architecture, load_config
from ..models.base import DecoderModel
from ..parts.base import Runtime
from ..weights.loader import RandomSource, SafetensorsSource
from .batch import StepEntry, build_context

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}

_STATUS_TEXT = {
    1: "a token id lies outside the embedding table",
    2: "a position lies outside the rotation table",
    3: "a block-table entry lies outside the page pool",
    4: "a token's sequence index lies outside the step",
    5: "a row index lies outside its tensor",
    6: "a bounded wait inside a kernel ran out",
}


class DeviceStatusError(RuntimeError):
    """A kernel met an index it must not follow (it skipped the access and went on)."""


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', found {dtype!r}") from None


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, rt: Runtime):
        self.model, self.cache, self.rt = model, cache, rt
        self.status = torch.zeros(2, dtype=torch.int32, device=rt.device)
        self._status_host = None
        self.steps = 0
        self.last_h2d_bytes = 0
        # single-token steps are replayed as CUDA graphs where every part allows it
        self.use_graphs = rt.device.type == "cuda" and model.graph_safe()
        self.max_graph_batch = 256
        self._graphs = {}

    # ---- construction --------------------------------------------------------------------
    @classmethod
    def build(cls, config, source_factory, *, dtype="bfloat16", device="cuda:0", page_size: int = DEFAULT_PAGE_SIZE,
              num_pages: Optional[int] = None, max_tokens: Optional[int] = None, max_requests: int = 8,
              max_seq_len: Optional[int] = None, ops=None, fp32_weights: str = "keep") -> "ModelRunner":
        """``source_factory(param_table)`` returns the ``WeightSource``.  The pool holds
        ``num_pages`` pages in each group, or enough for ``max_tokens`` tokens.  ``fp32_weights``: what becomes of
        a matrix stored in 32-bit when ``dtype`` is bfloat16: "keep" (it stays 32-bit and its products run the
        32-bit kernels; a warning says so) or "round" (to bfloat16, to nearest even; a line reports how many values
        became infinite or zero)."""
        if fp32_weights not in ("keep", "round"):
            raise ValueError(f"fp32_weights must be 'keep' or 'round', found {fp32_weights!r}")
        dt = parse_dtype(dtype)
        if torch.device(device).type == "cuda" and not torch.cuda.is_available():
            raise RuntimeError("vt_transformer_b200 runs on a CUDA device (B200, sm_100a) only; "
                               "torch.cuda.is_available() is False and there is no CPU path")
        rt = Runtime(device=torch.device(device), dtype=dt, ops=ops if ops is not None else _ops, fp32_weights=fp32_weights)
        spec = get_architecture(config.architecture).model_spec(config)
        model = DecoderModel(spec, rt)
        source = source_factory(model.param_specs())
        try:
            model.load(source)
        finally:
            source.close()
        for line in model.load_info:
            print(f"[vt_transformer_b200] {line}", file=sys.stderr, flush=True)
        for line in model.load_warnings:
            warnings.warn(line, stacklevel=2)
        limit = spec.max_positions or None
        if max_seq_len is None:
            max_seq_len = limit or 4096
        if limit is not None and max_seq_len > limit:
            raise ValueError(f"max_seq_len {max_seq_len} is above the model's {limit} positions")
        if num_pages is None:
            if max_tokens is None:
                max_tokens = max_seq_len * max_requests
            num_pages = -(-max_tokens // page_size)
        cache = CacheManager(model.cache_slots(), page_size=page_size, num_pages=num_pages,
                             max_requests=max_requests, max_seq_len=max_seq_len, dtype=dt, device=rt.device)
        return cls(model, cache, rt)

    @classmethod
    def from_folder(cls, folder: str, **kw) -> "ModelRunner":
        config = load_config(folder)
        return cls.build(config, lambda table: SafetensorsSource(folder), **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, sigma: float = 0.02, **kw) -> "ModelRunner":
        """Random weights made on the device, tensor by tensor (no folder is written)."""
        device = kw.get("device", "cuda:0")
        return cls.build(config, lambda table: RandomSource(table, seed, sigma, device=device), **kw)

    # ---- requests --------------------------------------------------------------------------
    def admit(self) -> int:
        return self.cache.admit()

    def release(self, row: int) -> None:
        self.cache.release(row)

    # ---- the step ----------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], carried: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the entries as one batch and returns float32 logits [wanted, vocab] on the
        device, in the order of the entries and of their ``want``.  Raises ``OutOfPages``
        (and changes nothing) if a group cannot cover the new tokens.

        ``carried``: int32 token ids on the device, one for each entry in order, which stand in
        for the entries' single tokens (the ids that the step before sampled, which the host has
        not read yet: the step is enqueued behind it and reads them there)."""
        entries = [e for e in entries if len(e.tokens) > 0]
        vocab = self.model.spec.vocab
        if not entries:
            return torch.empty((0, vocab), dtype=torch.float32, device=self.rt.device)
        if (self.use_graphs and len(entries) <= self.max_graph_batch and all(len(e.tokens) == 1 for e in entries)
                and all(len(e.want) == 0 or (len(e.want) == 1 and e.want[0] == 0) for e in entries)):
            return self._graph_step(entries, carried)
        seen = set()
        for e in entries:
            if e.row in seen:
                raise ValueError(f"row {e.row} appears twice in one step")
            seen.add(e.row)
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"row {e.row}: wanted place {w} is outside its {len(e.tokens)} tokens")
        self.cache.extend([(e.row, self.cache.length(e.row) + len(e.tokens)) for e in entries])
        ctx = build_context(entries, self.cache, self.rt.device, status=self.status, carried=carried)
        self.last_h2d_bytes = ctx.h2d_bytes
        logits = self.model.forward(ctx, self.cache.views(ctx.block_tables))
        if ctx.want_inverse is not None:
            logits = logits[torch.as_tensor(ctx.want_inverse, device=logits.device)]
        for e in entries:
            self.cache.commit(e.row, self.cache.length(e.row) + len(e.tokens))
        self.steps += 1
        return logits

    def _graph_step(self, entries: Sequence[StepEntry], carried: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A step of single tokens through a captured graph.  The logits lie in the graph's own
        buffer: they are valid until the next step."""
        from .graphs import DecodeGraph, batch_bucket, context_bucket
        rows = [e.row for e in entries]
        group, needed, free, max_kv, min_kv = self.cache.book.extend_each(rows, 1)      # pages for the tokens, all or none
        if group >= 0:
            from ..cache.manager import OutOfPages
            raise OutOfPages(group, needed, free)
        # a graph a (batch, bound of the cached lengths, whether all lengths are at least a quarter of that bound: the
        # keys of sequences of like lengths are cut over CTAs in another way than those of very different ones)
        bound = context_bucket(max_kv)
        key = (batch_bucket(len(entries)), bound, 4 * min_kv >= bound)
        graph = self._graphs.get(key)
        if graph is None:
            graph = DecodeGraph(self, key[0], key[1], like_lengths=key[2])
            self._graphs[key] = graph
        logits = graph.run(entries, carried)
        self.cache.book.commit_each(rows, 1)
        self.steps += 1
        self.last_h2d_bytes = graph.layout.total * 4
        wanted = [i for i, e in enumerate(entries) if len(e.want) > 0]
        if len(wanted) != len(entries):
            logits = logits[torch.as_tensor(wanted, dtype=torch.long, device=logits.device)]
        return logits

    def stage_status(self) -> None:
        """Enqueues a copy of the kernels' status word to pinned host memory.  A caller that then waits for a
        later operation of the stream (the read of the sampled tokens) finds it there and ``check_status(staged=
        True)`` costs no wait of its own."""
        if self._status_host is None:
            self._status_host = torch.zeros(2, dtype=torch.int32, pin_memory=self.status.is_cuda)
        self._status_host.copy_(self.status, non_blocking=True)

    def check_status(self, staged: bool = False) -> None:
        """Raises if a kernel reported a bad index.  Reads the kernels' status word (this waits for the
        device), or, with ``staged``, the copy that ``stage_status`` enqueued and that the caller has waited
        for since."""
        code, detail = (int(v) for v in (self._status_host if staged and self._status_host is not None else self.status).tolist())
        if code:
            self.status.zero_()
            raise DeviceStatusError(f"{_STATUS_TEXT.get(code, 'unknown status')} (code {code}, value {detail})")

    # ---- figures for the roofline ----------------------------------------------------------------
    def weight_bytes(self, n_tokens: int = 1) -> int:
        return self.model.weight_bytes(n_tokens)
