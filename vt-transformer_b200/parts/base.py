"""Interfaces of the parts a model is put together from, and their registry.

Seven categories: ``embedding``, ``norm``, ``position``, ``mixer``, ``feed_forward``, ``block``, ``head``.  A part is
built from its spec (sizes and constants), the prefix of its tensor names and the
``Runtime`` (device, compute dtype, kernels).  It says which tensors it wants
(``param_specs``), takes them (``load``) and runs on the flat token batch of one step.
No part knows which model it is in.

What a mixer keeps between steps it declares with ``cache_spec``: pages of keys and
values (``KVCacheSpec``), a block of fixed size for each request (``StateSpec``), or
nothing.  The cache manager gives the mixer a ``CacheView`` of what it declared.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Mapping, Optional, Tuple

import torch


# ----------------------------------------------------------------------------- parameters


@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part reads from the weights.

    ``role``: "matrix" and "vector" are floating point (stored in bfloat16 by the random
    initialiser; a file may hold them in 32-bit); "table" is an integer table (int32).
    ``init``: how the random initialiser fills it: "normal" is N(0, sigma),
    "one_plus_normal" is 1 + N(0, sigma), "zeros"; or a name given to ``weights.register_initialiser``.
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False


# ----------------------------------------------------------------------------- runtime


@dataclass
class Runtime:
    """Where and in which precision a model runs.  ``dtype`` is torch.bfloat16 (the
    serving path) or torch.float32 (everything in true 32-bit); ``ops`` is the kernel
    module (``vt_transformer_b200.ops``)."""
    device: torch.device
    dtype: torch.dtype
    ops: object
    loaded: Dict[Tuple[str, str], torch.Tensor] = field(default_factory=dict)
    # what happens to a matrix that is stored in 32-bit when the compute dtype is bfloat16: "keep" (it stays 32-bit
    # and its products run the 32-bit kernels) or "round" (to bfloat16, round to nearest even)
    fp32_weights: str = "keep"
    notes: Dict[str, int] = field(default_factory=dict)      # counts of what ``param`` did, for the load report

    def load(self, get: Callable, name: str, role: str = "matrix") -> torch.Tensor:
        """``param(get(name), role)``, made once for each (name, role): parts that read the same tensor (an
        output head tied to the embedding) share one copy on the device."""
        key = (name, role)
        if key not in self.loaded:
            self.loaded[key] = self.param(get(name), role)
        return self.loaded[key]

    def param(self, t: torch.Tensor, role: str = "matrix") -> torch.Tensor:
        """A stored tensor as the kernels read it.  Matrices are used in the compute
        dtype (a bfloat16 tensor is widened exactly for the 32-bit path; a tensor stored
        in 32-bit stays 32-bit and its products run through the 32-bit kernels, unless
        ``fp32_weights`` is "round").
        Vectors are read in 32-bit by every kernel.  Tables are int32."""
        if role == "table":
            return t.to(device=self.device, dtype=torch.int32).contiguous()
        if role == "vector":
            return t.to(device=self.device, dtype=torch.float32).contiguous()
        if self.dtype == torch.float32:
            return t.to(device=self.device, dtype=torch.float32).contiguous()
        if t.dtype == torch.float32:
            if self.fp32_weights != "round":
                self.notes["kept_fp32"] = self.notes.get("kept_fp32", 0) + 1
                return t.to(device=self.device, dtype=torch.float32).contiguous()
            wide = t.to(device=self.device)
            out = wide.to(self.dtype).contiguous()             # round to nearest even
            for key, n in (("rounded", 1), ("rounded_values", t.numel()),
                           ("to_inf", int((torch.isinf(out) & torch.isfinite(wide)).sum())),
                           ("to_zero", int(((out == 0) & (wide != 0)).sum()))):
                self.notes[key] = self.notes.get(key, 0) + n
            return out
        return t.to(device=self.device, dtype=self.dtype).contiguous()


# ----------------------------------------------------------------------------- caches


@dataclass(frozen=True)
class KVCacheSpec:
    """Keys and values in pages: ``kv_heads`` heads of ``head_dim`` for each token;
    ``window`` None keeps all tokens, w keeps the last w."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """A block of fixed size for each request, zero when the request is admitted."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class PagedLayout:
    """What a kind of cache spec keeps for every token, in pages.  ``tensors``: (name, outer, inner) for each
    tensor; the pool's tensor of that name is [pages, outer, page_size, inner] for a slot (keys: outer = KV heads,
    inner = head size, so that a (page, head) run of keys is contiguous).  ``window`` None keeps all tokens, w
    the last w: pages that the window has passed go back to the pool."""
    tensors: Tuple[Tuple[str, int, int], ...]
    window: Optional[int] = None


@dataclass(frozen=True)
class StateLayout:
    """A block of fixed size for each request, zero at admission."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


_CACHE_KINDS: Dict[type, Callable] = {}


def register_cache_kind(spec_class: type, layout: Callable) -> None:
    """Tells the cache manager what a kind of cache spec needs: ``layout(spec)`` returns a ``PagedLayout`` or a
    ``StateLayout``.  Slots whose paged layouts are equal share a pool and a block table for each request."""
    _CACHE_KINDS[spec_class] = layout


def unregister_cache_kind(spec_class: type) -> None:
    _CACHE_KINDS.pop(spec_class, None)


def cache_layout(spec):
    for cls in type(spec).__mro__:
        if cls in _CACHE_KINDS:
            return _CACHE_KINDS[cls](spec)
    raise TypeError(f"unknown kind of cache spec {spec!r}; known: {', '.join(c.__name__ for c in _CACHE_KINDS) or 'none'} "
                    f"(parts.register_cache_kind adds one)")


register_cache_kind(KVCacheSpec, lambda s: PagedLayout((("k", s.kv_heads, s.head_dim), ("v", s.kv_heads, s.head_dim)), s.window))
register_cache_kind(StateSpec, lambda s: StateLayout(tuple(s.shape), s.dtype))


@dataclass
class CacheView:
    """What one run of a block sees of the cache.

    For a paged slot: ``pages[name]`` is [pages, outer, page_size, inner] for every tensor of the slot's layout
    (``k`` and ``v``, [pages, kv_heads, page_size, head_dim], are those of a ``KVCacheSpec``), ``block_table`` is the
    int32 device table [sequences of this step, stride] of the slot's group, ``page_size`` the tokens in a page.
    For a state slot: ``state`` is [request rows, *shape]; the step's ``rows`` index it.  ``writes`` is False for
    a run that only reads another run's slot."""
    spec: object = None
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    state: Optional[torch.Tensor] = None
    writes: bool = True
    pages: Optional[Dict[str, torch.Tensor]] = None


# ----------------------------------------------------------------------------- parts


class Part:
    category = ""
    # True if ``forward`` only enqueues kernels that read the step's description from device
    # memory, so that a captured CUDA graph of it can be replayed for another step.  A part that
    # loops over ``ctx.seqs`` on the host, or allocates by the step's contents, must leave it False.
    graph_safe = False
    # What the step streams from HBM after this part is done: ``ops.product_hint(...)`` of the first matrix product
    # of the part that runs next, or None.  The model sets it once the weights are loaded; a part hands it to its own
    # last product (``then=``), whose kernel asks for the first of those weights while it ends.  A hint only.
    then = None

    def __init__(self, spec, prefix: str, rt: Runtime):
        self.spec = spec
        self.prefix = prefix
        self.rt = rt

    def first_product(self):
        """``ops.product_hint(...)`` of the matrix product with which this part's ``forward`` begins, or None."""
        return None

    def param_specs(self) -> Dict[str, ParamSpec]:
        """Full tensor name -> what is expected under it."""
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Takes the tensors named by ``param_specs`` (as stored) and keeps what the
        kernels need on the device."""

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads (for the roofline)."""
        return 0


class Norm(Part):
    """``__call__(x, delta=None, rows=None)``: x is the 32-bit residual stream [T, H].
    With ``delta`` (a tensor [T, H] of the compute dtype) the sum x + delta is formed in 32-bit, written back to
    x, and normed.  With ``rows`` (int32 indices) only those rows are done, packed in that order.
    Returns the normed rows in the compute dtype.

    A norm whose kernel can add the unadded 32-bit shares of a matrix product itself sets ``takes_shares``; it is
    then given what ``ops.linear_to_stream`` returned as it is.  Any other norm gets an ordinary tensor."""
    category = "norm"
    takes_shares = False

    def __call__(self, x, delta=None, rows=None, status=None):
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"


class Mixer(Part):
    """``forward(h, ctx, cache)``: h [T, hidden] normed input in the compute dtype, ctx the
    ``StepContext`` of the step, cache the ``CacheView`` of this run (None if
    ``cache_spec`` is None).  Returns [T, hidden] in the compute dtype (or, for a last product
    done with ``ops.linear_to_stream``, what that returned): the block adds it to the stream."""
    category = "mixer"

    def cache_spec(self):
        return None

    def forward(self, h, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(h, ctx)``: [T, hidden] -> [T, hidden] in the compute dtype."""
    category = "feed_forward"

    def forward(self, h, ctx):
        raise NotImplementedError


class Block(Part):
    """``forward(stream, ctx, cache)`` runs the layer on the ``ResidualStream``."""
    category = "block"

    def cache_spec(self):
        return None

    def link(self, then) -> None:
        """``then``: the first product of what runs after this block (see ``Part.then``); a block hands it to the
        part it runs last, and gives the parts before it the first product of their successors."""

    def forward(self, stream, ctx, cache):
        raise NotImplementedError


class Embedding(Part):
    """``forward(ctx) -> x``: the step's token ids (``ctx.token_ids``, -1 for padding) as the 32-bit residual
    stream [T, hidden].  ``prefix`` is the tensor's full name.  ``step_bytes(n_tokens)``: bytes it reads a step."""
    category = "embedding"

    def forward(self, ctx):
        raise NotImplementedError

    def step_bytes(self, n_tokens: int) -> int:
        return 0


class Head(Part):
    """``forward(stream, ctx) -> logits``: float32 [wanted rows, vocab] for the rows ``ctx.want_rows`` of the
    ``ResidualStream`` (whose pending delta it must add: ``stream.normed`` does)."""
    category = "head"

    def forward(self, stream, ctx):
        raise NotImplementedError


class ResidualStream:
    """The 32-bit residual stream [T, H] and a delta not yet added to it.

    A block leaves the output of its last part in ``pending``; the next norm adds it
    while it reads the stream (one pass over memory instead of two), so the sum is
    formed in 32-bit whatever the compute dtype is.  The delta is a tensor [T, H] of the
    compute dtype or what ``ops.linear_to_stream`` returned (for small batches the unadded
    32-bit shares of the product, which the norm adds as well)."""

    def __init__(self, x: torch.Tensor, status: Optional[torch.Tensor] = None):
        self.x = x
        self.status = status
        self.pending: Optional[torch.Tensor] = None

    def normed(self, norm: Norm, rows=None):
        delta, self.pending = self.pending, None
        if delta is not None and not isinstance(delta, torch.Tensor) and not getattr(norm, "takes_shares", False):
            delta = norm.rt.ops.dense(delta, norm.rt.dtype)       # unadded shares, for a norm that wants a tensor
        return norm(self.x, delta=delta, rows=rows, status=self.status)

    def add(self, delta) -> None:
        if self.pending is not None:
            raise RuntimeError("the residual stream holds a delta that no norm has added yet")
        self.pending = delta


# ----------------------------------------------------------------------------- registry

_CATEGORIES = ("embedding", "norm", "position", "mixer", "feed_forward", "block", "head")
_PARTS: Dict[str, Dict[str, Callable]] = {c: {} for c in _CATEGORIES}


def register_part(category: str, kind: str, factory: Callable = None, replace: bool = False):
    """Registers ``factory(spec, prefix, rt)`` for specs of ``kind``.  Usable as a decorator."""
    if category not in _PARTS:
        raise ValueError(f"unknown category '{category}'; known: {', '.join(_CATEGORIES)}")

    def _do(f):
        if kind in _PARTS[category] and not replace:
            raise ValueError(f"{category} '{kind}' is registered already")
        _PARTS[category][kind] = f
        return f

    return _do if factory is None else _do(factory)


def unregister_part(category: str, kind: str) -> None:
    _PARTS[category].pop(kind, None)


def build_part(category: str, spec, prefix: str, rt: Runtime) -> Part:
    try:
        factory = _PARTS[category][spec.kind]
    except KeyError:
        raise ValueError(f"no {category} of kind '{spec.kind}' is registered; known: "
                         f"{', '.join(sorted(_PARTS[category])) or 'none'}") from None
    return factory(spec, prefix, rt)
