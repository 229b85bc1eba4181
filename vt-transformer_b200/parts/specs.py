"""Descriptions of a model as data: which parts, of which sizes, in which order.

A ``ModelSpec`` is what an architecture's ``model_spec(config)`` returns.  It plays
the role of vt-transformer's graph text (v1/models/qwen2-7b/inference_fp16.dag), whose
words take their constants as arguments (``RMS_EPS`` at :290, ``ROTARY_BASE`` at :39):
every part below carries its own sizes and constants, the blocks are chosen one by one,
and the order of runs is a list.  No spec names a model.

Each spec has a ``kind``: the key under which its implementation is registered
(``parts.base.register_part``).  A new kind of mixer, feed-forward, norm, position
encoding or block is a new spec class with a new ``kind`` and a class registered
for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """``rotary``: rotation of pairs (i, i + dim/2) by pos * base^(-2i/dim).  ``none``: nothing."""
    dim: int = 0
    base: float = 0.0
    max_positions: int = 0
    kind: str = "rotary"


@dataclass(frozen=True)
class MixerSpec:
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Grouped-query attention over a paged cache of keys and values.

    ``window``: None sees all earlier keys; w sees key j from position p if p - w < j <= p.
    ``names``: tensor names of the q, k, v and o projections below the part's prefix.
    """
    hidden: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = True
    out_bias: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None          # None: 1 / sqrt(head_dim)
    position: PositionSpec = field(default_factory=lambda: PositionSpec(kind="none"))
    names: Tuple[str, str, str, str] = ("q_proj", "k_proj", "v_proj", "o_proj")
    kind: str = "attention"


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str = "none"


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """down(act(gate(x)) * up(x)), no biases."""
    hidden: int = 0
    inter: int = 0
    activation: str = "silu"
    names: Tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj")
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer.  ``prenorm``: x += mixer(norm1(x)); x += ffn(norm2(x)).

    ``prefix`` is the tensor-name prefix of the layer; ``mixer_prefix`` and the others
    are appended to it for the parts below it."""
    mixer: MixerSpec
    ffn: FeedForwardSpec
    norm1: NormSpec
    norm2: NormSpec
    prefix: str
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    norm1_name: str = "input_layernorm"
    norm2_name: str = "post_attention_layernorm"
    kind: str = "prenorm"


@dataclass(frozen=True)
class RunSpec:
    """One entry of the run order: run block ``block`` with cache slot ``cache``.

    Cache slots are numbered by the model; a slot belongs to the run that writes it.  A
    run with ``writes=False`` reads a slot that an earlier run wrote (shared keys and
    values) and stores nothing.  A block may appear in several runs, each with a slot of
    its own."""
    block: int
    cache: Optional[int]
    writes: bool = True


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become the residual stream.  ``table``: x[t] = scale * table[id[t]] in 32-bit."""
    vocab: int
    hidden: int
    name: str = "model.embed_tokens.weight"
    scale: float = 1.0
    kind: str = "table"


@dataclass(frozen=True)
class HeadSpec:
    """How the stream's wanted rows become logits.  ``linear``: norm, then the product with a [vocab, hidden]
    matrix: its own (``name``), or, with ``tied_to``, the tensor of that name (the embedding's; one under ``name``
    is then allowed in the weights and not read); then logits * logit_scale and, with ``logit_cap`` c > 0,
    c * tanh(logits / c)."""
    vocab: int
    hidden: int
    norm: NormSpec
    norm_name: str = "model.norm"
    name: str = "lm_head.weight"
    tied_to: Optional[str] = None
    logit_scale: float = 1.0
    logit_cap: float = 0.0
    kind: str = "linear"


@dataclass(frozen=True)
class ModelSpec:
    """Embedding, blocks in their run order, head: each a part chosen by its spec's kind."""
    vocab: int
    hidden: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[RunSpec, ...]
    embedding: EmbeddingSpec
    head: HeadSpec
    max_positions: int = 0
    # patterns (fnmatch) of tensor names that a checkpoint of the architecture may hold and the model does not read
    ignored: Tuple[str, ...] = ()
    # token ids at which generation ends unless a request says otherwise (from the architecture's configuration)
    eos_token_ids: Tuple[int, ...] = ()

    @staticmethod
    def default_order(n_blocks: int) -> Tuple[RunSpec, ...]:
        return tuple(RunSpec(block=i, cache=i) for i in range(n_blocks))
