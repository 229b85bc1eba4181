"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401
from .base import (Block, CacheView, Embedding, FeedForward, Head, KVCacheSpec, Mixer, Norm, ParamSpec, Part, PositionEncoding,
                   ResidualStream, Runtime, StateLayout, StateSpec, PagedLayout, build_part, register_cache_kind, register_part,
                   unregister_cache_kind, unregister_part)
from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, FeedForwardSpec, GatedMLPSpec, HeadSpec, MixerSpec, ModelSpec, NormSpec,
                    PositionSpec, RunSpec)
