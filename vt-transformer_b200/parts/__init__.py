"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, mlp, norm, rope  # noqa: F401
from .base import (Block, CacheView, FeedForward, KVCacheSpec, Mixer, Norm, ParamSpec, Part, PositionEncoding,
                   ResidualStream, Runtime, StateSpec, build_part, register_part, unregister_part)
from .specs import (AttentionSpec, BlockSpec, FeedForwardSpec, GatedMLPSpec, MixerSpec, ModelSpec, NormSpec,
                    PositionSpec, RunSpec)
