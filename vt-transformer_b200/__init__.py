"""vt_transformer_b200: a single-GPU inference engine for B200 (sm_100a), built after
viitrix/vt-transformer's Qwen2 engine: model folder in, next tokens out."""
from . import config, models, parts, weights  # noqa: F401  (registers architectures and parts)
from .engine import LLM, ModelRunner, SchedulerConfig, StepEntry
from .sampling import SamplingParams

__version__ = "0.1.0"
__all__ = ["LLM", "ModelRunner", "SamplingParams", "SchedulerConfig", "StepEntry"]
