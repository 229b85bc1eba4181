"""Configuration of the Qwen2 dense decoder ("Qwen2ForCausalLM").

The keys are those of the architecture's own config.json.  vt-transformer fixes the
same quantities as literals: RMS_EPS, ROTARY_BASE, VOCAB_SIZE, HIDDEN_SIZE, KV_PROJ,
INTERMEDIATE_SIZE, HEADS_NUM, KV_HEADS_NUM, HEAD_HIDDEN and the layer count
(v1/models/qwen2-7b/inference_fp16.dag:1-14,355).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig, architecture_name


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None
    torch_dtype: Optional[str] = None
    eos_token_id: Optional[Tuple[int, ...]] = None
    bos_token_id: Optional[int] = None

    # ---- derived sizes -------------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Number of keys layer ``layer`` sees, or None if it sees all of them.

        vt-transformer's graph has no window (its mask is causal only,
        v1/tensortype/cuda_kernels/causal_mask.cu:69-84).  The meaning taken here is that
        of the config keys themselves: ``layer_types[layer]`` if the list is given
        ("full_attention" or "sliding_attention"); else, with ``use_sliding_window``, the
        layers from ``max_window_layers`` on see the last ``sliding_window`` keys: key j
        is seen from position p if p - sliding_window < j <= p.  With ``use_sliding_window`` false no layer has
        a window, whatever ``layer_types`` and ``sliding_window`` say (the architecture's own reading of its keys:
        the 7B checkpoint's config carries sliding_window 131072 beside use_sliding_window false).
        """
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return self.sliding_window if layer >= first else None

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "Qwen2Config":
        r = KeyReader(data, where)
        arch = architecture_name(data, where)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        if "head_dim" not in data or data["head_dim"] is None:
            if hidden % heads:
                raise ConfigError(f"{where}: 'hidden_size' {hidden} is not a multiple of "
                                  f"'num_attention_heads' {heads} and no 'head_dim' is given")
        head_dim = r.integer("head_dim", default=hidden // heads, minimum=1)
        layers = r.integer("num_hidden_layers", minimum=1)

        # rope_theta stands at the top level, or inside rope_parameters in newer files
        rope_params = r.raw("rope_parameters", default=None)
        rope_scaling = r.raw("rope_scaling", default=None)
        for name, block in (("rope_parameters", rope_params), ("rope_scaling", rope_scaling)):
            if block is not None:
                if not isinstance(block, dict):
                    raise ConfigError(f"{where}: key '{name}' must be an object")
                kind = block.get("rope_type", block.get("type", "default"))
                if kind not in ("default", None):
                    raise ConfigError(f"{where}: key '{name}' asks for rotation scaling '{kind}'; "
                                      f"only the plain rotation (no scaling) is built")
        if "rope_theta" in data and data["rope_theta"] is not None:
            theta = r.number("rope_theta", positive=True)
        elif isinstance(rope_params, dict) and "rope_theta" in rope_params:
            theta = float(rope_params["rope_theta"])
            if not theta > 0:
                raise ConfigError(f"{where}: 'rope_parameters.rope_theta' must be positive")
        else:
            raise ConfigError(f"{where}: key 'rope_theta' is required and missing")

        eos = r.raw("eos_token_id", default=None)
        if eos is not None:
            eos_list = eos if isinstance(eos, list) else [eos]
            if not all(isinstance(e, int) and not isinstance(e, bool) for e in eos_list):
                raise ConfigError(f"{where}: key 'eos_token_id' must be an integer or a list of integers")
            eos = tuple(eos_list)
        layer_types = r.raw("layer_types", default=None)
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != layers:
                raise ConfigError(f"{where}: key 'layer_types' must list one entry for each of the {layers} layers")
            for t in layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"{where}: key 'layer_types' holds '{t}'; known are "
                                      f"'full_attention' and 'sliding_attention'")
            layer_types = tuple(layer_types)
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default=None)

        cfg = cls(
            architecture=arch,
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps", positive=True),
            rope_theta=theta,
            max_position_embeddings=r.integer("max_position_embeddings", minimum=1),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            hidden_act=r.string("hidden_act", default="silu"),
            use_sliding_window=r.boolean("use_sliding_window", default=False),
            sliding_window=r.integer("sliding_window", default=None, minimum=1),
            max_window_layers=r.integer("max_window_layers", default=None, minimum=0),
            layer_types=layer_types,
            torch_dtype=dtype,
            eos_token_id=eos,
            bos_token_id=r.integer("bos_token_id", default=None),
        )
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config.json") -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{where}: 'num_attention_heads' {self.num_attention_heads} is not a multiple "
                              f"of 'num_key_value_heads' {self.num_key_value_heads}")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ConfigError(f"{where}: 'head_dim' {self.head_dim} is not supported: the attention kernels "
                              f"take head sizes that are multiples of 16, up to 256")
        for key, v in (("hidden_size", self.hidden_size), ("intermediate_size", self.intermediate_size)):
            if v % 8:
                raise ConfigError(f"{where}: '{key}' {v} is not supported: the matrix kernels read rows in "
                                  f"16-byte pieces, so it must be a multiple of 8")
        if self.hidden_act != "silu":
            raise ConfigError(f"{where}: 'hidden_act' is '{self.hidden_act}'; this architecture's feed-forward "
                              f"is built with 'silu' only")
        wants_window = self.use_sliding_window or (
            self.layer_types is not None and "sliding_attention" in self.layer_types)
        if wants_window and self.sliding_window is None:
            raise ConfigError(f"{where}: a sliding window is asked for but 'sliding_window' is missing")
        if self.max_window_layers is not None and self.max_window_layers > self.num_hidden_layers:
            # files in the wild carry max_window_layers above the layer count: no layer has a window then
            pass

    def to_dict(self) -> Dict[str, Any]:
        d = super().to_dict()
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) > 1 else self.eos_token_id[0]
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        d["model_type"] = "qwen2"
        return d
