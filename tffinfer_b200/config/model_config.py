"""Typed model configuration, read from the architecture's own config.json keys.

The reference keeps hyper-parameters and user flags in one struct
(src/core/model/BaseDefine.h:101-149 ``ModelConfig``) and fills it from GGUF
metadata (src/core/model/gguf/GGUFLoader.cpp:244-283).  Here the hyper-parameters
come from config.json and live in :class:`Qwen3Config`; run-time options live in
``EngineConfig``.  Every size and every constant the model needs is a field of the
configuration: nothing about a particular checkpoint is written in code.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used: names the offending key."""


_REQUIRED = object()


def _get(d: Dict[str, Any], key: str, kind, default=_REQUIRED):
    if key not in d or d[key] is None:
        if default is _REQUIRED:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is float and isinstance(v, (int, float)) and not isinstance(v, bool):
        return float(v)
    if kind is int and isinstance(v, int) and not isinstance(v, bool):
        return int(v)
    if kind is bool and isinstance(v, bool):
        return v
    if kind is str and isinstance(v, str):
        return v
    raise ConfigError(f"config.json: key '{key}' has value {v!r}, expected {kind.__name__}")


@dataclass(frozen=True)
class ModelConfig:
    """Base of all typed architecture configurations."""
    architecture: str

    def to_json_dict(self) -> Dict[str, Any]:
        raise NotImplementedError


FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Hyper-parameters of a Qwen3 dense model.

    Field             config.json key             reference (GGUF) counterpart
    hidden_size       hidden_size                 embedding_length  (_n_embd)
    num_layers        num_hidden_layers           block_count       (_n_layer)
    num_heads         num_attention_heads         attention.head_count
    num_kv_heads      num_key_value_heads         attention.head_count_kv
    head_dim          head_dim                    attention.key_length; the reference
                                                  instead derives hidden/heads
                                                  (src/core/runtime/InferRuntime.cu:50),
                                                  which is wrong when heads*head_dim !=
                                                  hidden; that quotient is used here only
                                                  when the key is absent
    intermediate_size intermediate_size           feed_forward_length
    vocab_size        vocab_size                  tokenizer list length
    rms_norm_eps      rms_norm_eps                attention.layer_norm_rms_epsilon
    rope_theta        rope_theta                  user flag _rope_freq_base (test/main.cu:27)
    max_position      max_position_embeddings     context_length (_n_ctx)
    tie_word_embeddings                           (none: the reference cannot tie)
    sliding_window / layer_types                  _n_swa / _swa_layers (BaseDefine.h:141-144)
    """
    hidden_size: int = 0
    num_layers: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    max_position: int = 0
    tie_word_embeddings: bool = False
    sliding_window: Optional[int] = None
    layer_types: tuple = ()
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ checks
    def validate(self) -> "Qwen3Config":
        pos = ["hidden_size", "num_layers", "num_heads", "num_kv_heads", "head_dim",
               "intermediate_size", "vocab_size", "max_position"]
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"config: '{k}' must be positive, got {getattr(self, k)}")
        if self.num_heads % self.num_kv_heads != 0:
            raise ConfigError(
                f"config: num_attention_heads ({self.num_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_kv_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config: head_dim ({self.head_dim}) must be even for rotate-half RoPE")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config: rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config: rope_theta must be > 0, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"config: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if len(self.layer_types) != self.num_layers:
            raise ConfigError(
                f"config: layer_types has {len(self.layer_types)} entries for {self.num_layers} layers")
        for t in self.layer_types:
            if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise ConfigError(f"config: unknown layer type '{t}' in layer_types")
        if SLIDING_ATTENTION in self.layer_types:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("config: sliding_attention layers need a positive 'sliding_window'")
        return self

    def window_of_layer(self, i: int) -> int:
        """Number of keys a query of layer ``i`` sees (itself included); 0 = all."""
        return int(self.sliding_window) if self.layer_types[i] == SLIDING_ATTENTION else 0

    # ------------------------------------------------------------- conversion
    @staticmethod
    def from_json_dict(d: Dict[str, Any]) -> "Qwen3Config":
        archs = d.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
        hidden = _get(d, "hidden_size", int)
        heads = _get(d, "num_attention_heads", int)
        layers = _get(d, "num_hidden_layers", int)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _get(d, "head_dim", int)
        else:
            if heads <= 0 or hidden % heads != 0:
                raise ConfigError("config.json: 'head_dim' is absent and hidden_size is not a "
                                  "multiple of num_attention_heads")
            head_dim = hidden // heads
        if _get(d, "attention_bias", bool, False):
            raise ConfigError("config.json: 'attention_bias' = true is not supported "
                              "(the reference's projections have no bias, "
                              "src/core/runtime/GraphOptimizer.cpp:230-232)")
        if d.get("rope_scaling") is not None:
            raise ConfigError("config.json: 'rope_scaling' is not supported (must be null)")
        window = d.get("sliding_window")
        if window is not None and (not isinstance(window, int) or isinstance(window, bool)):
            raise ConfigError(f"config.json: key 'sliding_window' has value {window!r}, expected int or null")
        use_window = _get(d, "use_sliding_window", bool, False)
        if "layer_types" in d and d["layer_types"] is not None:
            lt = d["layer_types"]
            if not isinstance(lt, list) or not all(isinstance(t, str) for t in lt):
                raise ConfigError("config.json: 'layer_types' must be a list of names")
            layer_types = tuple(lt)
        elif use_window and window is not None:
            first = _get(d, "max_window_layers", int, 0)
            layer_types = tuple(SLIDING_ATTENTION if i >= first else FULL_ATTENTION
                                for i in range(layers))
        else:
            layer_types = tuple(FULL_ATTENTION for _ in range(layers))
        if SLIDING_ATTENTION not in layer_types:
            window = None
        cfg = Qwen3Config(
            architecture=archs[0],
            hidden_size=hidden,
            num_layers=layers,
            num_heads=heads,
            num_kv_heads=_get(d, "num_key_value_heads", int),
            head_dim=head_dim,
            intermediate_size=_get(d, "intermediate_size", int),
            vocab_size=_get(d, "vocab_size", int),
            rms_norm_eps=_get(d, "rms_norm_eps", float),
            rope_theta=_get(d, "rope_theta", float),
            max_position=_get(d, "max_position_embeddings", int),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            sliding_window=window,
            layer_types=layer_types,
            hidden_act=_get(d, "hidden_act", str, "silu"),
            torch_dtype=_get(d, "torch_dtype", str, "bfloat16"),
        )
        return cfg.validate()

    def to_json_dict(self) -> Dict[str, Any]:
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "rope_scaling": None,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
            "sliding_window": self.sliding_window,
            "use_sliding_window": SLIDING_ATTENTION in self.layer_types,
            "layer_types": list(self.layer_types),
        }
        return d


def read_config_json(model_dir: str) -> Dict[str, Any]:
    """Parse ``<model_dir>/config.json`` (cf. ModelConfigReader::read,
    src/core/model/base/ModelConfigReader.h:27-61, which reads 'architectures' only)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def write_config_json(model_dir: str, cfg: ModelConfig) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg.to_json_dict(), f, indent=2)
        f.write("\n")
