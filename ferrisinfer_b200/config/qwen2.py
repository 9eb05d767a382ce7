"""Typed configuration of the Qwen2 dense decoder, read from config.json.

Which keys are required, which are optional and what the defaults are follows
the reference's parser (crates/ferrisinfer-io/src/hf.rs:315-369) and its
validation (crates/ferrisinfer-model/src/config.rs:27-71):

* required: hidden_size, intermediate_size, num_attention_heads,
  num_hidden_layers, vocab_size, max_position_embeddings, rms_norm_eps,
  hidden_act, model_type;
* optional: num_key_value_heads (= heads), rope_theta (= 10000.0),
  partial_rotary_factor (= 1.0), tie_word_embeddings (= false);
* an optional key whose value is ``null`` counts as absent
  (crates/ferrisinfer-io/src/hf.rs:629-680).

Beyond the reference, the keys of the architecture's own config.json that the
reference never reads are honoured where they change the result:
``head_dim`` (default hidden_size / heads) and the sliding-window keys
``use_sliding_window`` / ``sliding_window`` / ``max_window_layers`` (layers with
index >= max_window_layers attend a window of ``sliding_window`` keys when
``use_sliding_window`` is true).  ``rope_scaling`` other than null is refused.

No size of the model is written anywhere else in the package: everything is
derived from an instance of this class.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, asdict
from typing import Any, Optional

from .json_file import read_config_json
from ..errors import ConfigError, UnsupportedError

_MISSING = object()


def _get(d: dict, key: str, kind, default=_MISSING):
    """Read ``d[key]`` as ``kind``; ``null`` counts as absent for optional keys."""
    value = d.get(key, None)
    if value is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value)
            raise ConfigError(f"config.json: key '{key}' must be an integer, found {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: key '{key}' must be a number, found {value!r}")
        value = float(value)
        if not math.isfinite(value):
            raise ConfigError(f"config.json: key '{key}' must be finite, found {value!r}")
        return value
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config.json: key '{key}' must be true or false, found {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config.json: key '{key}' must be a string, found {value!r}")
        return value
    raise AssertionError(kind)


@dataclass(frozen=True)
class Qwen2Config:
    """Every number that a Qwen2 model folder's config.json gives."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    hidden_act: str = "silu"
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    architecture: str = "Qwen2ForCausalLM"
    model_type: str = "qwen2"

    # ------------------------------------------------------------------ derived
    @property
    def rotary_dim(self) -> int:
        """Leading dims of a head that are rotated: round(head_dim * factor)
        (crates/ferrisinfer-io/src/hf.rs:334-335)."""
        return int(round(self.head_dim * self.partial_rotary_factor))

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        """Number of keys (the query's own included) that layer ``layer`` attends,
        or None for all of them."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        first_windowed = (
            self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        )
        return self.sliding_window if layer >= first_windowed else None

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "max_position_embeddings",
        ):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be > 0, found {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "config.json: num_attention_heads must be divisible by num_key_value_heads "
                f"({self.num_attention_heads} / {self.num_key_value_heads})"
            )
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config.json: rms_norm_eps must be > 0, found {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta must be > 0, found {self.rope_theta}")
        r = self.rotary_dim
        if r < 0 or r > self.head_dim or r % 2 != 0:
            raise ConfigError(
                f"config.json: rotary dims ({r}) must be even and at most head_dim ({self.head_dim})"
            )
        if self.hidden_act not in ("silu", "swish"):
            raise UnsupportedError(
                f"activation '{self.hidden_act}' is not supported (the gated feed-forward is SiLU only)"
            )
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError(
                    "config.json: use_sliding_window is true but sliding_window is not a positive integer"
                )
            if self.max_window_layers is not None and self.max_window_layers < 0:
                raise ConfigError("config.json: max_window_layers must be >= 0")

    # --------------------------------------------------------------------- I/O
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        model_type = _get(d, "model_type", str)
        if model_type != "qwen2":
            raise UnsupportedError(f"model_type '{model_type}' is not supported by Qwen2Config")
        archs = d.get("architectures") or ["Qwen2ForCausalLM"]
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of strings")
        hidden = _get(d, "hidden_size", int)
        heads = _get(d, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be > 0")
        head_dim = _get(d, "head_dim", int, None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    "config.json: hidden_size must be divisible by num_attention_heads "
                    "when head_dim is not given"
                )
            head_dim = hidden // heads
        scaling = d.get("rope_scaling")
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                raise UnsupportedError(f"rope_scaling {scaling!r} is not supported")
        cfg = cls(
            vocab_size=_get(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_get(d, "intermediate_size", int),
            num_hidden_layers=_get(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=_get(d, "num_key_value_heads", int, heads),
            head_dim=head_dim,
            max_position_embeddings=_get(d, "max_position_embeddings", int),
            rms_norm_eps=_get(d, "rms_norm_eps", float),
            rope_theta=_get(d, "rope_theta", float, 10000.0),
            partial_rotary_factor=_get(d, "partial_rotary_factor", float, 1.0),
            hidden_act=_get(d, "hidden_act", str),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            use_sliding_window=_get(d, "use_sliding_window", bool, False),
            sliding_window=_get(d, "sliding_window", int, None),
            max_window_layers=_get(d, "max_window_layers", int, None),
            bos_token_id=_get(d, "bos_token_id", int, None),
            eos_token_id=_get(d, "eos_token_id", int, None),
            architecture=archs[0],
            model_type=model_type,
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        return d

    @classmethod
    def from_json(cls, path: str) -> "Qwen2Config":
        return cls.from_dict(read_config_json(path))
