"""Model configurations, read from the architecture's own ``config.json`` keys.

``GPT2Config`` keeps the Hugging Face short names (``n_layer``, ``n_embd`` ...)
and also accepts the long spellings the reference uses
(``models/gpt2.py:68-75``).  Defaults and checks follow ``models/gpt2.py:91-134``
with one difference: ``scale_attn_by_inverse_layer_idx`` is supported here (the
reference raises on it, ``models/gpt2.py:131-132``).
"""

from __future__ import annotations

import dataclasses
import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar, Mapping


class ConfigError(ValueError):
    """A configuration value is missing, of the wrong type or out of range."""


def _require_int(value: Any, name: str, minimum: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"{name} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"{name} must be >= {minimum}, got {value}")
    return value


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    ``from_dict`` renames aliases, keeps the keys the dataclass declares and
    drops the rest (``models/_common.py:82-111``)."""

    ALIASES: ClassVar[Mapping[str, str]] = {}
    ARCHITECTURE: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, values: Mapping[str, Any]):
        names = {f.name for f in dataclasses.fields(cls)}
        picked: dict[str, Any] = {}
        for key, value in values.items():
            key = cls.ALIASES.get(key, key)
            if key in names:
                if key in picked and picked[key] != value:
                    raise ConfigError(f"{key} is given twice with different values")
                picked[key] = value
        return cls(**picked)

    @classmethod
    def from_folder(cls, folder):
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text(encoding="utf-8")))

    def to_dict(self) -> dict[str, Any]:
        """The config.json document of this configuration."""
        doc = {"architectures": [self.ARCHITECTURE]}
        doc.update(dataclasses.asdict(self))
        return doc


_GPT2_ACTIVATIONS = ("gelu", "gelu_new", "gelu_fast", "gelu_pytorch_tanh", "quick_gelu")


@dataclass(frozen=True)
class GPT2Config(ModelConfig):
    ALIASES: ClassVar[Mapping[str, str]] = {
        "hidden_size": "n_embd",
        "num_hidden_layers": "n_layer",
        "num_attention_heads": "n_head",
        "max_position_embeddings": "n_positions",
        "intermediate_size": "n_inner",
        "layer_norm_eps": "layer_norm_epsilon",
    }
    ARCHITECTURE: ClassVar[str] = "GPT2LMHeadModel"

    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: int | None = None
    activation_function: str = "gelu_new"
    layer_norm_epsilon: float = 1e-5
    scale_attn_weights: bool = True
    scale_attn_by_inverse_layer_idx: bool = False
    reorder_and_upcast_attn: bool = False
    tie_word_embeddings: bool = True
    bos_token_id: int = 50256
    eos_token_id: int = 50256
    model_type: str = "gpt2"

    def __post_init__(self) -> None:
        for name in ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head"):
            _require_int(getattr(self, name), name)
        if self.n_inner is not None:
            _require_int(self.n_inner, "n_inner")
        if self.n_embd % self.n_head:
            raise ConfigError(f"n_embd ({self.n_embd}) must be divisible by n_head ({self.n_head})")
        if self.activation_function not in _GPT2_ACTIVATIONS:
            raise ConfigError(
                f"unsupported activation_function {self.activation_function!r}; "
                f"expected one of {sorted(_GPT2_ACTIVATIONS)}")
        eps = self.layer_norm_epsilon
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not math.isfinite(eps) or eps <= 0:
            raise ConfigError("layer_norm_epsilon must be finite and positive")
        for name in ("scale_attn_weights", "scale_attn_by_inverse_layer_idx",
                     "reorder_and_upcast_attn", "tie_word_embeddings"):
            if not isinstance(getattr(self, name), bool):
                raise ConfigError(f"{name} must be true or false")
        if self.reorder_and_upcast_attn:
            # It only asks for 32-bit attention scores, which every kernel here
            # computes anyway (the reference refuses it, models/gpt2.py:133-134).
            pass

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_size(self) -> int:
        """``n_inner``, or 4 * n_embd when it is null (models/gpt2.py:140-145)."""
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    def attention_scale(self, layer: int) -> float:
        """Dh^-0.5 when ``scale_attn_weights`` (models/gpt2.py:147-149), divided
        by (layer + 1) when ``scale_attn_by_inverse_layer_idx``."""
        scale = self.head_dim ** -0.5 if self.scale_attn_weights else 1.0
        if self.scale_attn_by_inverse_layer_idx:
            scale /= float(layer + 1)
        return scale
