"""Typed model configuration, read from the architecture's own config.json keys.

The reference reads config.json through `transformers.AutoConfig`
(liteinfer/models/loader.py:100) and then reads these attributes in
liteinfer/models/llama.py:64-74,108-111,130-140,171-172,204-208,246. This
module parses the same keys directly, so nothing here depends on a library's
model code.  Sizes have no defaults: a config.json that leaves one out is
refused.  Options that the architecture defines a default for (no rope scaling,
untied head, no biases) take that default when the key is absent.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine cannot run."""


_ROPE_TYPES = ("default", "linear", "llama3")
_ACTIVATIONS = ("silu", "gelu", "gelu_pytorch_tanh", "relu")


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling of rotary embeddings (config.json `rope_scaling` / `rope_parameters`).

    `default`: none.  `linear`: every frequency divided by `factor`.  `llama3`:
    wavelengths above `original_max_position_embeddings / low_freq_factor` are
    divided by `factor`, those below `original / high_freq_factor` are kept, and
    the band between is interpolated (the rule the reference gets from
    ROPE_INIT_FUNCTIONS["llama3"], liteinfer/models/llama.py:73-74).
    """

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0

    def __post_init__(self) -> None:
        if self.rope_type not in _ROPE_TYPES:
            raise ConfigError(f"rope_type {self.rope_type!r} is not supported; known: {list(_ROPE_TYPES)}")
        if self.rope_type != "default" and not self.factor > 0:
            raise ConfigError("rope scaling factor must be > 0")
        if self.rope_type == "llama3":
            if self.original_max_position_embeddings < 1:
                raise ConfigError("llama3 rope scaling needs original_max_position_embeddings >= 1")
            if not self.high_freq_factor > self.low_freq_factor > 0:
                raise ConfigError("llama3 rope scaling needs high_freq_factor > low_freq_factor > 0")


def _require(raw: dict[str, Any], key: str, kind: type) -> Any:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json has no {key!r}")
    value = raw[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json {key!r} must be an integer, got {value!r}")
    if kind is float and (isinstance(value, bool) or not isinstance(value, (int, float))):
        raise ConfigError(f"config.json {key!r} must be a number, got {value!r}")
    return kind(value)


# What the architecture's configuration class assumes for keys a config.json leaves out (sizes have no defaults here).
_DEFAULT_ROPE_THETA = 10000.0
_DEFAULT_RMS_NORM_EPS = 1e-6


def _parse_rope(raw: dict[str, Any]) -> tuple[float, RopeScaling]:
    """Both spellings: legacy `rope_theta` + `rope_scaling`, and the merged `rope_parameters`."""
    merged: dict[str, Any] = {}
    if isinstance(raw.get("rope_scaling"), dict):
        merged.update(raw["rope_scaling"])
    if isinstance(raw.get("rope_parameters"), dict):
        merged.update(raw["rope_parameters"])
    # A config.json that names no base gets the architecture's own default, as it does through the reference's
    # configuration class (liteinfer/models/llama.py:64-70 reads what that class filled in).
    theta = merged.get("rope_theta", raw.get("rope_theta", _DEFAULT_ROPE_THETA))
    if theta is None:
        theta = _DEFAULT_ROPE_THETA
    rope_type = merged.get("rope_type", merged.get("type", "default"))
    scaling = RopeScaling(
        rope_type=str(rope_type),
        factor=float(merged.get("factor", 1.0)),
        low_freq_factor=float(merged.get("low_freq_factor", 1.0)),
        high_freq_factor=float(merged.get("high_freq_factor", 4.0)),
        original_max_position_embeddings=int(merged.get("original_max_position_embeddings", 0) or 0),
    )
    return float(theta), scaling


@dataclass(frozen=True)
class LlamaConfig:
    """The dense grouped-query Llama decoder's sizes and options."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    eos_token_id: tuple[int, ...] = ()
    bos_token_id: int | None = None
    architecture: str = "LlamaForCausalLM"

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be >= 1, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary embeddings")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be > 0")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be > 0")
        if self.hidden_act not in _ACTIVATIONS:
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported; known: {list(_ACTIVATIONS)}")

    @property
    def num_kv_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> LlamaConfig:
        heads = _require(raw, "num_attention_heads", int)
        hidden = _require(raw, "hidden_size", int)
        kv_heads = raw.get("num_key_value_heads")
        head_dim = raw.get("head_dim")
        if head_dim is None:
            # liteinfer/models/llama.py:130 — fallback hidden_size // num_attention_heads.
            if hidden % heads:
                raise ConfigError("hidden_size is not a multiple of num_attention_heads and no head_dim is given")
            head_dim = hidden // heads
        theta, scaling = _parse_rope(raw)
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        architectures = raw.get("architectures") or ["LlamaForCausalLM"]
        return cls(
            vocab_size=_require(raw, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size", int),
            num_hidden_layers=_require(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=int(kv_heads) if kv_heads is not None else heads,
            head_dim=int(head_dim),
            rms_norm_eps=_require(raw, "rms_norm_eps", float) if raw.get("rms_norm_eps") is not None else _DEFAULT_RMS_NORM_EPS,
            rope_theta=theta,
            rope_scaling=scaling,
            max_position_embeddings=int(raw.get("max_position_embeddings") or 0),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            hidden_act=str(raw.get("hidden_act", "silu")),
            attention_bias=bool(raw.get("attention_bias", False)),
            mlp_bias=bool(raw.get("mlp_bias", False)),
            eos_token_id=eos_ids,
            bos_token_id=raw.get("bos_token_id"),
            architecture=str(architectures[0]),
        )

    def to_dict(self) -> dict[str, Any]:
        """config.json contents that `from_dict` reads back to an equal config."""
        out = asdict(self)
        out.pop("architecture")
        out["architectures"] = [self.architecture]
        out["model_type"] = "llama"
        scaling = out.pop("rope_scaling")
        if scaling["rope_type"] == "default":
            out["rope_scaling"] = None
        elif scaling["rope_type"] == "linear":
            out["rope_scaling"] = {"rope_type": "linear", "factor": scaling["factor"]}
        else:
            out["rope_scaling"] = scaling
        eos = out.pop("eos_token_id")
        out["eos_token_id"] = list(eos) if len(eos) != 1 else eos[0]
        if not eos:
            out["eos_token_id"] = None
        return out


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    """config.json of a model folder (liteinfer/models/loader.py:31-39: a missing file is FileNotFoundError)."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"missing config.json under {model_dir}")
    raw = json.loads(path.read_text())
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return raw
