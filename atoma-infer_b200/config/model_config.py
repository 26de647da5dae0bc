"""Typed view of a Llama ``config.json``.

Keys, optionals and defaults follow the reference's serde struct
(models/src/llama.rs:36-52): ``num_key_value_heads`` defaults to the number of
query heads (:54-57), ``rope_theta`` to 10000 (:60-62), ``tie_word_embeddings``
to false (:79); ``rope_scaling``, when present, needs all five keys (:21-28) and
its ``rope_type`` is "llama3" or "default" (:12-19); ``eos_token_id`` is an int
or a list (:29-34).  The head size is ``hidden_size / num_attention_heads``
unless ``head_dim`` is given (the reference fixes the quotient in code, :147, :326).

Keys the reference ignores but that would change the math are checked here, so a
checkpoint this engine cannot run is refused instead of run wrongly.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency scaling (models/src/llama.rs:21-28)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int
    rope_type: str  # "llama3" | "default"

    _KEYS = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")

    @staticmethod
    def from_dict(d: dict) -> "RopeScaling":
        if not isinstance(d, dict):
            raise ConfigError(f"rope_scaling must be an object, got {type(d).__name__}")
        kind = d.get("rope_type", d.get("type"))
        if kind is None:
            raise ConfigError("rope_scaling.rope_type is missing")
        if kind not in ("llama3", "default"):
            raise ConfigError(f"rope_scaling.rope_type {kind!r} is not supported (known: 'llama3', 'default')")
        missing = [k for k in RopeScaling._KEYS if k not in d]
        if missing:
            raise ConfigError(f"rope_scaling is missing {missing}")
        rs = RopeScaling(
            factor=float(d["factor"]),
            low_freq_factor=float(d["low_freq_factor"]),
            high_freq_factor=float(d["high_freq_factor"]),
            original_max_position_embeddings=int(d["original_max_position_embeddings"]),
            rope_type=kind,
        )
        if kind == "llama3":
            if rs.factor <= 0:
                raise ConfigError("rope_scaling.factor must be > 0")
            if rs.high_freq_factor == rs.low_freq_factor:
                raise ConfigError("rope_scaling.high_freq_factor must differ from low_freq_factor")
            if rs.original_max_position_embeddings <= 0:
                raise ConfigError("rope_scaling.original_max_position_embeddings must be > 0")
        return rs

    def to_dict(self) -> dict:
        return {k: getattr(self, k) for k in self._KEYS} | {"rope_type": self.rope_type}


def _require(d: dict, key: str, typ):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json is missing the required key {key!r}")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json key {key!r} must be an integer, got {v!r}")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json key {key!r} must be a number, got {v!r}")
        return float(v)
    return v


@dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of the architecture; nothing of these stands in code."""

    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "LlamaForCausalLM"

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_dict(d: dict) -> "LlamaConfig":
        hidden = _require(d, "hidden_size", int)
        heads = _require(d, "num_attention_heads", int)
        kv = d.get("num_key_value_heads")
        kv = heads if kv is None else _require(d, "num_key_value_heads", int)
        if heads <= 0 or kv <= 0:
            raise ConfigError("num_attention_heads and num_key_value_heads must be positive")
        if d.get("head_dim") is not None:
            head_dim = _require(d, "head_dim", int)
        else:
            if hidden % heads:
                raise ConfigError(
                    f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} and no head_dim is given"
                )
            head_dim = hidden // heads
        if heads % kv:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv}")
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even (rotary pairs)")
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ConfigError("attention_bias / mlp_bias = true is not supported (the architecture has no biases)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (the architecture uses 'silu')")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        scaling = d.get("rope_scaling")
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        cfg = LlamaConfig(
            hidden_size=hidden,
            intermediate_size=_require(d, "intermediate_size", int),
            vocab_size=_require(d, "vocab_size", int),
            num_hidden_layers=_require(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            rms_norm_eps=_require(d, "rms_norm_eps", float),
            rope_theta=float(d["rope_theta"]) if d.get("rope_theta") is not None else 10000.0,
            max_position_embeddings=_require(d, "max_position_embeddings", int),
            rope_scaling=RopeScaling.from_dict(scaling) if scaling is not None else None,
            tie_word_embeddings=bool(d.get("tie_word_embeddings") or False),
            bos_token_id=d.get("bos_token_id"),
            eos_token_ids=eos_ids,
            architecture=str(archs[0]),
        )
        for k in ("hidden_size", "intermediate_size", "vocab_size", "num_hidden_layers", "max_position_embeddings"):
            if getattr(cfg, k) <= 0:
                raise ConfigError(f"config.json key {k!r} must be positive, got {getattr(cfg, k)}")
        if cfg.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be > 0")
        if cfg.rope_theta <= 0:
            raise ConfigError("rope_theta must be > 0")
        return cfg

    @staticmethod
    def from_file(path: str) -> "LlamaConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return LlamaConfig.from_dict(json.load(f))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": list(self.eos_token_ids) if len(self.eos_token_ids) != 1 else self.eos_token_ids[0],
        }
        if not self.eos_token_ids:
            d["eos_token_id"] = None
        return d

    # ------------------------------------------------------------------ derived
    @property
    def softmax_scale(self) -> float:
        """1/sqrt(head_dim) (models/src/llama.rs:342)."""
        return 1.0 / (self.head_dim ** 0.5)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_parameters(self) -> int:
        per_layer = (
            self.hidden_size * (self.q_size + 2 * self.kv_size)
            + self.q_size * self.hidden_size
            + 3 * self.hidden_size * self.intermediate_size
            + 2 * self.hidden_size
        )
        n = self.num_hidden_layers * per_layer + self.vocab_size * self.hidden_size + self.hidden_size
        if not self.tie_word_embeddings:
            n += self.vocab_size * self.hidden_size
        return n
