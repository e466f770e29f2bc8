"""Typed configuration of the dense Llama decoder, read from config.json.

Every size and constant the model uses comes from here; no layer code holds a
number that config.json gives.  The admission rules follow the reference's
metadata-only preflight (src/model/arch/llama/preflight.rs:49-116): required
keys must be positive, geometry must divide, and a key the engine does not
implement rejects the file instead of being ignored.  The GGUF keys of
src/model/arch/llama.rs:16-38 map one to one onto the config.json keys below
(block_count -> num_hidden_layers, embedding_length -> hidden_size,
feed_forward_length -> intermediate_size, attention.head_count ->
num_attention_heads, attention.head_count_kv -> num_key_value_heads,
rope.freq_base -> rope_theta, attention.layer_norm_rms_epsilon ->
rms_norm_eps, context_length -> max_position_embeddings).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a bad value, or asks for something unbuilt."""


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency scaling: long wavelengths are slowed by `factor`,
    short ones kept, the band between blended."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def validate(self) -> None:
        if self.rope_type != "llama3":
            raise ConfigError(
                f"rope_scaling.rope_type {self.rope_type!r} is not implemented (only 'llama3')")
        for name in ("factor", "low_freq_factor", "high_freq_factor"):
            v = getattr(self, name)
            if not (isinstance(v, (int, float)) and math.isfinite(v) and v > 0):
                raise ConfigError(f"rope_scaling.{name} must be a finite positive number, got {v!r}")
        if self.factor < 1.0:
            raise ConfigError("rope_scaling.factor must be >= 1")
        if not self.high_freq_factor > self.low_freq_factor:
            raise ConfigError("rope_scaling.high_freq_factor must exceed low_freq_factor")
        if not (isinstance(self.original_max_position_embeddings, int)
                and self.original_max_position_embeddings > 0):
            raise ConfigError("rope_scaling.original_max_position_embeddings must be a positive integer")


# Keys that change nothing the engine computes.
_COSMETIC_KEYS = {
    "architectures", "model_type", "torch_dtype", "dtype", "transformers_version",
    "bos_token_id", "pad_token_id", "use_cache", "initializer_range", "_name_or_path",
}
# Keys that are accepted only at the one value the engine implements.
_PINNED_KEYS = {
    "hidden_act": ("silu",),
    "attention_bias": (False,),
    "mlp_bias": (False,),
    "attention_dropout": (0, 0.0),
    "pretraining_tp": (1,),
    "sliding_window": (None,),
}

_REQUIRED_INT = ("num_hidden_layers", "hidden_size", "intermediate_size",
                 "num_attention_heads", "max_position_embeddings", "vocab_size")


@dataclass(frozen=True)
class LlamaConfig:
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0          # llama.rs:14 default when the key is absent
    rope_scaling: Optional[RopeScaling] = None
    rope_layout: str = "split_half"      # "split_half" pairs (i, i+d/2); "interleaved" pairs (2i, 2i+1)
    tie_word_embeddings: bool = False
    eos_token_id: tuple = field(default_factory=tuple)
    architecture: str = "LlamaForCausalLM"

    # ---- derived sizes -------------------------------------------------
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ---- construction --------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "LlamaConfig":
        d = dict(d)
        for key in _REQUIRED_INT:
            v = d.get(key)
            if not (isinstance(v, int) and not isinstance(v, bool) and v > 0):
                raise ConfigError(f"{key} must be a positive integer, got {v!r}")
        eps = d.get("rms_norm_eps")
        if not (isinstance(eps, (int, float)) and not isinstance(eps, bool)
                and math.isfinite(eps) and eps > 0):
            raise ConfigError(f"rms_norm_eps must be a finite positive float, got {eps!r}")
        heads = d["num_attention_heads"]
        kv_heads = d.get("num_key_value_heads", heads)
        if kv_heads is None:
            kv_heads = heads
        if not (isinstance(kv_heads, int) and kv_heads > 0):
            raise ConfigError(f"num_key_value_heads must be a positive integer, got {kv_heads!r}")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if d["hidden_size"] % heads:
                raise ConfigError(
                    f"hidden_size {d['hidden_size']} is not a multiple of num_attention_heads {heads} "
                    "and no head_dim is given")
            head_dim = d["hidden_size"] // heads
        if not (isinstance(head_dim, int) and head_dim > 0):
            raise ConfigError(f"head_dim must be a positive integer, got {head_dim!r}")
        theta = d.get("rope_theta", 10000.0)
        if not (isinstance(theta, (int, float)) and math.isfinite(theta) and theta > 0):
            raise ConfigError(f"rope_theta must be a finite positive float, got {theta!r}")

        scaling = d.get("rope_scaling")
        rs = None
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError("rope_scaling must be an object or null")
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind not in (None, "default", "llama3"):
                raise ConfigError(f"rope_scaling.rope_type {kind!r} is not implemented (only 'llama3')")
            if kind == "llama3":
                known = {"rope_type", "type", "factor", "low_freq_factor", "high_freq_factor",
                         "original_max_position_embeddings"}
                extra = sorted(set(scaling) - known)
                if extra:
                    raise ConfigError(f"rope_scaling has unimplemented keys {extra}")
                try:
                    rs = RopeScaling(
                        rope_type=kind,
                        factor=scaling["factor"],
                        low_freq_factor=scaling["low_freq_factor"],
                        high_freq_factor=scaling["high_freq_factor"],
                        original_max_position_embeddings=scaling["original_max_position_embeddings"],
                    )
                except KeyError as e:
                    raise ConfigError(f"rope_scaling is missing {e.args[0]!r}") from None
                rs.validate()

        layout = d.get("rope_layout", "split_half")
        if layout not in ("split_half", "interleaved"):
            raise ConfigError(f"rope_layout must be 'split_half' or 'interleaved', got {layout!r}")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")

        for key, allowed in _PINNED_KEYS.items():
            if key in d and d[key] not in allowed:
                raise ConfigError(f"{key}={d[key]!r} is not implemented (only {allowed[0]!r})")

        known = (set(_REQUIRED_INT) | _COSMETIC_KEYS | set(_PINNED_KEYS) |
                 {"rms_norm_eps", "num_key_value_heads", "head_dim", "rope_theta", "rope_scaling",
                  "rope_layout", "tie_word_embeddings", "eos_token_id"})
        unknown = sorted(set(d) - known)
        if unknown:
            raise ConfigError(f"unimplemented configuration keys {unknown}")

        arch = d.get("architectures") or [d.get("model_type") or "LlamaForCausalLM"]
        cfg = cls(
            num_hidden_layers=d["num_hidden_layers"],
            hidden_size=d["hidden_size"],
            intermediate_size=d["intermediate_size"],
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=d["vocab_size"],
            max_position_embeddings=d["max_position_embeddings"],
            rms_norm_eps=float(eps),
            rope_theta=float(theta),
            rope_scaling=rs,
            rope_layout=layout,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_id=eos_ids,
            architecture=arch[0],
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        # Geometry rules of preflight.rs:76-85; head_dim is explicit here, so the
        # hidden width need not equal heads x head_dim.
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even (rotary pairs)")

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": asdict(self.rope_scaling) if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rope_layout != "split_half":
            d["rope_layout"] = self.rope_layout
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path} does not exist")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d
