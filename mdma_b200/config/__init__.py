"""Configuration: typed per-architecture configs and the architecture registry."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable

from ..registry import ARCHITECTURES, RegistryError
from ..spec import ModelSpec
from .llama import ConfigError, LlamaConfig, RopeScaling, read_config_json


@dataclass(frozen=True)
class Architecture:
    """What the registry holds for one architecture name."""
    name: str
    config_from_dict: Callable[[dict], Any]
    describe: Callable[[Any], ModelSpec]     # typed config -> ModelSpec


def architecture_name(raw: dict) -> str:
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs:
        return archs[0]
    if isinstance(raw.get("model_type"), str):
        return raw["model_type"]
    raise ConfigError("config.json names no architecture (`architectures` or `model_type`)")


def load_config(model_dir_or_dict):
    """Read config.json (or take its dict) and return (Architecture, typed config)."""
    raw = (read_config_json(model_dir_or_dict)
           if isinstance(model_dir_or_dict, (str, os.PathLike)) else dict(model_dir_or_dict))
    arch = ARCHITECTURES.get(architecture_name(raw))
    return arch, arch.config_from_dict(raw)


from . import llama_arch  # noqa: E402,F401  registers the Llama architecture

__all__ = ["Architecture", "ConfigError", "LlamaConfig", "RopeScaling", "RegistryError",
           "architecture_name", "load_config", "read_config_json"]
