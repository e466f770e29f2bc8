"""Seeded random weights, and a writer that turns a configuration and a seed
into a model folder (config.json + model.safetensors).

Matrices are N(0, 0.02) and norm weights 1.0.  Each tensor is drawn from its
own generator keyed by (seed, tensor name), so any tensor can be regenerated
alone and the result does not depend on the order of generation.  (The
reference only generates weights in tests: src/model/arch/llama/tests.rs:86-94.)
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Optional

import torch

from ..spec import TensorSpec
from .safetensors_io import write_safetensors

INIT_STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: Optional[torch.device] = None) -> torch.Tensor:
    device = torch.device(device) if device is not None else torch.device("cpu")
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.kind == "vector":
        return torch.ones(spec.shape, dtype=dtype, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    t = torch.empty(spec.shape, dtype=torch.float32 if device.type == "cpu" else dtype, device=device)
    t.normal_(0.0, INIT_STD, generator=gen)
    return t.to(dtype)


def random_tensors(expected: dict[str, TensorSpec], seed: int, dtype: torch.dtype,
                   device: Optional[torch.device] = None) -> dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, dtype, device) for name, spec in expected.items()}


def write_random_model(model_dir: str, config_dict: dict, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write config.json and model.safetensors for `config_dict` with seeded weights."""
    from ..config import load_config
    from ..engine.model import expected_tensors
    arch, cfg = load_config(config_dict)
    expected = expected_tensors(arch.describe(cfg))
    os.makedirs(model_dir, exist_ok=True)
    out = dict(config_dict)
    out.setdefault("torch_dtype", {torch.bfloat16: "bfloat16", torch.float32: "float32",
                                   torch.float16: "float16"}[dtype])
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(expected, seed, dtype), metadata={"format": "pt", "seed": seed})
    return model_dir
