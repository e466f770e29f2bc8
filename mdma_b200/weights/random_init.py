"""Seeded random weights, and a writer that turns a configuration and a seed
into a model folder (config.json + model.safetensors).

Matrices are N(0, std) with std 0.02 by default, and norm weights 1.0.  Every
element is a function of (seed, tensor name, element index) alone: a
counter-based hash picks a quantile of the normal distribution from a table.
So any tensor can be regenerated alone, the order of generation does not
matter, and the device fills its weights with the same bits as the folder
writer on the host (`normal_values` here, `fill_normal_kernel` in
csrc/elementwise.cu: the same integer hash, and floating-point steps that are
single correctly rounded operations on both sides).  The reference generates
weights only in tests, with a closed form of the index for the same reason
(src/model/arch/llama/tests.rs:86-94).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Optional

import numpy as np
import torch

from ..spec import TensorSpec
from .safetensors_io import write_safetensors

INIT_STD = 0.02
_TABLE_SIZE = 65537
_table: Optional[np.ndarray] = None


def tensor_key(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little")


def quantile_table() -> np.ndarray:
    """float32 [65537]: the normal quantiles at (j + 0.5) / 65537."""
    global _table
    if _table is None:
        q = (torch.arange(_TABLE_SIZE, dtype=torch.float64) + 0.5) / _TABLE_SIZE
        _table = (torch.erfinv(2.0 * q - 1.0) * (2.0 ** 0.5)).to(torch.float32).numpy()
    return _table


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def normal_values(key: int, start: int, count: int, std: float) -> np.ndarray:
    """float32 [count]: elements start .. start+count of the stream of `key`."""
    table = quantile_table()
    with np.errstate(over="ignore"):
        i = np.arange(start, start + count, dtype=np.uint64)
        z = _mix64(_mix64(np.uint64(key) ^ i))
    j = (z >> np.uint64(48)).astype(np.int64)
    f = ((z >> np.uint64(40)) & np.uint64(0xFF)).astype(np.float32) * np.float32(1.0 / 256.0)
    lo = table[j]
    v = lo + (table[j + 1] - lo) * f            # float32 throughout: three single rounded operations
    return v * np.float32(std)


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: Optional[torch.device] = None, std: float = INIT_STD,
                  out: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The tensor `name` of the model seeded with `seed`.  On a CUDA device (or into a CUDA `out`)
    the values are made by the device kernel; they are the host's, bit for bit."""
    if out is not None:
        device, dtype = out.device, out.dtype
    device = torch.device(device) if device is not None else torch.device("cpu")
    how = spec.initial()
    if how not in ("normal", "ones", "zeros"):
        raise ValueError(f"{name}: unknown initialisation {how!r}")
    if spec.kind == "int" or how != "normal":
        t = (torch.ones if how == "ones" else torch.zeros)(
            spec.shape, dtype=torch.int32 if spec.kind == "int" else dtype, device=device)
    elif device.type == "cuda":
        from .. import ops
        t = out if out is not None else torch.empty(spec.shape, dtype=dtype, device=device)
        if table is None:
            table = torch.from_numpy(quantile_table()).to(device)
        ops.fill_normal(t, tensor_key(seed, name), table, std)
        return t
    else:
        n = int(np.prod(spec.shape))
        key = tensor_key(seed, name)
        t = torch.empty(n, dtype=dtype)
        for lo in range(0, n, 1 << 24):         # in pieces: the hash works on 64-bit temporaries
            hi = min(n, lo + (1 << 24))
            t[lo:hi] = torch.from_numpy(normal_values(key, lo, hi - lo, std)).to(dtype)
        t = t.reshape(spec.shape)
    if out is not None:
        out.copy_(t)
        return out
    return t


def random_tensors(expected: dict[str, TensorSpec], seed: int, dtype: torch.dtype,
                   device: Optional[torch.device] = None, std: float = INIT_STD) -> dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, dtype, device, std) for name, spec in expected.items()}


def write_random_model(model_dir: str, config_dict: dict, seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: float = INIT_STD) -> str:
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
                      random_tensors(expected, seed, dtype, std=std), metadata={"format": "pt", "seed": seed})
    return model_dir
