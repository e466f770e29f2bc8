"""Weights by tensor name, checked against what the model's parts declare.

All checks run on headers only, before a byte is uploaded (the reference's
rule: src/model/preflight.rs:119-175, tested with a backend that counts
allocations, src/model/arch/llama/preflight/tests.rs:98-116).  Every problem
of a folder is reported in one `WeightsError`: tensors the model needs and the
file lacks, tensors the file has and no part claims (src/model/preflight.rs:135-140),
wrong shapes and unusable dtypes.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from ..spec import TensorSpec
from .safetensors_io import CheckpointError, SafetensorsFile

_FLOATS = (torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightsError(ValueError):
    """The folder's tensors do not match the model. Lists every mismatch."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, where=""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)      # (name, found, expected)
        self.wrong_dtype = sorted(wrong_dtype)      # (name, found, expected kind)
        lines = [f"weights in {where} do not match the model:" if where else
                 "weights do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(f)}, expected {list(e)}" for n, f, e in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {f}, expected {e}" for n, f, e in self.wrong_dtype))
        super().__init__("\n".join(lines))


def open_model_files(model_dir: str) -> list[SafetensorsFile]:
    """`model.safetensors`, or the shards named by `model.safetensors.index.json`."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            try:
                weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise CheckpointError(f"{index}: no usable weight_map") from None
        files = [SafetensorsFile(os.path.join(model_dir, shard)) for shard in sorted(set(weight_map.values()))]
        seen: dict[str, str] = {}
        for sf in files:
            for name in sf.entries:
                if name in seen:
                    raise CheckpointError(f"tensor {name!r} is in both {seen[name]} and {sf.path}")
                seen[name] = sf.path
        return files
    raise CheckpointError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")


def check_entries(entries: dict, expected: dict[str, TensorSpec], where: str = "") -> None:
    """Compare header entries (name -> object with .shape/.dtype) with the model's needs."""
    missing = [n for n in expected if n not in entries]
    unexpected = [n for n in entries if n not in expected]
    wrong_shape, wrong_dtype = [], []
    for name, spec in expected.items():
        e = entries.get(name)
        if e is None:
            continue
        if tuple(e.shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(e.shape), tuple(spec.shape)))
        if spec.kind == "int":
            if e.dtype not in _INTS:
                wrong_dtype.append((name, str(e.dtype), "an integer type"))
        elif e.dtype not in _FLOATS:
            wrong_dtype.append((name, str(e.dtype), "float32, float16 or bfloat16"))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(missing, unexpected, wrong_shape, wrong_dtype, where)


def resident_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is held in.  In the bfloat16 engine matrices are
    bfloat16, integer tables int32, and vectors stay as stored (float32 stays
    float32); in the float32 engine every float tensor is float32."""
    if spec.kind == "int":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if spec.kind == "matrix":
        return torch.bfloat16
    return torch.float32 if stored in (torch.float32, torch.float16) else torch.bfloat16


class _Staging:
    """Two pinned host buffers that take turns: a piece of a tensor is converted into one (on the host,
    to the dtype it is kept in) while the copy of the piece before runs out of the other.  The reference
    stages its uploads through one host buffer the size of the largest tensor (src/model/planning.rs:44-53);
    here the pieces are of a fixed size, so host memory does not grow with the model."""

    def __init__(self, nbytes: int):
        self.nbytes = max(int(nbytes), 1 << 12)
        self.bufs = [torch.empty(self.nbytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.events = [torch.cuda.Event(), torch.cuda.Event()]
        self.turn = 0

    def copy(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        """dst (device, contiguous) <- src (host, same shape, any float/int dtype)."""
        flat_src, flat_dst = src.reshape(-1), dst.view(-1) if dst.is_contiguous() else None
        if flat_dst is None:
            dst.copy_(src.to(dst.dtype))
            return
        per = self.nbytes // dst.element_size()
        for lo in range(0, flat_dst.numel(), per):
            hi = min(flat_dst.numel(), lo + per)
            self.turn ^= 1
            self.events[self.turn].synchronize()            # the copy that used this buffer last is done
            stage = self.bufs[self.turn][:(hi - lo) * dst.element_size()].view(dst.dtype)
            stage.copy_(flat_src[lo:hi])                    # dtype conversion on the host, into pinned memory
            flat_dst[lo:hi].copy_(stage, non_blocking=True)
            self.events[self.turn].record()

    def finish(self) -> None:
        for e in self.events:
            e.synchronize()


def load_tensors(model_dir: str, expected: dict[str, TensorSpec], compute: torch.dtype,
                 device: Optional[torch.device] = None, into: Optional[dict] = None,
                 staging_bytes: int = 64 << 20) -> dict[str, torch.Tensor]:
    """Validate the folder against `expected`, then fetch each tensor by name.  With `into`
    (name -> a tensor of the right shape and resident dtype, e.g. a view of an engine's arena)
    the values are copied there and no device memory is taken for them here: pieces of
    `staging_bytes` are converted on the host into pinned memory and copied from there while the
    next piece is being converted."""
    files = open_model_files(model_dir)
    entries = {}
    for sf in files:
        entries.update(sf.entries)
    check_entries(entries, expected, where=model_dir)
    by_file = {sf.path: sf for sf in files}
    out: dict[str, torch.Tensor] = {}
    staging = None
    for name, spec in expected.items():
        e = entries[name]
        t = by_file[e.file].tensor(name)
        dtype = resident_dtype(spec, e.dtype, compute)
        if into is not None:
            dst = into[name]
            if dst.dtype != dtype or tuple(dst.shape) != tuple(spec.shape):
                raise ValueError(f"{name}: the place prepared for it is {list(dst.shape)} {dst.dtype}, "
                                 f"it is {list(spec.shape)} {dtype}")
            if dst.is_cuda:
                if staging is None:
                    staging = _Staging(staging_bytes)
                staging.copy(t, dst)
            else:
                dst.copy_(t.to(dtype=dtype))
            out[name] = dst
        elif device is not None:
            out[name] = t.to(device=device, dtype=dtype, non_blocking=False).contiguous()
        else:
            out[name] = t.to(dtype=dtype).contiguous()
    if staging is not None:
        staging.finish()
    return out


def stored_dtypes(model_dir: str) -> dict:
    """name -> dtype as stored, from the headers alone."""
    return {n: e.dtype for sf in open_model_files(model_dir) for n, e in sf.entries.items()}
