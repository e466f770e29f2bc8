"""What every part is: sizes and constants as parameters, the tensors it reads
declared by local name, and a forward that knows nothing about the model it
sits in.

Interfaces (duck-typed; `Part` holds what is common):

  norm          forward(ctx, x_f32 [T,W], out [T,W], rows=None, n_rows=None)
  position      encode_and_store(ctx, qkv, n_heads, n_kv_heads, head_dim, view, write_kv)
  mixer         kv_need() -> KVNeed | None; state_need() -> StateNeed | None;
                forward(ctx, h [T,W], x_f32 [T,W], view: KVView, owns_cache: bool)
                adds its output into x
  feed-forward  forward(ctx, h [T,W], x_f32 [T,W]); adds its output into x
  block         forward(ctx, x_f32, view, owns_cache); runs norms, mixer, feed-forward

`ctx` is the step context: batch metadata on the device (ids, tok_seq, tok_pos,
seq_slot, seq_start, n_tokens, n_seqs, max_new, max_len), `buf(name, cols,
dtype)` for workspace, and `rt`, the runtime (compute dtype, device, kernel
choices).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..spec import PartSpec, TensorSpec


@dataclass
class Runtime:
    """Where and how parts compute."""
    dtype: torch.dtype                 # activations, matrices, cache: bfloat16 or float32
    device: torch.device
    gemm: str = "simt"                 # "simt" | "tensor" (tcgen05; bfloat16 only)
    attention: str = "simple"          # "simple" | "fast"
    tc: object = None                  # the engine's `ops_tensor.TensorState` (None: a shared default)
    alloc: object = None               # alloc(shape, dtype) for the device tensors a part derives at bind

    def derived(self, host: torch.Tensor) -> torch.Tensor:
        """A device copy of a small tensor a part computed on the host (a table of frequencies):
        taken from the engine's arena when there is one (the part then names it in `device_tensors`)."""
        if self.alloc is None:
            return host.to(self.device)
        dev = self.alloc(tuple(host.shape), host.dtype)
        dev.copy_(host)
        return dev


class Part:
    """Base: keeps the spec, declares tensors, takes them when bound."""

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params = spec.params

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def children(self) -> list["Part"]:
        return []

    def workspace(self) -> dict[str, tuple[int, str]]:
        """Per-token workspace this part asks for: name -> (columns, 'act' | 'f32')."""
        return {}

    def fused_tensors(self) -> dict[str, tuple]:
        """Tensors this part wants stored as consecutive rows of one matrix, in this order:
        {name of the whole: (local names...)}.  The loader then fills the one matrix and `bind`
        gets the whole under its name next to the pieces (views of its rows)."""
        return {}

    def device_tensors(self) -> dict[str, tuple]:
        """Device tensors this part makes itself at bind, beyond its weights: name -> (shape, dtype).
        The engine counts them in its memory plan; the part gets them through `rt.derived`."""
        return {}

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        """Take the device tensors named in tensor_specs()."""
        self.rt = rt

    def resident_tensors(self) -> list:
        """The device tensors this part holds (for the memory account)."""
        return []
