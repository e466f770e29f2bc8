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

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        """Take the device tensors named in tensor_specs()."""
        self.rt = rt

    def resident_tensors(self) -> list:
        """The device tensors this part holds (for the memory account)."""
        return []
