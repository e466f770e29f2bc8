"""Rotary position encoding with a per-pair frequency table.

angle = float32(position) * inv_freq[i]; the pair (x0, x1) becomes
(x0 cos - x1 sin, x0 sin + x1 cos) (src/backend/cpu.rs:68-84).  `layout`
chooses which elements pair up: "interleaved" (2i, 2i+1) as the reference's
Llama does, or "split_half" (i, i + rotary_dim/2) as in its split-half
rotation (src/backend/cpu.rs:135-156), which checkpoint folders use.  The
table is theta^(-2i/d) computed once on the host in float64 (the reference
builds it on the host too: src/backend/cuda.rs:383-398); llama3 scaling
divides each frequency by a factor chosen by its wavelength.  Rotated keys are
written straight into the cache, so the encoding is fixed at write time
(src/model/arch/llama.rs:198-209).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..registry import POSITIONS
from .base import Part


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """float32 [rotary_dim/2]."""
    out = []
    for i in range(rotary_dim // 2):
        f = float(theta) ** (-2.0 * i / rotary_dim)
        if scaling is not None:
            wavelength = 2.0 * math.pi / f
            span = float(scaling.original_max_position_embeddings)
            if wavelength < span / scaling.high_freq_factor:
                pass
            elif wavelength > span / scaling.low_freq_factor:
                f = f / scaling.factor
            else:
                s = (span / wavelength - scaling.low_freq_factor) / (
                    scaling.high_freq_factor - scaling.low_freq_factor)
                f = (1.0 - s) * f / scaling.factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


@POSITIONS.register("rotary")
class Rotary(Part):
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        self.interleaved = p.get("layout", "split_half") == "interleaved"
        if p.get("layout", "split_half") not in ("split_half", "interleaved"):
            raise ValueError(f"unknown rotary layout {p['layout']!r}")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.table_host = inverse_frequencies(self.rotary_dim, p["theta"], p.get("scaling"))

    def bind(self, tensors, rt):
        if getattr(self, "rt", None) is rt and getattr(self, "inv_freq", None) is not None:
            return                  # bound by its mixer and again by the model: one table
        super().bind(tensors, rt)
        self.inv_freq = rt.derived(self.table_host)

    fuses_pending = True        # adds up a deferred K-split projection itself

    def resident_tensors(self):
        return []                 # the frequency table is derived, not a weight

    def device_tensors(self):
        return {"inv_freq": ((self.rotary_dim // 2,), torch.float32)}

    def rotary_table(self):
        """(inverse frequencies on the device, rotated width, interleaved?): what a mixer needs to do this
        encoding inside a kernel of its own instead of calling `encode_and_store`."""
        return self.inv_freq, self.rotary_dim, self.interleaved

    def encode_and_store(self, ctx, qkv, n_heads, n_kv_heads, head_dim, view, write_kv):
        partial, splits, stride = None, 0, 0
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            pend = ops_tensor.take_pending(qkv, ops.GEMM_STORE, ctx.n_tokens, self.rt.tc)
            if pend is not None:
                partial, splits, stride = pend
            else:
                ops_tensor.flush_pending(qkv.device, self.rt.tc)
        ops.rope_cache_write(qkv, ctx.n_tokens, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, self.inv_freq,
                             view.k if write_kv else None, view.v if write_kv else None,
                             view.page_table if write_kv else None, view.max_pages, view.page_size,
                             n_heads, n_kv_heads, head_dim, self.rotary_dim, self.interleaved, write_kv,
                             partial, splits, stride)
