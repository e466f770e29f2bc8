"""Grouped-query causal attention over the cache.

q, k, v = h Wq^T, h Wk^T, h Wv^T (no biases unless `bias` is set); q and k take the position
encoding, k and v go to the cache; a query at position p reads the keys
[first, p] of its own sequence (first = 0, or p+1-window), kv head = q head //
(heads / kv heads), scores (q.k) * scale through a float softmax; the result
times Wo^T is added to the residual stream (src/model/arch/llama.rs:195-212,
src/backend/cpu.rs:530-590).  Heads, groups, head size, scale and window are
parameters.  A site that reads another site's cache has no k/v matrices and
writes nothing.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..cache import KVNeed
from ..registry import MIXERS, POSITIONS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


FUSED_ROTARY = os.environ.get("MDMA_FUSED_ROTARY", "1") != "0"


@MIXERS.register("attention")
class Attention(Part):
    graph_safe = True      # forward reads no host-side per-step values
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = int(p.get("window", 0) or 0)
        self.shared_cache = bool(p.get("shared_cache", False))
        self.bias = bool(p.get("bias", False))              # a vector added after each of the four products
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide over {self.n_kv_heads} kv heads")
        pos = p["position"]
        self.position = POSITIONS.get(pos.kind)(pos)
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.row_width = self.q_width + (0 if self.shared_cache else 2 * self.kv_width)

    def children(self):
        return [self.position]

    def tensor_specs(self):
        specs = {"q_proj.weight": TensorSpec((self.q_width, self.hidden))}
        if not self.shared_cache:
            specs["k_proj.weight"] = TensorSpec((self.kv_width, self.hidden))
            specs["v_proj.weight"] = TensorSpec((self.kv_width, self.hidden))
        specs["o_proj.weight"] = TensorSpec((self.hidden, self.q_width))
        if self.bias:
            for name in [n for n in specs]:
                specs[name[:-len("weight")] + "bias"] = TensorSpec((specs[name].shape[0],), "vector", "normal")
        return specs

    MAX_HEAD_DIM = 256        # the plain attention kernel's limit (csrc/attention_simple.cu)

    def check_limits(self, rt):
        """Sizes no kernel of this library takes are refused when the engine is built, before
        anything is loaded (src/model/arch/llama/preflight.rs:35-42)."""
        if self.head_dim > self.MAX_HEAD_DIM:
            raise ValueError(f"head_dim {self.head_dim} is beyond the attention kernels' limit of {self.MAX_HEAD_DIM}")

    def fused_tensors(self):
        # one product for q, k and v
        if self.shared_cache:
            return {}
        fused = {"qkv_proj.weight": ("q_proj.weight", "k_proj.weight", "v_proj.weight")}
        if self.bias:
            fused["qkv_proj.bias"] = ("q_proj.bias", "k_proj.bias", "v_proj.bias")
        return fused

    def kv_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def state_need(self):
        return None

    def workspace(self):
        return {"qkv": (self.row_width, "act"), "attn_out": (self.q_width, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        if not self.position.tensor_specs():
            self.position.bind({}, rt)      # a position part with tensors of its own is bound by the model
        if self.shared_cache:
            fused = tensors["q_proj.weight"]
        elif "qkv_proj.weight" in tensors:
            fused = tensors["qkv_proj.weight"]        # the loader filled the one matrix (see fused_tensors)
        else:
            # bound by hand with three separate matrices: rows [q heads | k heads | v heads]
            fused = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                               tensors["v_proj.weight"]], dim=0).contiguous()
        fused_bias = None
        if self.bias:
            if self.shared_cache:
                fused_bias = tensors["q_proj.bias"]
            elif "qkv_proj.bias" in tensors:
                fused_bias = tensors["qkv_proj.bias"]
            else:
                fused_bias = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]).contiguous()
        self._fast_ok = False
        if rt.attention == "fast":
            from .. import ops_tensor
            self._fast_ok = ops_tensor.attention_supported(self.n_heads, self.n_kv_heads, self.head_dim)
        self.qkv_proj = Linear(fused, rt, bias=fused_bias)
        self.o_proj = Linear(tensors["o_proj.weight"], rt, bias=tensors.get("o_proj.bias"))

    def forward(self, ctx, h, x, view, owns_cache=True):
        n = ctx.n_tokens
        qkv = ctx.buf("qkv", self.row_width)
        out = ctx.buf("attn_out", self.q_width)
        write = owns_cache and not self.shared_cache
        if write and ctx.max_new == 1 and self._fast_ok and self._fusable(ctx, view):
            # single tokens: the attention kernel rotates q and k and writes the cache itself
            from .. import ops_tensor
            inv_freq, rotary_dim, interleaved = self.position.rotary_table()
            self.qkv_proj.store(h, qkv, n, defer=True)
            ops_tensor.attention_decode_rotary(ctx, qkv, view, out, self.n_heads, self.n_kv_heads, self.head_dim,
                                               self.window, self.scale, inv_freq, rotary_dim, interleaved, st=self.rt.tc)
            self.o_proj.accumulate(out, x, n)
            return
        self.qkv_proj.store(h, qkv, n, defer=getattr(self.position, "fuses_pending", False))
        self.position.encode_and_store(ctx, qkv, self.n_heads, self.n_kv_heads, self.head_dim, view, write)
        if self.rt.attention == "fast" and self._fast_ok:
            from .. import ops_tensor
            ops_tensor.attention(ctx, qkv, view, out, self.n_heads, self.n_kv_heads, self.head_dim,
                                 self.window, self.scale, st=self.rt.tc)
        else:
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(qkv.device, self.rt.tc)
            ops.attention_simple(qkv, n, view.k, view.v, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                                 view.page_table, view.max_pages, view.page_size, out,
                                 self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.scale)
        self.o_proj.accumulate(out, x, n)

    def _fusable(self, ctx, view) -> bool:
        """Whether this step's attention kernel should do the position encoding and the cache write
        itself.  It pays while the kernel's blocks have three warps or more (up to four blocks per SM).  Measured
        at the 8B layer shape, the chain of a layer with and without: batch 8 93.6 against 96.4 us; batch 32
        112.7 against 113.5, batch 64 136.6 against 138.2 (with the QKV product split four ways; with six it was
        the other way round, because every block adds up the projection's partial rows itself); batch 96 173.9
        against 163.3, batch 128 187.9 against 176.6 (blocks of one or two warps).  MDMA_FUSED_ROTARY=0 turns it
        off, for comparisons."""
        if self.rt.attention != "fast" or not hasattr(self.position, "rotary_table") or not FUSED_ROTARY:
            return False
        from .. import ops_tensor
        sms = self.rt.tc.sms if self.rt.tc is not None else 0
        return (ctx.n_seqs * self.n_kv_heads <= 4 * sms and
                ops_tensor.fused_rotary_supported(self.n_heads, self.n_kv_heads, self.head_dim, view.page_size,
                                                  self.position.rotary_table()[1]))

    def resident_tensors(self):
        return [t for t in (self.qkv_proj.w, self.o_proj.w, self.qkv_proj.bias, self.o_proj.bias) if t is not None]
