"""Gated feed-forward: act = f(h Wg^T) * (h Wu^T); x += act Wd^T, f = SiLU
(src/model/arch/llama.rs:222-230, src/backend/cpu.rs:447-458).  Dense: every
token uses the same three matrices.  The two first products and the
activation run as one kernel.  Parameters beyond the reference's Llama:
`activation` ("silu", "gelu_tanh") and `bias` (a vector added after each of
the three products)."""
from __future__ import annotations

from .. import ops
from ..registry import FEED_FORWARDS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(Part):
    graph_safe = True      # forward reads no host-side per-step values
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.inner = int(self.params["intermediate_size"])
        self.activation = str(self.params.get("activation", "silu"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not implemented (have {sorted(ops.ACTIVATIONS)})")
        self.bias = bool(self.params.get("bias", False))

    def tensor_specs(self):
        specs = {"gate_proj.weight": TensorSpec((self.inner, self.hidden)),
                 "up_proj.weight": TensorSpec((self.inner, self.hidden)),
                 "down_proj.weight": TensorSpec((self.hidden, self.inner))}
        if self.bias:
            specs["gate_proj.bias"] = TensorSpec((self.inner,), "vector", "normal")
            specs["up_proj.bias"] = TensorSpec((self.inner,), "vector", "normal")
            specs["down_proj.bias"] = TensorSpec((self.hidden,), "vector", "normal")
        return specs

    def workspace(self):
        return {"act": (self.inner, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.gate_up = Linear(tensors["gate_proj.weight"], rt, tensors["up_proj.weight"],
                              tensors.get("gate_proj.bias"), tensors.get("up_proj.bias"), self.activation)
        self.down = Linear(tensors["down_proj.weight"], rt, bias=tensors.get("down_proj.bias"))

    def forward(self, ctx, h, x):
        act = ctx.buf("act", self.inner)
        self.gate_up.gated(h, act, ctx.n_tokens)
        self.down.accumulate(act, x, ctx.n_tokens)

    def resident_tensors(self):
        return [t for t in (self.gate_up.w, self.gate_up.w2, self.down.w, self.gate_up.bias, self.gate_up.bias2,
                            self.down.bias) if t is not None]
