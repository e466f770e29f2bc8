"""Gated feed-forward: act = silu(h Wg^T) * (h Wu^T); x += act Wd^T
(src/model/arch/llama.rs:222-230, src/backend/cpu.rs:447-458).  Dense: every
token uses the same three matrices.  The two first products and the
activation run as one kernel."""
from __future__ import annotations

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
        if self.params.get("activation", "silu") != "silu":
            raise ValueError(f"activation {self.params['activation']!r} is not implemented (only 'silu')")

    def tensor_specs(self):
        return {"gate_proj.weight": TensorSpec((self.inner, self.hidden)),
                "up_proj.weight": TensorSpec((self.inner, self.hidden)),
                "down_proj.weight": TensorSpec((self.hidden, self.inner))}

    def workspace(self):
        return {"act": (self.inner, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.gate_up = Linear(tensors["gate_proj.weight"], rt, tensors["up_proj.weight"])
        self.down = Linear(tensors["down_proj.weight"], rt)

    def forward(self, ctx, h, x):
        act = ctx.buf("act", self.inner)
        self.gate_up.swiglu(h, act, ctx.n_tokens)
        self.down.accumulate(act, x, ctx.n_tokens)

    def resident_tensors(self):
        return [self.gate_up.w, self.gate_up.w2, self.down.w]
