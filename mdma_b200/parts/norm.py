"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w (src/backend/cpu.rs:388-401;
no +1 on the weight, no mean subtraction).  Reads the float residual stream,
writes the compute dtype; sums in float."""
from __future__ import annotations

from .. import ops
from ..registry import NORMS
from ..spec import TensorSpec
from .base import Part


@NORMS.register("rmsnorm")
class RMSNorm(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.eps = float(self.params["eps"])

    def tensor_specs(self):
        return {"weight": TensorSpec((self.width,), "vector")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    fuses_pending = True        # adds up a deferred K-split product on x itself

    def forward(self, ctx, x, out, rows=None, n_rows=None):
        n = n_rows if n_rows is not None else (None if rows is not None else ctx.n_tokens)
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            pend = ops_tensor.take_pending(x, ops.GEMM_ACCUMULATE, ctx.n_tokens, self.rt.tc) if rows is None else None
            if pend is not None:
                scratch, splits, stride = pend
                ops.rmsnorm(x, self.weight, self.eps, out, None, n, scratch, splits, stride)
                return
            ops_tensor.flush_pending(x.device, self.rt.tc)
        ops.rmsnorm(x, self.weight, self.eps, out, rows, n)

    def resident_tensors(self):
        return [self.weight]
