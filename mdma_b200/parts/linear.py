"""Matrix products of the parts: y = a @ W.T (+ b), with the three endings the
model needs (store, add into the float residual stream, act(gate) * up of two
products).  Chooses the tensor-core kernel when the runtime asks for it and
the shape allows, else the CUDA-core kernel; both are this library's own."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, rt: Runtime, weight2: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None, bias2: Optional[torch.Tensor] = None,
                 activation: str = "silu"):
        self.w, self.w2, self.rt = weight, weight2, rt
        self.bias, self.bias2 = bias, bias2
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not implemented (have {sorted(ops.ACTIVATIONS)})")
        self.act = ops.ACTIVATIONS[activation]
        self.out_features, self.in_features = weight.shape
        self._tensor_ok = False
        if rt.gemm == "tensor" and weight.dtype == torch.bfloat16:
            from .. import ops_tensor
            self._tensor_ok = ops_tensor.gemm_supported(self.out_features, self.in_features)

    def _run(self, mode: int, a: torch.Tensor, out: torch.Tensor, m: int, defer: bool = False) -> None:
        if self._tensor_ok:
            from .. import ops_tensor
            ops_tensor.gemm(a, self.w, out, mode, self.w2, m, defer=defer, st=self.rt.tc,
                            bias=self.bias, bias2=self.bias2, act=self.act)
        else:
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(a.device, self.rt.tc)
            ops.gemm_simt(a, self.w, out, mode, self.w2, m, self.bias, self.bias2, self.act)

    def store(self, a, out, m, defer: bool = False):
        """out = a W^T.  `defer`: a K-split product may leave its partial sums for the
        next kernel to add up (the caller promises that kernel asks for them)."""
        self._run(ops.GEMM_STORE, a, out, m, defer)

    def accumulate(self, a, x, m, defer: bool = True):
        """x += a W^T.  Deferred by default: the norm that reads x next adds the partial sums."""
        self._run(ops.GEMM_ACCUMULATE, a, x, m, defer)

    def gated(self, a, out, m):
        """out = act(a W^T) * (a W2^T)."""
        self._run(ops.GEMM_SWIGLU, a, out, m)

