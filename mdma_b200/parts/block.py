"""How a layer's parts are arranged.  "prenorm": x += mixer(norm(x)); x +=
feed_forward(norm(x)), the residual stream x kept in float
(src/model/arch/llama.rs:181-231)."""
from __future__ import annotations

from ..registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from ..spec import LayerSpec


@BLOCKS.register("prenorm")
class PreNormBlock:
    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer)
        self.ffn_norm = NORMS.get(spec.ffn_norm.kind)(spec.ffn_norm)
        self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn)

    handles_pending = True      # completes x itself where a product left partial sums (see _settle)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def workspace(self):
        """Per-token workspace of the arrangement itself: name -> (columns, 'act' | 'f32')."""
        return {"normed": (int(self.mixer_norm.params["width"]), "act")}

    def forward(self, ctx, x, view, owns_cache=True):
        h = ctx.buf("normed", x.shape[1])
        self._settle(ctx, x, self.mixer_norm)
        self.mixer_norm.forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, view, owns_cache)
        self._settle(ctx, x, self.ffn_norm)
        self.ffn_norm.forward(ctx, x, h)
        self.ffn.forward(ctx, h, x)

    @staticmethod
    def _settle(ctx, x, norm):
        """A matrix product may have left partial sums of x for the next norm to add up;
        a norm that does not do that gets x completed first."""
        if ctx.rt.gemm == "tensor" and not getattr(norm, "fuses_pending", False):
            from .. import ops_tensor
            ops_tensor.flush_pending(x.device, ctx.rt.tc)
