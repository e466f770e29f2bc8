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

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def forward(self, ctx, x, view, owns_cache=True):
        h = ctx.buf("normed", x.shape[1])
        self.mixer_norm.forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, view, owns_cache)
        self.ffn_norm.forward(ctx, x, h)
        self.ffn.forward(ctx, h, x)
