"""Token embedding (x[t,:] = table[ids[t],:], src/backend/cpu.rs:370-384) and
the output head (logits = h W^T over the wanted rows only,
src/model.rs:370-373, 462-467).  A tied head names the embedding's tensor."""
from __future__ import annotations

from .. import ops
from ..registry import EMBEDDINGS, HEADS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


@EMBEDDINGS.register("embedding")
class Embedding(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab, self.width = int(self.params["vocab_size"]), int(self.params["width"])

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab, self.width))}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"]

    def forward(self, ctx, ids, x):
        ops.embed_rows(self.weight, ids, x)

    def resident_tensors(self):
        return [self.weight]


@HEADS.register("lm_head")
class LMHead(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab, self.width = int(self.params["vocab_size"]), int(self.params["width"])

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab, self.width))}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.proj = Linear(tensors["weight"], rt)

    def forward(self, ctx, h_rows, logits, n_rows):
        self.proj.store(h_rows, logits, n_rows)

    def resident_tensors(self):
        return [self.proj.w]
