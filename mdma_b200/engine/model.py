"""A decoder assembled from a `ModelSpec`: embedding, blocks run in the order
the schedule gives, a final norm over the wanted rows and the output head.
Nothing here names an architecture; the parts come from the registries."""
from __future__ import annotations

from typing import Optional

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..cache import KVNeed, SequenceCache, StateNeed
from ..parts.base import Part, Runtime
from ..registry import BLOCKS, EMBEDDINGS, HEADS, NORMS
from ..spec import ModelSpec, TensorSpec


def _walk(part: Part):
    yield part
    for child in part.children():
        yield from _walk(child)


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding)
        self.blocks = [BLOCKS.get(layer.block)(layer) for layer in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm)
        self.head = HEADS.get(spec.lm_head.kind)(spec.lm_head)
        for n, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {n} names layer {entry.layer}, there are {len(self.blocks)}")
            if entry.cache is not None:
                if not 0 <= entry.cache < n or spec.schedule[entry.cache].cache is not None:
                    raise ValueError(f"schedule entry {n} must read the cache of an earlier entry that owns one")

    # ---- inventory -----------------------------------------------------
    def all_parts(self) -> list[Part]:
        tops = [self.embedding, self.final_norm, self.head]
        for b in self.blocks:
            tops.extend(b.parts())
        return [p for top in tops for p in _walk(top)]

    def expected_tensors(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        for part in self.all_parts():
            for local, ts in part.tensor_specs().items():
                name = part.spec.tensor_name(local)
                if name in out and out[name] != ts:
                    raise ValueError(f"tensor {name} is declared twice with different shapes")
                out[name] = ts
        return out

    def kv_needs(self) -> list[Optional[KVNeed]]:
        """Per schedule entry: the storage it owns (None if it reads another entry's or keeps none)."""
        needs = []
        for entry in self.spec.schedule:
            mixer = self.blocks[entry.layer].mixer
            needs.append(mixer.kv_need() if entry.cache is None else None)
        return needs

    def state_needs(self) -> list[Optional[StateNeed]]:
        return [self.blocks[e.layer].mixer.state_need() for e in self.spec.schedule]

    def workspace_columns(self) -> dict[str, tuple[int, str]]:
        cols: dict[str, tuple[int, str]] = {"x": (self.spec.hidden_size, "f32"),
                                             "normed": (self.spec.hidden_size, "act"),
                                             "h_rows": (self.spec.hidden_size, "act")}
        for part in self.all_parts():
            for name, (c, kind) in part.workspace().items():
                old = cols.get(name)
                if old is not None and old[1] != kind:
                    raise ValueError(f"workspace buffer {name!r} is asked for as {old[1]} and {kind}")
                cols[name] = (max(c, old[0]) if old else c, kind)
        return cols

    # ---- weights ---------------------------------------------------------
    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        for part in self.all_parts():
            local = {l: tensors[part.spec.tensor_name(l)] for l in part.tensor_specs()}
            part.bind(local, rt)

    def resident_bytes(self) -> int:
        """Bytes of weights on the device; a tensor shared by two parts (a tied head) counts once."""
        seen, total = set(), 0
        for part in self.all_parts():
            for t in part.resident_tensors():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # ---- forward ---------------------------------------------------------
    def forward(self, ctx, cache: SequenceCache, logits: Optional[torch.Tensor]) -> None:
        """Run the tokens of `ctx` through every scheduled layer, from the cache
        and into it; write logits of ctx.want_rows into `logits` [n_want, vocab]."""
        x = ctx.buf("x", self.spec.hidden_size, torch.float32)
        self.embedding.forward(ctx, ctx.ids, x)
        for n, entry in enumerate(self.spec.schedule):
            site = n if entry.cache is None else entry.cache
            self.blocks[entry.layer].forward(ctx, x, cache.view(site, state_site=n),
                                             owns_cache=entry.cache is None)
        if ctx.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(x.device)
        if ctx.n_want:
            h = ctx.buf("h_rows", self.spec.hidden_size)
            self.final_norm.forward(ctx, x, h, rows=ctx.want_rows, n_rows=ctx.n_want)
            self.head.forward(ctx, h, logits, ctx.n_want)


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    return DecoderModel(spec).expected_tensors()
