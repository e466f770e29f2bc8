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
        # the model's own: the residual stream and the normed rows the head reads; the rest is asked for by
        # the block arrangements and the parts
        cols: dict[str, tuple[int, str]] = {"x": (self.spec.hidden_size, "f32"),
                                             "h_rows": (self.spec.hidden_size, "act")}
        askers = [b for b in self.blocks if hasattr(b, "workspace")] + self.all_parts()
        for part in askers:
            for name, (c, kind) in part.workspace().items():
                old = cols.get(name)
                if old is not None and old[1] != kind:
                    raise ValueError(f"workspace buffer {name!r} is asked for as {old[1]} and {kind}")
                cols[name] = (max(c, old[0]) if old else c, kind)
        return cols

    def device_tensor_bytes(self, align: int = 256) -> int:
        """Bytes of the device tensors the parts derive at bind (each rounded up to `align`)."""
        total = 0
        for part in self.all_parts():
            for shape, dtype in part.device_tensors().values():
                n = 1
                for d in shape:
                    n *= int(d)
                total += -(-n * torch.empty((), dtype=dtype).element_size() // align) * align
        return total

    # ---- weights ---------------------------------------------------------
    def lay_out_weights(self, expected: dict[str, TensorSpec], held_dtype, take) -> dict:
        """Where every tensor lives: `take(shape, dtype)` hands out (zeroed) device memory, or None
        when only sizes are wanted.  Tensors that a part wants as rows of one matrix (`fused_tensors`)
        (or as pieces of one vector) get one region, the pieces are views of its rows; the whole is returned
        under its own name.
        `held_dtype(name, spec)` is the dtype a tensor is kept in."""
        tensors: dict = {}
        for part in self.all_parts():
            for whole, locals_ in part.fused_tensors().items():
                whole_name = part.spec.tensor_name(whole)
                names = [part.spec.tensor_name(l) for l in locals_]
                if whole_name in tensors or any(n in tensors for n in names):
                    continue          # placed already (a part that runs at two places of the schedule)
                specs = [expected[n] for n in names]
                dtypes = {held_dtype(n, s) for n, s in zip(names, specs)}
                if (len(specs[0].shape) not in (1, 2) or any(tuple(s.shape[1:]) != tuple(specs[0].shape[1:]) for s in specs)
                        or len(dtypes) != 1):
                    raise ValueError(f"{whole_name}: only matrices of one width (or vectors) of one dtype can be "
                                     f"laid out as one")
                rows = sum(s.shape[0] for s in specs)
                t = take((rows,) + tuple(specs[0].shape[1:]), dtypes.pop())
                tensors[whole_name] = t
                r = 0
                for n, sp in zip(names, specs):
                    tensors[n] = None if t is None else t[r:r + sp.shape[0]]
                    r += sp.shape[0]
        for name, ts in expected.items():
            if name not in tensors:
                tensors[name] = take(ts.shape, held_dtype(name, ts))
        return tensors

    def bind(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        for part in self.all_parts():
            local = {l: tensors[part.spec.tensor_name(l)] for l in part.tensor_specs()}
            for whole in part.fused_tensors():
                if part.spec.tensor_name(whole) in tensors:
                    local[whole] = tensors[part.spec.tensor_name(whole)]
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
            block = self.blocks[entry.layer]
            if ctx.rt.gemm == "tensor" and not getattr(block, "handles_pending", False):
                # a product of the block before may have left partial sums of x for a norm to add up; an
                # arrangement that does not know of that gets x complete
                from .. import ops_tensor
                ops_tensor.flush_pending(x.device, ctx.rt.tc)
            block.forward(ctx, x, cache.view(site, state_site=n), owns_cache=entry.cache is None)
        if ctx.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(x.device, ctx.rt.tc)
        if logits is not None and ctx.n_want:
            self.logits_of(ctx, ctx.want_rows, ctx.n_want, logits)

    def logits_of(self, ctx, rows: torch.Tensor, n_rows: int, logits: torch.Tensor) -> None:
        """After `forward`: logits [n_rows, vocab] of the pass's rows `rows` (device indices)."""
        x = ctx.buf("x", self.spec.hidden_size, torch.float32)
        h = ctx.buf("h_rows", self.spec.hidden_size)
        self.final_norm.forward(ctx, x, h, rows=rows, n_rows=n_rows)
        self.head.forward(ctx, h, logits, n_rows)


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    return DecoderModel(spec).expected_tensors()
