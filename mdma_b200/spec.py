"""Declarative description of a model: which parts each layer is made of,
which tensors they read, and the order in which layers run.

An architecture turns its typed configuration into a `ModelSpec`; the engine
builds every part from the registries and never asks which model it is
running.  Sizes and constants live in `PartSpec.params`; tensor names are
`prefix + local name`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs. `kind` is 'matrix' (kept in the compute dtype),
    'vector' (kept as stored: bfloat16 or float32) or 'int' (held as int32).
    `init` says what the seeded random mode puts there: 'normal', 'ones' or 'zeros'
    (by default matrices are normal, vectors ones, integer tables zeros)."""
    shape: tuple
    kind: str = "matrix"
    init: str = ""

    def initial(self) -> str:
        return self.init or {"matrix": "normal", "vector": "ones", "int": "zeros"}[self.kind]


@dataclass
class PartSpec:
    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    prefix: str = ""
    # local tensor name -> full name in the file, for tensors that do not live
    # under `prefix` (a tied output matrix names the embedding's tensor)
    aliases: dict[str, str] = field(default_factory=dict)

    def tensor_name(self, local: str) -> str:
        return self.aliases.get(local, self.prefix + local)


@dataclass
class LayerSpec:
    """One layer's parts. `block` names the arrangement (registry BLOCKS).  An arrangement that has
    more parts than these four (a norm on the queries and keys, norms after the mixer and the
    feed-forward, a second feed-forward) finds them by name in `extras`."""
    block: str
    mixer_norm: PartSpec
    mixer: PartSpec
    ffn_norm: PartSpec
    ffn: PartSpec
    extras: dict[str, PartSpec] = field(default_factory=dict)


@dataclass
class ScheduleEntry:
    """One run of a layer. `cache` names the schedule entry whose cache this run
    reads and writes; None = its own.  An entry that names an earlier entry's
    cache reads it and writes nothing."""
    layer: int
    cache: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: list[LayerSpec]
    schedule: list[ScheduleEntry]
    final_norm: PartSpec
    lm_head: PartSpec
    stop_token_ids: tuple = ()
