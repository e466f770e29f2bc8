"""One device allocation for everything an engine holds.

The reference adds up what a model and a request will need from sizes alone,
reserves that against the budget and only then allocates, and its tests ask
that the bytes reserved equal the bytes held (src/model/planning.rs:55-125,
src/model/memory.rs:158-179, src/model/arch/llama/tests.rs:8-66).  Here the
same function lays the engine's memory out twice: once with a `Carver` that
only adds up (the plan, which needs no device), once with a `Carver` over a
single device buffer of exactly the planned size.  Nothing the engine keeps is
allocated anywhere else, so plan and holdings agree by construction.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

ALIGN = 256          # every region starts on a 256-byte boundary (TMA wants 16, vector loads 16)


def _nbytes(shape, dtype: torch.dtype) -> int:
    return int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()


class Carver:
    """Hands out regions in the order they are asked for.  Without a buffer it only adds up
    (`take` returns None); with one it returns views, at the offsets the planning pass saw."""

    def __init__(self, buffer: Optional[torch.Tensor] = None):
        self.buffer = buffer
        self.offset = 0
        self.by_category: dict[str, int] = {}

    @property
    def planning(self) -> bool:
        return self.buffer is None

    def take(self, category: str, shape, dtype: torch.dtype) -> Optional[torch.Tensor]:
        shape = tuple(int(s) for s in shape)
        n = _nbytes(shape, dtype)
        padded = -(-n // ALIGN) * ALIGN
        start = self.offset
        self.offset += padded
        self.by_category[category] = self.by_category.get(category, 0) + padded
        if self.buffer is None:
            return None
        if self.offset > self.buffer.numel():
            raise RuntimeError(f"the arena of {self.buffer.numel()} bytes is too small for a {category} region "
                               f"of {n} bytes at {start}: plan and layout disagree")
        return self.buffer[start:start + n].view(dtype).view(shape)

    def taker(self, category: str):
        """`alloc(shape, dtype)` for a component that takes all its memory from one category."""
        return lambda shape, dtype: self.take(category, shape, dtype)
