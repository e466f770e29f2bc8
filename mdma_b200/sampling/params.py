"""Sampling options, with the reference sampler's names, defaults and meanings
(src/sampler.rs:5-23): temperature (<= 0 means argmax), top_p, min_p,
repetition_penalty (a positive logit is divided, another multiplied),
repetition_window (how many last tokens of prompt + output are penalised).
`greedy()` is the reference client's MDMA_GREEDY preset
(src/bin/mdma-client/sampling.rs:8-17).  Randomness is always explicit: a seed,
from which each (request, step) gets its own uniform number, so a request's
tokens do not depend on what else is in its batch."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8
    top_p: float = 0.95
    min_p: float = 0.05
    repetition_penalty: float = 1.1
    repetition_window: int = 64
    seed: int = 0

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0, top_p=1.0, min_p=0.0, repetition_penalty=1.0, repetition_window=0)

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 and (self.repetition_penalty == 1.0 or self.repetition_window == 0)

    def validate(self) -> None:
        if not self.repetition_penalty > 0:
            raise ValueError("repetition_penalty must be positive")
        if self.repetition_window < 0:
            raise ValueError("repetition_window must not be negative")
        if not 0.0 < self.top_p:
            raise ValueError("top_p must be positive")
        if self.min_p < 0.0:
            raise ValueError("min_p must not be negative")


_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, request: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits for (seed, request, step)."""
    z = _mix(_mix(_mix(seed & _MASK) ^ (request & _MASK)) ^ (step & _MASK))
    return (z >> 40) / float(1 << 24)
