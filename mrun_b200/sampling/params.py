"""Sampling settings of one request, with the reference's names, meanings and refusals
(crates/mrun-engine/src/engine.rs:326-375).  Temperature 0 means greedy."""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: Optional[int] = None
    repetition_penalty: float = 1.0

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    def validate(self) -> None:
        """Raises ValueError for values that would give NaN logits or an empty candidate set."""
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError(f"temperature must be 0 or more, got {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be 0 or more, got {self.top_k}")
        if not (math.isfinite(self.repetition_penalty) and self.repetition_penalty > 0.0):
            raise ValueError(f"repetition_penalty must be more than 0, got {self.repetition_penalty}")
        if self.seed is not None and not 0 <= self.seed <= _MASK:
            raise ValueError(f"seed must fit in 64 bits, got {self.seed}")


GREEDY = SamplingParams()

# How many of the most recent token ids (prompt and generated) the repetition penalty looks at
# (crates/mrun-engine/src/sample.rs:19-21).
REPETITION_CONTEXT = 20


def mix64(z: int) -> int:
    z = (z + _GOLDEN) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def draw_key(seed: int, draw: int) -> int:
    """Key of a request's ``draw``-th sampled token (counted from 1): the reference's
    ``seed * 0x9E3779B97F4A7C15 + n`` (crates/mrun-engine/src/nuvec_engine.rs:224-231), mixed."""
    return mix64((seed * _GOLDEN + draw) & _MASK)


def fresh_seed() -> int:
    """An unseeded request draws a seed of its own (the reference uses the clock)."""
    return int.from_bytes(os.urandom(8), "little")
