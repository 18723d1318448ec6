"""Sampling options and seeds.  The choice itself runs on the device
(``csrc/sampling.cu``); this module holds what the host decides.

Option names and meanings follow the reference's request
(crates/esp/src/infer/provider.rs:91-117, crates/esp/src/infer/decoder/provider.rs:484-501):
temperature 0 is greedy, a positive temperature samples, ``top_p`` is an
optional nucleus cut that greedy ignores, ``seed`` makes the stream
reproducible and, when absent, is drawn from the process's entropy.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional

from ..errors import InvalidRequest

_M = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def splitmix64_next(state: int):
    """(new state, output) of one splitmix64 step
    (crates/esp/src/infer/decoder/sample.rs:40-46)."""
    state = (state + GOLDEN) & _M
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return state, z ^ (z >> 31)


def skip_draws(state: int, draws: int) -> int:
    """State after ``draws`` draws, in O(1) (sample.rs:64-69)."""
    return (state + GOLDEN * draws) & _M


def entropy_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


def as_signed64(v: int) -> int:
    """Two's-complement view for storage in an int64 tensor."""
    v &= _M
    return v - (1 << 64) if v >= (1 << 63) else v


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: Optional[float] = None
    seed: Optional[int] = None

    def validate(self) -> None:
        t = self.temperature
        if not isinstance(t, (int, float)) or math.isnan(t) or math.isinf(t) or t < 0:
            raise InvalidRequest(f"temperature must be a finite number >= 0, got {t!r}")
        if self.top_p is not None and (not isinstance(self.top_p, (int, float)) or math.isnan(self.top_p)):
            raise InvalidRequest(f"top_p must be a number, got {self.top_p!r}")
        if self.seed is not None and (not isinstance(self.seed, int) or self.seed < 0 or self.seed > _M):
            raise InvalidRequest("seed must be an integer in [0, 2^64)")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    def resolved_seed(self) -> int:
        """The seed of this request's stream: the given one, or a fresh one."""
        return self.seed if self.seed is not None else entropy_seed()
