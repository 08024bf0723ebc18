"""Sampling options and the seeds of the draws.

Names, defaults and meanings follow maeddesg/ROCmForge: ``temperature`` divides the logits
(clamped to >= 1e-6, src/cpu/sampler.rs:27), ``top_p`` is the nucleus threshold (:41-59),
``top_k`` exists as a function without a flag (:76-177); temperature 0 selects greedy
decoding (src/cli/chat.rs:483).  The seed starts at 0xdeadbeef and grows by one before
every draw (src/main.rs:739,747,979); a request of a batch walks its own sequence of
seeds so that its draws do not depend on its neighbours.
"""
from __future__ import annotations

from dataclasses import dataclass

MASK64 = (1 << 64) - 1
DEFAULT_SEED = 0xDEADBEEF
REQUEST_STRIDE = 0x9E3779B97F4A7C15


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = DEFAULT_SEED

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must lie in [0, 1]")       # src/cli/chat.rs:195-197
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0 switches it off)")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


def draw_seed(seed: int, request: int, draw: int) -> int:
    """Seed of the ``draw``-th draw (from 0) of request ``request``."""
    return (seed + 1 + draw + request * REQUEST_STRIDE) & MASK64


def as_int64(u: int) -> int:
    """The same 64 bits as a signed integer (torch has no uint64 arithmetic)."""
    return u - (1 << 64) if u >= (1 << 63) else u
