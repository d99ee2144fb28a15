"""How the next token is picked from a row of logits.

The reference picks the largest logit, always (src/minimax.rs:373-376); a
temperature of 0 is that.  A temperature above 0 samples softmax(logits / T) by
inverse CDF with one uniform number per token (see :mod:`.uniform`).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"a temperature of {self.temperature} is below 0")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
