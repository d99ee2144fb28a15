"""How the next token is picked from a row of logits.

The reference picks the largest logit, always (src/minimax.rs:373-376); a
temperature of 0 is that.  A temperature above 0 samples softmax(logits / T) by
inverse CDF with one uniform number per token (see :mod:`.uniform`), optionally
among the ``top_k`` largest logits and the smallest set of them that holds
``top_p`` of the probability; logits equal to the last one that stays stay too.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0
    top_k: int = 0              # 0: no limit
    top_p: float = 1.0          # 1: no limit

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"a temperature of {self.temperature} is below 0")
        if self.top_k < 0:
            raise ValueError(f"a top_k of {self.top_k} is below 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"a top_p of {self.top_p} is outside (0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
