"""Sampling options, with the reference's names, meanings and defaults
(include/sampler.h:12-20, src/sampler.c:8-18; command-line flags src/main.c:951-964)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Tuple


@dataclass(frozen=True)
class SamplingParams:
    temp: float = 0.0              # <= 0: greedy (first maximum); > 0: stochastic
    top_k: int = 0                 # keep the k best (0: off)
    top_p: float = 1.0             # nucleus (1.0: off)
    min_p: float = 0.0             # drop tokens below min_p * p_max (0: off)
    repeat_penalty: float = 1.0    # > 1 penalises the recent tokens (1.0: off)
    repeat_last_n: int = 64        # how many recent tokens the penalty sees
    seed: int = 0                  # 0: taken from the clock when the request is added
    max_new_tokens: int = 128      # the command line's -n
    stop_token_ids: Tuple[int, ...] = field(default=())   # generation ends after one of these (none by default:
                                                          # the reference's LFM path always runs -n tokens)

    def __post_init__(self):
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        if self.top_k < 0 or self.repeat_last_n < 0:
            raise ValueError("top_k and repeat_last_n must not be negative")
        if not (self.top_p > 0.0 and self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if not (0.0 <= self.min_p < 1.0):
            raise ValueError("min_p must be in [0, 1)")

    @property
    def greedy(self) -> bool:
        return not self.temp > 0.0
