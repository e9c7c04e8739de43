"""Per-request sampling options.

Names, meanings and checks are the reference's ``sample(logits, temperature, top_k,
top_p)`` (sampling.py:95-137): temperature finite and > 0, ``top_k >= 0`` (0 = off),
``0 < top_p <= 1`` (1 = off), applied in the order temperature, top-k, top-p, softmax,
draw.  ``greedy`` (sampling.py:5-6) is argmax; ``temperature == 0`` selects it too.
Each request draws from its own counter-based generator (seed, number of tokens drawn
so far), so what it samples does not depend on which requests share its batch; the
reference draws from the global generator (sampling.py:132).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 100              # inference.py:226  --tokens
    temperature: float = 1.0               # inference.py:227
    top_k: int = 0                         # inference.py:228
    top_p: float = 1.0                     # inference.py:229
    greedy: bool = False
    seed: int = 0
    ignore_eos: bool = False

    def __post_init__(self):
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")                  # inference.py:126-127
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise ValueError("temperature must be finite and > 0 (0 selects greedy)")
        if self.temperature == 0:
            object.__setattr__(self, "greedy", True)
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")                           # sampling.py:106-107
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")                      # sampling.py:108-109

    @property
    def is_greedy(self) -> bool:
        return self.greedy
