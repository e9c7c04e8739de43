"""Device-side sampling with per-request state.

One row of an int32 table per state slot holds a request's sampler: seed (two words),
number of draws so far, top-k, and the bit patterns of temperature and top-p.  The
sampling kernel reads the row of each request by its slot id, applies the reference's
order (temperature, top-k threshold, top-p, softmax, draw; sampling.py:110-135), writes
the token and advances the draw counter, so one launch samples every row of a step and
one device-to-host copy brings the tokens back.
"""
from __future__ import annotations

import struct

import torch

from .params import SamplingParams

STATE_WORDS = 8        # seed_lo, seed_hi, draws, top_k, temperature bits, top_p bits, greedy, pad


def _f32_bits(x: float) -> int:
    return struct.unpack("<i", struct.pack("<f", float(x)))[0]


def _i32(x: int) -> int:
    x &= 0xFFFFFFFF
    return x - (1 << 32) if x >= (1 << 31) else x


class Sampler:
    def __init__(self, ops, max_slots: int, vocab_size: int, device):
        self.ops, self.vocab_size = ops, vocab_size
        self.device = torch.device(device)
        self.state = torch.zeros((max_slots, STATE_WORDS), dtype=torch.int32, device=self.device)

    def set_request(self, slot: int, params: SamplingParams, draws_so_far: int = 0) -> None:
        row = torch.tensor([_i32(params.seed), _i32(params.seed >> 32), int(draws_so_far), int(params.top_k),
                            _f32_bits(params.temperature if not params.is_greedy else 1.0),
                            _f32_bits(params.top_p), 1 if params.is_greedy else 0, 0], dtype=torch.int32)
        self.state[slot].copy_(row, non_blocking=False)

    def sample(self, logits: torch.Tensor, slot_ids: torch.Tensor) -> torch.Tensor:
        """logits float32 [R, V]; slot_ids int32 [R] -> int32 tokens [R] (device)."""
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        if logits.shape[0]:
            self.ops.sample(logits, slot_ids, self.state, out)
        return out
