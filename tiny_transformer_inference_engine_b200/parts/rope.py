"""Rotary position encoding.

Reference formula (models/rope.py:14-35): ``inv_freq[j] = 1 / base**(2j/dim)`` for
``j < dim/2`` (32-bit), ``theta = pos * inv_freq[j]`` (32-bit), and the rotation of
**interleaved pairs**: ``out[2j] = x[2j]*cos - x[2j+1]*sin``,
``out[2j+1] = x[2j]*sin + x[2j+1]*cos``.  The reference's CUDA rope kernel rotates
half-split pairs ``(j, j+dim/2)`` instead (kernels/rope_kernel/rope_kernel.cu:133-157);
its serving path and its golden generation use the interleaved form, which is the
default here, and ``style="half"`` gives the other.  The base is fixed in the
reference (models/rope.py:6); here it is this part's parameter.

``inv_freq`` is built once with the reference's own expression so that the angle
``float(pos) * inv_freq[j]`` has the very same 32-bit rounding; the kernels take
sine and cosine of that product in 32-bit.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding
from ..registry import register_part

ROTARY_STYLES = {"interleaved": 0, "half": 1}


@register_part("position", "rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, prefix: str, dim: int, base: float, style: str = "interleaved"):
        super().__init__(prefix)
        if dim % 2:
            raise ValueError(f"rotary dimension {dim} must be even (models/rope.py:8)")
        if style not in ROTARY_STYLES:
            raise ValueError(f"unknown rotary style {style!r}; known: {sorted(ROTARY_STYLES)}")
        self.dim, self.base, self.style = int(dim), float(base), style
        self._inv_freq = None

    def bind(self, ops, dtype, device):
        super().bind(ops, dtype, device)
        inv_freq = 1.0 / (self.base ** (torch.arange(0, self.dim, 2).float() / self.dim))
        self._inv_freq = inv_freq.to(device=device, dtype=torch.float32).contiguous()

    def rotary_table(self):
        return self._inv_freq, ROTARY_STYLES[self.style]

    def step_table(self, ctx):
        """cos/sin of every token of the step, computed once per step and shared by all layers whose
        encoding has the same dimension and base (kept in the step's context)."""
        if not hasattr(self.ops, "rope_table"):
            return None
        tables = ctx.step_cache
        key = ("rope_table", self.dim, self.base)
        if key not in tables:
            tables[key] = self.ops.rope_table(ctx.positions, self._inv_freq)
        return tables[key]

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary encoding runs inside the fused rotate-and-store kernel")


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No position encoding: keys and queries are stored and used as projected."""

    def __init__(self, prefix: str = ""):
        super().__init__(prefix)

    def rotary_table(self):
        return None, 0

    def step_table(self, ctx):
        return None

    def apply(self, q, k, positions):
        return None
