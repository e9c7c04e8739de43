"""Arrangement of a layer's parts.

``pre_norm`` is the reference's block (models/transformer_block.py:149-158):
``x = x + mixer(norm1(x))``, ``x = x + ffn(norm2(x))``.  The sums are formed in the
32-bit residual stream by the norm kernels: a sub-layer's output waits in
``stream.delta`` and the next norm adds it while normalising.
"""
from __future__ import annotations

from .base import Block, PartSpec, ResidualStream, StepContext, mixer_cache_argument
from ..registry import register_part, build_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, prefix: str, mixer_norm: PartSpec, mixer: PartSpec, ffn_norm: PartSpec, ffn: PartSpec):
        super().__init__(prefix)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer = build_part("mixer", mixer)
        self.ffn_norm = build_part("norm", ffn_norm)
        self.ffn = build_part("ffn", ffn)

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def cache_needs(self):
        return self.mixer.cache_needs()                            # the feed-forward parts here keep nothing between steps

    def forward(self, stream: ResidualStream, ctx: StepContext, caches) -> None:
        h = self.mixer_norm.add_norm(stream.resid, stream.delta)
        a = self.mixer.forward(h, ctx, mixer_cache_argument(self.mixer, caches))
        h = self.ffn_norm.add_norm(stream.resid, a)
        stream.delta = self.ffn.forward(h, ctx)
