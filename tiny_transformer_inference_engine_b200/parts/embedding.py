"""Token embedding and output head.

Embedding (models/embedding.py:9-15): a row gather, no scale, no position term; the
gathered row starts the 32-bit residual sum.  Head (models/transformer_block.py:170,181):
``logits = x @ W.T`` without bias, untied from the embedding; logits leave in 32-bit.
"""
from __future__ import annotations

import torch

from .base import Embedding, Head, ParamSpec, StepContext
from ..registry import register_part


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    def __init__(self, prefix: str, vocab_size: int, dim: int, name: str = "weight"):
        super().__init__(prefix)
        self.vocab_size, self.dim, self.name = int(vocab_size), int(dim), name
        self.table = None

    def param_specs(self):
        return {self.name: ParamSpec((self.vocab_size, self.dim))}

    def load(self, params):
        self.table = params[self.name].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        resid = torch.empty((ctx.num_tokens, self.dim), dtype=torch.float32, device=ctx.device)
        self.ops.embed(ctx.token_ids, self.table, resid)
        return resid


@register_part("head", "linear")
class LinearHead(Head):
    def __init__(self, prefix: str, dim: int, vocab_size: int):
        super().__init__(prefix)
        self.dim, self.vocab_size = int(dim), int(vocab_size)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.dim))}

    def load(self, params):
        self.weight = params["weight"].contiguous()

    def product_weights(self):
        return [self.weight]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.ops.linear(x, self.weight, None, out_dtype=torch.float32)
