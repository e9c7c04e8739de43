"""A model built from a ``ModelSpec``: parts, their tensors, and the run order.

This class is the same for every architecture.  It builds the parts through the
registry, tells the weight loader which tensors exist, tells the cache manager what
each run entry needs, and runs one step: embedding, the run entries in order, final
norm at the wanted rows, head.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import (ModelSpec, ParamSpec, Part, ResidualStream, StepContext, PagedKVNeed, FixedStateNeed)
from ..registry import build_part


def _walk(part: Part):
    yield part
    for c in part.children():
        yield from _walk(c)


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.blocks = [build_part("block", layer.block) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.run_order = list(spec.run_order)
        for e, entry in enumerate(self.run_order):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"run entry {e} names layer {entry.layer}; the model has {len(self.blocks)}")
            if entry.cache_from is not None and not 0 <= entry.cache_from < e:
                raise ValueError(f"run entry {e} reads the cache of entry {entry.cache_from}, which is not earlier")
            if entry.cache_from is not None and self.run_order[entry.cache_from].cache_from is not None:
                raise ValueError(f"run entry {e} reads the cache of entry {entry.cache_from}, which owns none")

    # ---------------------------------------------------------------- tensors
    def parts(self) -> List[Part]:
        tops = [self.embedding, *self.blocks, self.final_norm, self.head]
        return [p for top in tops for p in _walk(top)]

    def param_specs(self) -> Dict[str, Tuple[Part, str, ParamSpec]]:
        """Full tensor name -> (owning part, relative name, spec)."""
        out = {}
        for part in self.parts():
            for rel, ps in part.param_specs().items():
                full = f"{part.prefix}.{rel}" if part.prefix else rel
                if full in out:
                    raise ValueError(f"two parts claim tensor {full!r}")
                out[full] = (part, rel, ps)
        return out

    def bind(self, ops, dtype: torch.dtype, device) -> None:
        self.ops, self.dtype, self.device = ops, dtype, torch.device(device)
        for top in [self.embedding, *self.blocks, self.final_norm, self.head]:
            top.bind(ops, dtype, self.device)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        per_part: Dict[int, Dict[str, torch.Tensor]] = {}
        owners = {}
        for full, (part, rel, _) in self.param_specs().items():
            per_part.setdefault(id(part), {})[rel] = tensors[full]
            owners[id(part)] = part
        for pid, params in per_part.items():
            owners[pid].load(params)
        tune = getattr(getattr(self, "ops", None), "tune_products", None)
        if tune is not None:                                       # the kernel library may measure which product suits each shape
            tune([w for p in self.parts() for w in p.product_weights() if w is not None])

    # ---------------------------------------------------------------- cache
    def cache_needs(self) -> List[List[object]]:
        """What each run entry needs of the cache manager: the list its block reports (empty for an entry that
        reads another entry's cache or keeps nothing)."""
        return [[] if entry.cache_from is not None else list(self.blocks[entry.layer].cache_needs())
                for entry in self.run_order]

    @property
    def capturable(self):
        """What of this model's steps can run inside a captured CUDA graph: True (any step), "decode" (steps of
        single tokens only) or False - the least that any part allows."""
        kinds = [p.capturable for p in self.parts()]
        if not all(kinds):
            return False
        return True if all(k is True for k in kinds) else "decode"

    def validate(self, ops, dtype: torch.dtype, page_size: int) -> None:
        """Asks every part whether its kernels take its sizes (raises with the part's message if not)."""
        for p in self.parts():
            p.validate(ops, dtype, page_size)

    # ---------------------------------------------------------------- step
    def forward(self, ctx: StepContext, cache_views: List[List[object]]) -> torch.Tensor:
        """Runs the step's tokens; returns float32 logits [ctx.num_logit_rows, vocab]."""
        stream = ResidualStream(self.embedding.forward(ctx))
        for e, entry in enumerate(self.run_order):
            self.blocks[entry.layer].forward(stream, ctx, cache_views[e])
        x = self.final_norm.norm_rows(stream.resid, stream.delta, ctx.logit_rows, ctx.num_logit_rows)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        return self.head.forward(x)
