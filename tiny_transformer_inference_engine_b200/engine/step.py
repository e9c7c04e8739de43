"""The step function: a batch of (request, its next tokens) in, logits at the wanted
places out.

It generalises the reference's ``PagedTransformer.forward_batch`` (serving/paged_model.py:50-67):
any mix of prompt portions and single decoded tokens, cut anywhere, runs as ONE varlen
batch from the cache that earlier steps left; it runs only the tokens it is given and
returns 32-bit logits only where asked (the reference returns the last token of every
span).  The cache must already cover the new positions (``CacheManager.extend``).

Decode-only steps (one token per request, one wanted row each) can run from a captured
CUDA graph per batch-size bucket and context-length bucket: the metadata buffer keeps its
address and layout, so a replay needs only the one host-to-device copy.  The kernels of a
graph are planned for the longest context of its bucket (512, 2048, 8192, ... keys, at most
the model's ``max_seq_len``), so short contexts do not run kernels cut for long ones.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .batch import BatchPacker, StepEntry
from ..cache import CacheManager
from ..models.model import Model


class _DecodeGraph:
    def __init__(self, bucket, host, dev, graph, logits, tokens, ctx, launches):
        self.bucket, self.host, self.dev, self.graph, self.logits, self.ctx = bucket, host, dev, graph, logits, ctx
        self.tokens = tokens                # sampled tokens [bucket] if the graph samples, else None
        self.launches = launches            # kernels of this package inside the graph (counted while capturing)


class Stepper:
    def __init__(self, model: Model, manager: CacheManager, ops, dtype: torch.dtype, device,
                 graph_batch_sizes: Optional[List[int]] = None):
        self.model, self.manager, self.ops, self.dtype = model, manager, ops, dtype
        self.device = torch.device(device)
        self.packer = BatchPacker(manager, ops, dtype, device, model.spec.vocab_size, model.spec.max_seq_len)
        self.graph_batch_sizes = sorted(graph_batch_sizes or [])
        self._graphs: Dict[tuple, _DecodeGraph] = {}
        self.counters = {"steps": 0, "tokens": 0, "graph_replays": 0}
        self.last_tokens: Optional[torch.Tensor] = None      # tokens sampled inside the last step's graph, or None

    # ---------------------------------------------------------------- plain step
    @torch.no_grad()
    def step(self, entries: List[StepEntry], sampler=None, feed: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits (float32, [sum of wants, vocab]) in the order of the entries and of ``want``.
        With a ``sampler`` a captured decode step also samples (the kernel is part of the graph) and leaves the
        tokens in ``last_tokens``; any other step leaves None there and the caller samples from the logits.
        ``feed`` (captured decode steps only): token ids on the device, one per entry, that replace the entries'
        tokens - the step before this one sampled them and the host has not read them yet."""
        self.last_tokens = None
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        self.counters["steps"] += 1
        self.counters["tokens"] += sum(len(e.tokens) for e in entries)
        if self.graph_batch_sizes and self._is_decode(entries):
            bucket = next((b for b in self.graph_batch_sizes if b >= len(entries)), None)
            if bucket is not None:
                return self._step_graph(entries, bucket, sampler, feed)
        if feed is not None:
            raise ValueError("tokens can be fed on the device only into a captured decode step")
        ctx = self.packer.pack(entries)
        views = self.manager.views(ctx.block_tables)
        return self.model.forward(ctx, views)

    @staticmethod
    def _is_decode(entries) -> bool:
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    # ---------------------------------------------------------------- captured decode step
    def _fixed_pages(self) -> Dict[int, int]:
        return {gi: -(-self.model.spec.max_seq_len // g.page_size) for gi, g in enumerate(self.manager.groups)}

    def _context_bucket(self, entries) -> int:
        need = max(e.start for e in entries) + 1
        limit, b = self.model.spec.max_seq_len, 512
        while b < need and b < limit:
            b *= 4
        return min(b, limit)

    def _step_graph(self, entries, bucket: int, sampler=None, feed=None) -> torch.Tensor:
        n = len(entries)
        keys = self._context_bucket(entries)
        key = (bucket, keys, sampler is not None)
        g = self._graphs.get(key)
        pages = self._fixed_pages()
        if g is None:
            # The step that meets a new (batch, context) bucket runs eagerly - that is the warm-up - and its results
            # are the step's results; the capture that follows runs nothing, so per-request state that a part advances
            # (fixed-size state, sampler draw counters) moves once.
            words = 8 * (bucket + 4) + sum(bucket * w + 4 for w in pages.values()) + 64
            host = torch.empty(words, dtype=torch.int32, pin_memory=True)
            dev = torch.zeros(words, dtype=torch.int32, device=self.device)
            ctx = self.packer.pack(entries, pad_seqs=bucket, pages_per_seq=pages, buffers=(host, dev))
            if feed is not None:
                self.packer.feed_tokens(feed)
            # the captured kernels must cover every context length of the bucket: size them for the longest
            ctx.max_kv_len = keys                                # (a decode step is one class: nothing else carries a length)
            views = self.manager.views(ctx.block_tables)
            logits = self.model.forward(ctx, views)
            tokens = sampler.sample(logits, ctx.slot_ids) if sampler is not None else None
            torch.cuda.synchronize(self.device)
            ctx.step_cache.clear()                              # what parts computed once per step is computed again inside the graph
            graph = torch.cuda.CUDAGraph()
            before = getattr(self.ops, "launches", 0)
            with torch.cuda.graph(graph):
                g_logits = self.model.forward(ctx, views)
                g_tokens = sampler.sample(g_logits, ctx.slot_ids) if sampler is not None else None
            self._graphs[key] = _DecodeGraph(bucket, host, dev, graph, g_logits, g_tokens, ctx,
                                             getattr(self.ops, "launches", 0) - before)
            if tokens is not None:
                self.last_tokens = tokens[:n]
            return logits[:n]
        self.packer.pack(entries, pad_seqs=bucket, pages_per_seq=pages, buffers=(g.host, g.dev), copy_only=True)
        if feed is not None:
            self.packer.feed_tokens(feed)
        g.graph.replay()
        if hasattr(self.ops, "launches"):
            self.ops.launches += g.launches
        self.counters["graph_replays"] += 1
        if g.tokens is not None:
            self.last_tokens = g.tokens[:n]
        return g.logits[:n]
