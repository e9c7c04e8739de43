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

Any other step whose layout comes again - the same numbers of tokens per request in the
same order, the same wanted places, the same context buckets, as in a prompt that is fed in
equal portions beside a steady set of decoding requests - is captured the second time it is
seen and replayed from then on: a step of a few hundred tokens on a small model is otherwise
bound by the host's launches, not by the GPU.  A few such graphs are kept (least recently
used goes); long steps are left alone.
"""
from __future__ import annotations

from collections import OrderedDict
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
                 graph_batch_sizes: Optional[List[int]] = None, capture_repeated: bool = False,
                 step_graph_max_tokens: int = 1024, max_step_graphs: int = 64, split_classes: bool = True):
        self.model, self.manager, self.ops, self.dtype = model, manager, ops, dtype
        self.device = torch.device(device)
        self.packer = BatchPacker(manager, ops, dtype, device, model.spec.vocab_size, model.spec.max_seq_len, split_classes)
        self.graph_batch_sizes = sorted(graph_batch_sizes or [])
        self._graphs: Dict[tuple, _DecodeGraph] = {}
        self.capture_repeated = bool(capture_repeated)
        self.step_graph_max_tokens, self.max_step_graphs = int(step_graph_max_tokens), int(max_step_graphs)
        self._step_graphs: "OrderedDict[tuple, _DecodeGraph]" = OrderedDict()      # repeated layouts, least recently used first
        self._seen: Dict[tuple, int] = {}                                          # layouts met once and not captured yet
        self._step_pool = None                                                     # memory pool the graphs of repeated layouts share
        self.counters = {"steps": 0, "tokens": 0, "graph_replays": 0, "step_graph_replays": 0, "step_graphs_captured": 0}
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
        if self.capture_repeated and sum(len(e.tokens) for e in entries) <= self.step_graph_max_tokens:
            logits = self._step_repeated(entries)
            if logits is not None:
                return logits
        ctx = self.packer.pack(entries)
        views = self.manager.views(ctx.block_tables)
        return self.model.forward(ctx, views)

    # ---------------------------------------------------------------- repeated layouts
    def _bucket(self, keys: int) -> int:
        limit, b = self.model.spec.max_seq_len, 2048                 # coarse: every bucket is a layout of its own
        while b < keys and b < limit:
            b *= 4
        return min(b, limit)

    def _step_repeated(self, entries) -> Optional[torch.Tensor]:
        """Replays the graph of this step's layout if there is one, captures one if the layout was seen before
        (running the step eagerly for its results first), else notes the layout and returns None."""
        single = [e for e in entries if len(e.tokens) == 1]
        others = [e for e in entries if len(e.tokens) != 1]
        buckets = tuple(self._bucket(max(e.start + len(e.tokens) for e in cls)) if cls else 0 for cls in (single, others))
        key = (tuple((len(e.tokens), tuple(e.want)) for e in entries), buckets)
        pages = self._fixed_pages()
        g = self._step_graphs.get(key)
        if g is not None:
            self._step_graphs.move_to_end(key)
            self.packer.pack(entries, pages_per_seq=pages, buffers=(g.host, g.dev), copy_only=True)
            g.graph.replay()
            if hasattr(self.ops, "launches"):
                self.ops.launches += g.launches
            self.counters["step_graph_replays"] += 1
            return g.logits
        if key not in self._seen:
            if len(self._seen) > 4096:
                self._seen.clear()
            self._seen[key] = 1
            return None
        del self._seen[key]
        n, T = len(entries), sum(len(e.tokens) for e in entries)
        words = 4 * (T + 4) + 5 * (n + 5) + sum(len(e.want) for e in entries) + sum(n * w + 4 for w in pages.values()) + 64
        host = torch.empty(words, dtype=torch.int32, pin_memory=True)
        dev = torch.zeros(words, dtype=torch.int32, device=self.device)
        ctx = self.packer.pack(entries, pages_per_seq=pages, buffers=(host, dev))
        # the captured kernels must cover every context length of the buckets: size them for the longest
        classes = ctx.seq_classes or []
        if classes:
            for c, b in zip(classes, buckets):
                c.max_kv_len = b
        ctx.max_kv_len = max(buckets)
        views = self.manager.views(ctx.block_tables)
        # this step runs eagerly, planned as the graph will be: its results are the step's, and every kernel the
        # graph holds has run once before the capture (a kernel's first launch may load code, which a capture forbids)
        logits = self.model.forward(ctx, views)
        torch.cuda.synchronize(self.device)
        ctx.step_cache.clear()
        graph = torch.cuda.CUDAGraph()
        before = getattr(self.ops, "launches", 0)
        # the graphs of repeated layouts share one memory pool: one of them runs at a time, and a step's logits are
        # read (by the sampler, or copied out) before the next step starts, as with two replays of one graph
        if self._step_pool is None:
            self._step_pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(graph, pool=self._step_pool):
            g_logits = self.model.forward(ctx, views)
        while len(self._step_graphs) >= self.max_step_graphs:
            self._step_graphs.popitem(last=False)
        self._step_graphs[key] = _DecodeGraph(0, host, dev, graph, g_logits, None, ctx, getattr(self.ops, "launches", 0) - before)
        self.counters["step_graphs_captured"] += 1
        return logits

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
