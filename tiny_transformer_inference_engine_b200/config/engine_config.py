"""Options of the engine around the model: cache, scheduler, compute dtype.

Field names and derived quantities follow the reference's ``CacheConfig``,
``SchedulerConfig`` and ``EngineConfig`` (models/model_config.py:44-102).  What
the reference only declares (token budget, chunked prefill, recompute
preemption; models/model_config.py:53-67) is consumed here by the scheduler.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

COMPUTE_DTYPES = ("float32", "bfloat16")


@dataclass
class CacheConfig:
    block_size: int = 16                       # tokens per page (models/model_config.py:46)
    num_gpu_blocks: Optional[int] = None       # pages per cache group, scratch page 0 included
    kv_budget_bytes: int = 2 * 1024 ** 3       # used when num_gpu_blocks is None
    kv_dtype: Optional[str] = None             # None -> compute dtype
    enable_prefix_caching: bool = False        # declared by the reference, implemented nowhere

    def __post_init__(self):
        if not isinstance(self.block_size, int) or self.block_size <= 0:
            raise ValueError(f"block_size must be a positive integer, got {self.block_size!r}")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks < 2:
            raise ValueError("num_gpu_blocks must be at least 2: page 0 is scratch (serving/allocator.py:5)")
        if self.enable_prefix_caching:
            raise ValueError("prefix caching is not implemented (neither is it in the reference)")


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 32
    max_num_batched_tokens: int = 512
    enable_chunked_prefill: bool = True
    preemption: str = "recompute"
    policy: str = "fcfs"
    cudagraph_batch_sizes: List[int] = field(default_factory=lambda: [1, 2, 4, 8, 16, 32])

    def __post_init__(self):
        # models/model_config.py:63-67
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ValueError("every decode takes 1 token, so max_num_batched_tokens must cover max_num_seqs")
        if self.preemption != "recompute":
            raise ValueError("preemption must be 'recompute'")
        if self.policy != "fcfs":
            raise ValueError("policy must be 'fcfs'")
        self.cudagraph_batch_sizes = sorted(b for b in self.cudagraph_batch_sizes if b <= self.max_num_seqs)


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"                    # compute dtype of the step: "bfloat16" or "float32"
    cache: CacheConfig = field(default_factory=CacheConfig)
    sched: SchedulerConfig = field(default_factory=SchedulerConfig)
    use_cuda_graphs: bool = True
    pipelined_decode: bool = True              # launch the next captured decode step before the host has read this one's tokens
    split_step_classes: bool = True            # a mixed step's one-token requests and its portions run as two attention launches
    capture_repeated_steps: bool = True        # a step whose layout (tokens per request, wanted places) comes again is captured and replayed
    step_graph_max_tokens: int = 1024          # ... up to this many tokens (longer steps keep the GPU busy without it)
    max_step_graphs: int = 64                  # ... and at most this many such graphs are kept (least recently used goes; they share one memory pool)
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype not in COMPUTE_DTYPES:
            raise ValueError(f"compute dtype must be one of {COMPUTE_DTYPES}, got {self.dtype!r}")
        if self.cache.kv_dtype is not None and self.cache.kv_dtype != self.dtype:
            raise ValueError("a cache dtype other than the compute dtype is not supported (no quantized caches)")

    @property
    def kv_dtype(self) -> str:
        return self.cache.kv_dtype or self.dtype
