"""The Python entry point: load or make a model, generate.

In the reference's manner (inference.py:68-152, serving/generation.py:11-69):
``load_model(path)`` gives an engine, ``generate_ids(engine, prompt_ids, max_new_tokens,
temperature=, top_k=, top_p=)`` gives the new token ids of one prompt with the same
argument checks, ``Engine.generate`` does it for many prompts through the scheduler,
and ``add_request`` / ``step`` expose the continuous loop (serving/scheduler.py:24,46).
A generated EOS token is reported and ends the request, as in ``generate_ids``
(inference.py:147-150).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .. import models as _models  # noqa: F401  (registers the architecture)
from ..cache import CacheManager
from ..cache.allocator import OutOfPages
from ..config import ModelConfig, EngineConfig, CacheConfig, SchedulerConfig
from ..models.model import Model
from ..registry import model_spec
from ..sampling import SamplingParams, Sampler
from ..weights import load_folder, place, random_tensors
from .batch import StepEntry
from .scheduler import Scheduler
from .step import Stepper

_TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class _Pending:
    """A launched decode step whose sampled tokens the host has not read yet."""
    __slots__ = ("entries", "tokens_dev", "host", "event")

    def __init__(self, entries, tokens_dev, host, event):
        self.entries, self.tokens_dev, self.host, self.event = entries, tokens_dev, host, event


class Engine:
    def __init__(self, config: ModelConfig, tensors_or_folder, engine_config: Optional[EngineConfig] = None,
                 ops=None):
        self.config = config
        self.engine_config = ec = engine_config or EngineConfig()
        self.device = torch.device(ec.device)
        self.dtype = _TORCH[ec.dtype]
        if ops is None:
            from ..ops import get_ops
            ops = get_ops(self.device)
        self.ops = ops
        self.spec = model_spec(config)
        self.model = Model(self.spec)
        # sizes the kernels do not take are refused here, before weights are read or a pool is made
        if hasattr(ops, "check_dtype"):
            ops.check_dtype(self.dtype)
        self.model.validate(ops, self.dtype, ec.cache.block_size)
        specs = self.model.param_specs()
        # weights are checked against the configuration before anything large is allocated
        if isinstance(tensors_or_folder, (str, os.PathLike)):
            tensors = load_folder(str(tensors_or_folder), specs, self.dtype, self.device)
        else:
            tensors = place(tensors_or_folder, specs, self.dtype, self.device)
        self.model.bind(ops, self.dtype, self.device)
        self.model.load(tensors)
        del tensors
        needs = self.model.cache_needs()
        self.manager = CacheManager(needs, self.model.run_order, ec.cache.block_size, ec.cache.num_gpu_blocks,
                                    ec.sched.max_num_seqs, ec.kv_dtype, self.device,
                                    kv_budget_bytes=ec.cache.kv_budget_bytes,
                                    max_step_tokens=ec.sched.max_num_batched_tokens)
        # The reference insists that the pool hold one sequence of max_seq_len plus the scratch page
        # (models/model_config.py:101-102).  Here a smaller pool is allowed on purpose - a replay or a test sizes its
        # pool for the tokens it will hold - and add_request refuses a request that could never fit; what cannot work
        # at all is a group without a usable page.
        if any(g.allocator.num_usable < 1 for g in self.manager.groups):
            raise ValueError("a cache group holds no usable page")
        # a part that reads device values on the host keeps the whole model off the captured path
        graphs = ec.sched.cudagraph_batch_sizes if (ec.use_cuda_graphs and self.device.type == "cuda" and self.model.capturable) else []
        self.stepper = Stepper(self.model, self.manager, ops, self.dtype, self.device, graphs,
                               capture_repeated=bool(graphs) and ec.capture_repeated_steps and self.model.capturable is True,
                               step_graph_max_tokens=ec.step_graph_max_tokens, max_step_graphs=ec.max_step_graphs,
                               split_classes=ec.split_step_classes)
        self.sampler = Sampler(ops, ec.sched.max_num_seqs, config.vocab_size, self.device)
        self._slot_ids = None
        self._inflight: Optional[_Pending] = None
        if self.device.type == "cuda":
            self._pinned = [torch.zeros(ec.sched.max_num_seqs, dtype=torch.int32).pin_memory() for _ in range(2)]
            self._events = [torch.cuda.Event() for _ in range(2)]
        self._pin_turn = 0
        self.scheduler = Scheduler(self.manager, ec.sched, config.max_seq_len, config.eos_token_id)
        self._requests: Dict[int, object] = {}

    # ---------------------------------------------------------------- construction
    @classmethod
    def from_folder(cls, folder: str, engine_config: Optional[EngineConfig] = None, ops=None, **opts) -> "Engine":
        return cls(ModelConfig.from_json(folder), folder, _engine_config(engine_config, opts), ops)

    @classmethod
    def from_checkpoint(cls, ckpt_path: str, engine_config: Optional[EngineConfig] = None, ops=None, **opts) -> "Engine":
        """From a checkpoint file of the reference (inference.py:68-87): converted into a temporary model folder
        (``weights/convert.py``), loaded from there, and the folder removed."""
        import shutil
        import tempfile
        from ..weights.convert import convert_checkpoint
        folder = tempfile.mkdtemp(prefix="ttie_model_")
        try:
            convert_checkpoint(ckpt_path, folder)
            return cls.from_folder(folder, engine_config, ops, **opts)
        finally:
            shutil.rmtree(folder, ignore_errors=True)

    @classmethod
    def from_random(cls, config: Union[ModelConfig, dict, str], seed: int = 0,
                    engine_config: Optional[EngineConfig] = None, ops=None, **opts) -> "Engine":
        if isinstance(config, str):
            config = ModelConfig.from_json(config)
        elif isinstance(config, dict):
            config = ModelConfig.from_dict(config)
        return cls(config, random_tensors(config, seed), _engine_config(engine_config, opts), ops)

    # ---------------------------------------------------------------- continuous loop
    def add_request(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        for t in prompt_ids:
            if not 0 <= int(t) < self.config.vocab_size:
                raise ValueError(f"token id {t} outside [0, {self.config.vocab_size})")
        rid = self.scheduler.add_request(list(prompt_ids), params)
        self._requests[rid] = self.scheduler.waiting[-1]
        return rid

    def has_unfinished(self) -> bool:
        """Whether a call of ``step`` still has something to do: requests waiting or running, or a launched step whose
        tokens the host has not read yet."""
        return self._inflight is not None or self.scheduler.has_work

    @torch.no_grad()
    def step(self) -> List[Tuple[int, int, bool]]:
        """One scheduler step: plan, run the batch, sample on the device, read the tokens.

        With ``pipelined_decode`` a captured decode step is followed at once by its successor - the same
        requests one position on, fed on the device with the tokens just sampled - before the host reads
        its tokens, so the GPU does not wait while the host reads, updates and plans.  The results returned
        are then those of the older of the two steps; a call that finds a step in flight and cannot follow it
        up (a request about to end, requests waiting, pages short) only reads it."""
        pending = self._inflight
        self._inflight = None
        if pending is None:
            pending = self._plan_and_launch()
            if not isinstance(pending, _Pending):
                return pending                                                          # results of a step that was read at once
        follow = self._follow_up(pending) if self.engine_config.pipelined_decode else None
        results = self._read(pending)
        self._inflight = follow
        return results

    def _plan_and_launch(self):
        sched = self.scheduler
        before = {r.rid for r in sched.running}
        entries = sched.plan()
        if not entries:
            return []
        for r in sched.running:
            if r.rid not in before or r.num_cached == 0:
                self.sampler.set_request(self.manager.slot_of[r.rid], r.params, draws_so_far=len(r.output))
        logits = self.stepper.step(entries, self.sampler)
        if self.stepper.last_tokens is not None:                                        # a captured decode step sampled in its graph
            return self._pend(entries, self.stepper.last_tokens)
        slots = [self.manager.slot_of[e.rid] for e in entries if e.want]
        if slots:
            key = tuple(slots)
            if self._slot_ids is None or self._slot_ids[0] != key:                      # the same requests step after step: one upload
                self._slot_ids = (key, torch.tensor(slots, dtype=torch.int32).to(self.device))
            tokens = self.sampler.sample(logits[:len(slots)], self._slot_ids[1]).tolist()   # one device-to-host read
        else:
            tokens = []
        if hasattr(self.ops, "check_tc"):
            self.ops.check_tc()
        return sched.update(entries, tokens)

    def _pend(self, entries, tokens_dev: torch.Tensor) -> "_Pending":
        """Starts the copy of a launched step's tokens into pinned memory; the host reads them later."""
        n = tokens_dev.shape[0]
        self._pin_turn ^= 1
        host = self._pinned[self._pin_turn]
        host[:n].copy_(tokens_dev, non_blocking=True)
        event = self._events[self._pin_turn]
        event.record()
        return _Pending(entries, tokens_dev, host, event)

    def _follow_up(self, pending: "_Pending") -> Optional["_Pending"]:
        """Launches the decode step after ``pending`` for the same requests, or returns None where that step is not
        certain to be wanted as it stands: a request may reach its last token, may have ended already, requests
        wait for admission, or pages run short (the scheduler then decides, after the host has caught up)."""
        sched = self.scheduler
        if sched.waiting:
            return None
        running = {r.rid: r for r in sched.running}
        for e in pending.entries:
            r = running.get(e.rid)
            # its output does not hold the token of the step in flight yet: that one and the next must both be wanted
            if r is None or len(r.output) + 2 > r.params.max_new_tokens or e.start + 2 > self.config.max_seq_len:
                return None
        if len(pending.entries) != len(running):
            return None
        try:
            for e in pending.entries:
                self.manager.extend(e.rid, e.start + 1, e.start + 2)
        except OutOfPages:
            return None                                                                 # (pages taken so far are the requests' next ones anyway)
        entries = [StepEntry(e.rid, e.start + 1, [0], [0]) for e in pending.entries]
        self.stepper.step(entries, self.sampler, feed=pending.tokens_dev)
        if self.stepper.last_tokens is None:
            raise RuntimeError("the step after a captured decode step did not run from a graph")
        return self._pend(entries, self.stepper.last_tokens)

    def _read(self, pending: "_Pending") -> List[Tuple[int, int, bool]]:
        pending.event.synchronize()
        tokens = pending.host[:len(pending.entries)].tolist()
        if hasattr(self.ops, "check_tc"):
            self.ops.check_tc()
        return self.scheduler.update(pending.entries, tokens)

    # ---------------------------------------------------------------- whole generations
    def generate(self, prompts_ids: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[List[int]]:
        """New token ids for every prompt (host lists in, host lists out)."""
        if not prompts_ids:
            return []
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts_ids)
        if len(params) != len(prompts_ids):
            raise ValueError("one SamplingParams per prompt, or one for all")
        for ids, p in zip(prompts_ids, params):                                         # inference.py:126-135
            if p.max_new_tokens and not len(ids):
                raise ValueError("prompt must hold at least one token")
            if len(ids) + p.max_new_tokens > self.config.max_seq_len:
                raise ValueError("prompt plus requested generation exceeds max_seq_len")
        outputs: Dict[int, List[int]] = {}
        order = []
        for ids, p in zip(prompts_ids, params):
            if p.max_new_tokens == 0:
                order.append(None)
                continue
            rid = self.add_request(ids, p)
            order.append(rid)
            outputs[rid] = []
        while any(rid is not None and not self._requests[rid].finished for rid in order):
            for rid, tok, _ in self.step():
                if rid in outputs:
                    outputs[rid].append(tok)
        for rid in outputs:
            self._requests.pop(rid, None)
        return [outputs[rid] if rid is not None else [] for rid in order]

    def stats(self) -> dict:
        return {**self.scheduler.counters, **{f"step_{k}": v for k, v in self.stepper.counters.items()},
                "pages_free": self.manager.num_free_pages, "pages_usable": self.manager.num_usable_pages}


def _engine_config(engine_config: Optional[EngineConfig], opts: dict) -> EngineConfig:
    if engine_config is not None:
        if opts:
            raise ValueError("give either an EngineConfig or keyword options")
        return engine_config
    cache_keys = {"block_size", "num_gpu_blocks", "kv_budget_bytes"}
    sched_keys = {"max_num_seqs", "max_num_batched_tokens", "enable_chunked_prefill", "cudagraph_batch_sizes"}
    cache = CacheConfig(**{k: opts.pop(k) for k in list(opts) if k in cache_keys})
    sched = SchedulerConfig(**{k: opts.pop(k) for k in list(opts) if k in sched_keys})
    return EngineConfig(cache=cache, sched=sched, **opts)


# ------------------------------------------------------------------- the reference's names
def load_model(path: str, device: str = "cuda:0", **opts) -> Engine:
    """``inference.py:68`` takes a checkpoint file; this takes a model folder, or such a file."""
    import os
    if os.path.isfile(path):
        return Engine.from_checkpoint(path, device=device, **opts)
    return Engine.from_folder(path, device=device, **opts)


def generate_ids(engine: Engine, prompt_ids: Sequence[int], max_new_tokens: int, *, temperature: float = 1.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0, greedy: bool = False) -> List[int]:
    """``inference.py:124-152`` with its checks: a negative count raises, zero tokens give
    ``[]`` (and need no prompt), an empty or over-long prompt raises."""
    if max_new_tokens < 0:
        raise ValueError("max_new_tokens must be >= 0")
    if max_new_tokens == 0:
        return []
    if not len(prompt_ids):
        raise ValueError("prompt must encode to at least one token")
    if len(prompt_ids) > engine.config.max_seq_len:
        raise ValueError(f"prompt has {len(prompt_ids)} tokens; model limit is {engine.config.max_seq_len}")
    params = SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                            seed=seed, greedy=greedy)
    return engine.generate([list(prompt_ids)], params)[0]
