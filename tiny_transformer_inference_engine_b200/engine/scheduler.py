"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees, and decides what happens when pages run out.

The reference's ``Scheduler`` (serving/scheduler.py:7-79) admits first-come-first-served
while ``free - pages(prompt) >= running + 1``, feeds a whole prompt in one step, one
token per running request afterwards, frees a finished request's pages in the same step,
and *raises* when a decoding request cannot get its next page (serving/allocator.py:28-31).
Its ``SchedulerConfig`` declares a token budget, chunked prefill and
``preemption="recompute"`` without using them (models/model_config.py:53-67); here they
are used:

* every step first gives one token to each request that is decoding, then fills what is
  left of ``max_num_batched_tokens`` with prompt portions, oldest request first; a
  portion may be cut anywhere (>= 1 token); a request samples only in the step that
  holds its last uncached token;
* pages are taken portion by portion; admission keeps the reference's reserve rule;
* **out of pages -> preempt by recompute**: the most recently admitted running request
  gives back all its pages and its state slot and returns to the *front* of the waiting
  queue with the tokens it has generated so far; later it is prefilled again (prompt plus
  generated tokens) and goes on.  Its sampler counter goes on too, so the tokens it
  draws are the same as without preemption.  A request that could never fit an empty
  pool is refused at ``add_request``.

This class is pure host logic; the engine hands it a cache manager and runs the steps.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Tuple

from .batch import StepEntry
from ..cache import CacheManager, OutOfPages, pages_for
from ..config import SchedulerConfig
from ..sampling.params import SamplingParams


@dataclass
class Request:
    rid: int
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    num_cached: int = 0                    # tokens whose keys/values sit in the cache
    preemptions: int = 0
    finished: bool = False
    finish_reason: Optional[str] = None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.num_cached

    def span(self, start: int, n: int) -> List[int]:
        """Tokens start..start+n-1 of prompt + output, without building the whole list."""
        p = len(self.prompt)
        if start >= p:
            return self.output[start - p:start - p + n]
        if start + n <= p:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - p]


class Scheduler:
    def __init__(self, manager: CacheManager, config: SchedulerConfig, max_seq_len: int,
                 eos_token_id: Optional[int]):
        self.manager, self.config = manager, config
        self.max_seq_len, self.eos_token_id = max_seq_len, eos_token_id
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []           # in admission order
        self.next_rid = 0
        self.counters = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0,
                         "admitted": 0, "finished": 0}

    # ---------------------------------------------------------------- requests
    def add_request(self, prompt_ids: List[int], params: SamplingParams) -> int:
        # checks of inference.py:126-135
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("prompt must hold at least one token")
        if len(prompt) > self.max_seq_len:
            raise ValueError(f"prompt has {len(prompt)} tokens; model limit is {self.max_seq_len}")
        if len(prompt) + params.max_new_tokens > self.max_seq_len:
            raise ValueError("prompt plus requested generation exceeds max_seq_len")
        if params.max_new_tokens == 0:
            raise ValueError("max_new_tokens must be > 0 for a scheduled request")
        most = len(prompt) + params.max_new_tokens - 1      # the last sampled token is never cached
        if not self.manager.request_fits_empty_pool(most):
            raise ValueError(f"request needs {pages_for(most, self.manager.page_size)} pages of {self.manager.page_size} tokens; "
                             f"an empty pool has {self.manager.num_usable_pages}")
        req = Request(self.next_rid, prompt, params)
        self.next_rid += 1
        self.waiting.append(req)
        return req.rid

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- planning a step
    def _preempt(self, req: Request) -> None:
        self.manager.release(req.rid)
        self.running.remove(req)
        req.num_cached = 0
        req.preemptions += 1
        self.counters["preemptions"] += 1
        self.waiting.appendleft(req)

    def _reserve(self, req: Request, n: int, planned: Dict[int, int]) -> int:
        """Takes pages for the next ``n`` tokens of ``req``; when pages are short, preempts
        the youngest running request that is not in this step yet (possibly ``req``).
        Returns the number of tokens reserved (0 if ``req`` itself was preempted)."""
        while True:
            try:
                self.manager.extend(req.rid, req.num_cached, req.num_cached + n)
                return n
            except OutOfPages:
                victims = [r for r in self.running if r.rid not in planned]
                victim = victims[-1] if victims else None
                if victim is None or victim is req:
                    if len(self.running) == 1 and not planned:
                        raise RuntimeError("a lone request cannot get pages: the pool is smaller than add_request assumed")
                    self._preempt(req)
                    return 0
                self._preempt(victim)

    def _fit(self, req: Request, n: int) -> int:
        """Largest portion <= n of ``req`` that the free pages can hold without preemption."""
        while n > 0 and self.manager.pages_short(req.rid, req.num_cached, req.num_cached + n) > 0:
            ps = self.manager.page_size
            # shrink to the previous page edge
            end = req.num_cached + n
            end = (end - 1) // ps * ps
            n = end - req.num_cached
        return max(n, 0)

    def _admit_ok(self, req: Request) -> bool:
        if not self.manager.can_admit() or len(self.running) >= self.config.max_num_seqs:
            return False
        # serving/scheduler.py:33-37: keep one growth page for every running request and this one (in every cache group)
        return self.manager.admission_headroom(req.num_tokens, len(self.running) + 1) or not self.running

    def plan(self) -> List[StepEntry]:
        """Chooses the step's entries and takes their pages.  ``want`` is ``[last]`` for an
        entry that reaches the request's last uncached token, else empty."""
        budget = self.config.max_num_batched_tokens
        planned: Dict[int, int] = {}
        # 1. one token for every decoding request (oldest first)
        for req in list(self.running):
            if req not in self.running or req.remaining != 1 or budget <= 0:
                continue
            if self._reserve(req, 1, planned):
                planned[req.rid] = 1
                budget -= 1
        # 2. portions of prompts already running (oldest first)
        for req in list(self.running):
            if req not in self.running or req.rid in planned or budget <= 0:
                continue
            n = min(req.remaining, budget)
            if not self.config.enable_chunked_prefill and n < req.remaining:
                continue
            fit = self._fit(req, n)
            if fit == 0 and not planned:
                fit = self._reserve(req, min(n, self.manager.page_size), planned)   # forces progress by preemption
            elif fit:
                self.manager.extend(req.rid, req.num_cached, req.num_cached + fit)
            if fit:
                planned[req.rid] = fit
                budget -= fit
        # 3. admissions, first come first served, head-of-line blocking
        while self.waiting and budget > 0:
            req = self.waiting[0]
            if not self._admit_ok(req):
                break
            n = min(req.remaining, budget)
            if not self.config.enable_chunked_prefill and n < req.remaining:
                break
            self.manager.admit(req.rid)
            fit = self._fit(req, n)
            if fit == 0:
                self.manager.release(req.rid)
                break
            self.manager.extend(req.rid, 0, fit)
            self.waiting.popleft()
            self.running.append(req)
            self.counters["admitted"] += 1
            planned[req.rid] = fit
            budget -= fit
        entries = []
        for req in self.running:
            n = planned.get(req.rid)
            if not n:
                continue
            toks = req.span(req.num_cached, n)
            want = [n - 1] if n == req.remaining else []
            entries.append(StepEntry(req.rid, req.num_cached, toks, want))
        return entries

    # ---------------------------------------------------------------- after the step
    def update(self, entries: List[StepEntry], sampled: List[int]) -> List[Tuple[int, int, bool]]:
        """``sampled`` holds one token per entry that wanted logits, in order.  Returns the
        reference's result tuples ``(request id, token, done)`` (serving/scheduler.py:69,79)."""
        self.counters["steps"] += 1
        by_rid = {r.rid: r for r in self.running}
        results, k = [], 0
        for en in entries:
            req = by_rid.get(en.rid)
            if req is None:                 # it ended while this step, launched ahead of the host, was in flight
                k += len(en.want)
                continue
            n = len(en.tokens)
            if req.num_cached < len(req.prompt):
                self.counters["prefill_tokens"] += n
            else:
                self.counters["decode_tokens"] += n
            req.num_cached += n
            if not en.want:
                continue
            tok = int(sampled[k]); k += 1
            req.output.append(tok)
            eos = (self.eos_token_id is not None and tok == self.eos_token_id and not req.params.ignore_eos)
            done = eos or len(req.output) >= req.params.max_new_tokens      # serving/scheduler.py:66-67
            if done:
                req.finished, req.finish_reason = True, ("eos" if eos else "length")
                self.manager.release(req.rid)                               # same step (serving/scheduler.py:71-72)
                self.running.remove(req)
                self.counters["finished"] += 1
            results.append((req.rid, tok, done))
        return results
