"""The scheduler's decisions on the host, with a fake step function: admission, portions under
a token budget, decoding, finishing and freeing, and preemption by recompute when pages run out."""
import random

import pytest

from tiny_transformer_inference_engine_b200.cache import CacheManager
from tiny_transformer_inference_engine_b200.config import SchedulerConfig
from tiny_transformer_inference_engine_b200.engine.scheduler import Scheduler
from tiny_transformer_inference_engine_b200.parts.base import PagedKVNeed, RunEntry
from tiny_transformer_inference_engine_b200.sampling import SamplingParams


def make(pages=20, page=4, slots=4, budget=16, max_seq_len=64, eos=None, chunked=True):
    needs = [PagedKVNeed(1, 4)]
    mgr = CacheManager(needs, [RunEntry(0)], page, pages, slots, "float32", "cpu", allocate=False)
    cfg = SchedulerConfig(max_num_seqs=slots, max_num_batched_tokens=budget, enable_chunked_prefill=chunked,
                          cudagraph_batch_sizes=[])
    return Scheduler(mgr, cfg, max_seq_len, eos), mgr


def fake_token(rid, index):
    return (rid * 7 + index * 3) % 50


class Shadow:
    """Checks every step against what the cache must hold, and plays the model."""

    def __init__(self, sched, mgr):
        self.sched, self.mgr, self.cached, self.log = sched, mgr, {}, []

    def run_step(self):
        before = {r.rid: r.preemptions for r in list(self.sched.running) + list(self.sched.waiting)}
        entries = self.sched.plan()
        by = {r.rid: r for r in self.sched.running}
        for r in self.sched.waiting:
            if r.preemptions != before.get(r.rid, r.preemptions):
                self.cached.pop(r.rid, None)                      # preempted: its cache is gone
        assert sum(len(e.tokens) for e in entries) <= self.sched.config.max_num_batched_tokens
        assert len(entries) <= self.sched.config.max_num_seqs
        sampled = []
        for e in entries:
            req = by[e.rid]
            have = self.cached.get(e.rid, 0)
            assert e.start == have == req.num_cached, (e, have)
            assert list(e.tokens) == req.tokens[have:have + len(e.tokens)]
            table = self.mgr.table(0, e.rid)
            assert len(table) * self.mgr.page_size >= have + len(e.tokens)
            self.cached[e.rid] = have + len(e.tokens)
            if e.want:
                assert e.want == [len(e.tokens) - 1] and self.cached[e.rid] == len(req.tokens)
                sampled.append(fake_token(e.rid, len(req.output)))
        results = self.sched.update(entries, sampled)
        for rid, tok, done in results:
            if done:
                self.cached.pop(rid, None)
        self.mgr.check()
        self.log.append(entries)
        return results

    def drain(self, limit=10000):
        out = {}
        for _ in range(limit):
            if not self.sched.has_work:
                break
            for rid, tok, done in self.run_step():
                out.setdefault(rid, []).append(tok)
        assert not self.sched.has_work
        return out


def test_two_requests_finish_and_free():
    s, m = make()
    a = s.add_request([1, 2, 3, 4, 5], SamplingParams(max_new_tokens=3))
    b = s.add_request([6] * 9, SamplingParams(max_new_tokens=5))
    out = Shadow(s, m).drain()
    assert out[a] == [fake_token(a, i) for i in range(3)] and out[b] == [fake_token(b, i) for i in range(5)]
    assert m.num_free_pages == m.num_usable_pages and m.slots.num_free == 4
    assert s.counters["finished"] == 2 and s.counters["preemptions"] == 0


def test_budget_cuts_prompts_into_portions_and_decodes_first():
    s, m = make(budget=8, pages=40)
    a = s.add_request(list(range(20)), SamplingParams(max_new_tokens=4))
    sh = Shadow(s, m)
    sh.run_step()
    assert [len(e.tokens) for e in sh.log[-1]] == [8] and sh.log[-1][0].want == []
    b = s.add_request(list(range(5)), SamplingParams(max_new_tokens=4))
    sh.run_step()                                               # a's next portion takes the whole budget
    assert [(e.rid, len(e.tokens)) for e in sh.log[-1]] == [(a, 8)]
    res = sh.run_step()                                         # a's last 4 tokens, then b gets what is left
    assert [(e.rid, len(e.tokens)) for e in sh.log[-1]] == [(a, 4), (b, 4)]
    assert [r[0] for r in res] == [a]                           # a sampled; b has one prompt token left
    sh.run_step()                                               # a decodes first (1 token), b's last prompt token
    assert [(e.rid, len(e.tokens), e.want) for e in sh.log[-1]] == [(a, 1, [0]), (b, 1, [0])]
    sh.drain()
    assert m.num_free_pages == m.num_usable_pages


def test_without_chunking_a_prompt_waits_for_a_whole_step():
    s, m = make(budget=16, chunked=False, pages=40)
    a = s.add_request(list(range(10)), SamplingParams(max_new_tokens=2))
    b = s.add_request(list(range(10)), SamplingParams(max_new_tokens=2))
    sh = Shadow(s, m)
    sh.run_step()
    assert [(e.rid, len(e.tokens)) for e in sh.log[-1]] == [(a, 10)]     # b would have to be cut: it waits
    sh.run_step()
    assert [(e.rid, len(e.tokens)) for e in sh.log[-1]] == [(a, 1), (b, 10)]
    sh.drain()


def test_eos_and_length_finish():
    s, m = make(eos=fake_token(0, 2))
    a = s.add_request([1, 2], SamplingParams(max_new_tokens=10))
    out = Shadow(s, m).drain()
    assert out[a] == [fake_token(0, 0), fake_token(0, 1), fake_token(0, 2)]       # the EOS token is reported
    s2, m2 = make(eos=fake_token(0, 2))
    b = s2.add_request([1, 2], SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert len(Shadow(s2, m2).drain()[b]) == 6


def test_admission_waits_for_pages_and_slots():
    # 8 requests, pool of 8 usable pages (tests/test_scheduler.py:71-87 of the reference)
    s, m = make(pages=9, page=4, slots=3, budget=32)
    rids = [s.add_request([1] * 7, SamplingParams(max_new_tokens=3)) for _ in range(8)]
    sh = Shadow(s, m)
    first = sh.run_step()
    assert 0 < len(s.running) <= 3 and len(s.waiting) >= 5                        # queueing is seen
    out = sh.drain()
    for rid, tok, _ in first:
        out[rid] = [tok] + out.get(rid, [])
    assert sorted(out) == rids and all(len(v) == 3 for v in out.values())
    assert m.num_free_pages == m.num_usable_pages


def test_refusals():
    s, m = make(pages=5, page=4, max_seq_len=64)
    with pytest.raises(ValueError, match="at least one token"):
        s.add_request([], SamplingParams(max_new_tokens=2))
    with pytest.raises(ValueError, match="exceeds max_seq_len"):
        s.add_request([1] * 60, SamplingParams(max_new_tokens=10))
    with pytest.raises(ValueError, match="model limit"):
        s.add_request([1] * 65, SamplingParams(max_new_tokens=1))
    with pytest.raises(ValueError, match="empty pool"):
        s.add_request([1] * 16, SamplingParams(max_new_tokens=2))                  # 17 tokens cached > 4 pages
    s.add_request([1] * 15, SamplingParams(max_new_tokens=2))                      # 16 cached tokens fit exactly
    Shadow(s, m).drain()


def test_pages_run_out_preempts_the_youngest_and_recomputes():
    # two requests that each grow to 4 pages, pool of 6: the younger is preempted, then finishes
    s, m = make(pages=7, page=4, slots=4, budget=32)
    a = s.add_request([1] * 8, SamplingParams(max_new_tokens=8))
    b = s.add_request([2] * 8, SamplingParams(max_new_tokens=8))
    sh = Shadow(s, m)
    out = sh.drain()
    assert s.counters["preemptions"] >= 1
    assert out[a] == [fake_token(a, i) for i in range(8)] and out[b] == [fake_token(b, i) for i in range(8)]
    req_b = [e for step in sh.log for e in step if e.rid == b]
    assert any(e.start == 0 and len(e.tokens) > 8 for e in req_b)                  # re-prefilled with its outputs
    assert m.num_free_pages == m.num_usable_pages and m.slots.num_free == 4


@pytest.mark.parametrize("seed", range(6))
def test_random_load_never_loses_a_page_or_a_token(seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    s, m = make(pages=rng.choice([10, 14, 24]), page=page, slots=rng.choice([2, 4]), budget=rng.choice([4, 9, 32]),
                max_seq_len=48)
    sh, want, out = Shadow(s, m), {}, {}
    for step in range(400):
        if rng.random() < 0.3 and len(want) < 25:
            n, k = rng.randint(1, 20), rng.randint(1, 12)
            if -(-(n + k - 1) // page) <= m.num_usable_pages:
                rid = s.add_request([rng.randrange(50) for _ in range(n)], SamplingParams(max_new_tokens=k))
                want[rid] = k
        if s.has_work:
            for rid, tok, done in sh.run_step():
                out.setdefault(rid, []).append(tok)
    out2 = sh.drain()
    for rid, toks in out2.items():
        out.setdefault(rid, []).extend(toks)
    assert {r: len(t) for r, t in out.items()} == want
    assert all(out[r] == [fake_token(r, i) for i in range(k)] for r, k in want.items())
    assert m.num_free_pages == m.num_usable_pages and m.slots.num_free == m.max_slots
