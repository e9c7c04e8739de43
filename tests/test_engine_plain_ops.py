"""The engine's host side (cache manager, batch packer, step function, run order) on the
CPU, with the plain stand-ins for the kernels: every way of cutting the requests gives the
plain model's logits."""
import pytest
import torch

from plain_model import plain_forward
from plain_ops import PlainOps
from tiny_configs import TINY_A, TINY_B, SEEDS, PAGE
import trace_util as tu

from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig
from tiny_transformer_inference_engine_b200.weights import random_tensors


def make(cfg, seed, page, pages, dtype="float32"):
    mc = ModelConfig.from_dict(cfg)
    w = random_tensors(mc, seed, perturb_norms=True)
    ec = EngineConfig(dtype=dtype, device="cpu", use_cuda_graphs=False,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                      sched=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64))
    return Engine(mc, w, ec, ops=PlainOps()), w


def requests_for(cfg, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lens)}


@pytest.mark.parametrize("name,cfg,lens", [("A", TINY_A, (5, 17, 33, 64, 48, 21)), ("B", TINY_B, (1, 9, 40, 71, 128, 100))])
@pytest.mark.parametrize("mode", ["whole", "decode", "portions", "mixed"])
def test_cutting_does_not_change_logits(name, cfg, lens, mode):
    reqs = requests_for(cfg, lens, 5)
    steps = {"whole": tu.whole, "decode": tu.prefill_then_decode, "portions": tu.portions, "mixed": tu.mixed}[mode](reqs)
    pages = tu.max_live_tokens(steps) // PAGE[name] + 1
    eng, w = make(cfg, SEEDS[name], PAGE[name], pages)
    expected = {rid: plain_forward(cfg, w, toks) for rid, toks in reqs.items()}
    got = tu.run_steps(eng, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    worst, where = tu.worst_relative(got, expected)
    assert worst < 1e-5, (worst, where)


def test_steady_decode_steps_repack_to_the_same_buffer():
    """A decode step of the same requests in the same fixed layout rewrites only what changed; the device
    buffer must equal a full packing of the same step, across page boundaries, and a changed request set,
    a bad token or a table that does not cover the position must not slip through."""
    from tiny_transformer_inference_engine_b200.engine.batch import StepEntry
    eng, _ = make(TINY_A, SEEDS["A"], 4, 40)
    mgr, packer = eng.manager, eng.stepper.packer
    pages = {gi: -(-TINY_A["max_seq_len"] // g.page_size) for gi, g in enumerate(mgr.groups)}
    words = 8 * (4 + 4) + sum(4 * w + 4 for w in pages.values()) + 64

    def buffers():
        return torch.zeros(words, dtype=torch.int32), torch.zeros(words, dtype=torch.int32)

    lengths = {"a": 3, "b": 7, "c": 1}
    for rid, n in lengths.items():
        mgr.admit(rid)
        mgr.extend(rid, 0, n)
    fast, full = buffers(), buffers()
    short = []
    repack = packer._repack_decode
    packer._repack_decode = lambda entries, key: short.append(repack(entries, key)) or short[-1]
    g = torch.Generator().manual_seed(1)
    for step in range(14):                                           # pages of 4 tokens: every request crosses several
        entries = []
        for rid in lengths:
            mgr.extend(rid, lengths[rid], lengths[rid] + 1)
            entries.append(StepEntry(rid, lengths[rid], [int(torch.randint(0, 256, (1,), generator=g))], [0]))
            lengths[rid] += 1
        packer.pack(entries, pad_seqs=4, pages_per_seq=pages, buffers=fast, copy_only=True)
        assert short[-1] == (step > 0)                                # every step but the first takes the short path
        saved, packer._last = packer._last, None                     # a full packing into other buffers, then back
        packer.pack(entries, pad_seqs=4, pages_per_seq=pages, buffers=full, copy_only=True)
        packer._last = saved
        assert torch.equal(fast[1], full[1]), step
    # one request leaves: the layout key changes and the step is packed in full again
    mgr.release("b")
    del lengths["b"]
    entries = []
    for rid in lengths:
        mgr.extend(rid, lengths[rid], lengths[rid] + 1)
        entries.append(StepEntry(rid, lengths[rid], [5], [0]))
    packer.pack(entries, pad_seqs=4, pages_per_seq=pages, buffers=fast, copy_only=True)
    packer._last, saved = None, packer._last
    packer.pack(entries, pad_seqs=4, pages_per_seq=pages, buffers=full, copy_only=True)
    packer._last = saved
    assert torch.equal(fast[1], full[1])
    # the checks of a full packing hold on the short path too
    nxt = [StepEntry(rid, lengths[rid] + 1, [5], [0]) for rid in lengths]
    for rid in lengths:
        mgr.extend(rid, lengths[rid] + 1, lengths[rid] + 2)
    bad = [StepEntry(nxt[0].rid, nxt[0].start, [256], [0])] + nxt[1:]
    with pytest.raises(ValueError):
        packer.pack(bad, pad_seqs=4, pages_per_seq=pages, buffers=fast, copy_only=True)
    far = [StepEntry(nxt[0].rid, nxt[0].start + 9, [5], [0])] + nxt[1:]
    with pytest.raises(ValueError):
        packer.pack(far, pad_seqs=4, pages_per_seq=pages, buffers=fast, copy_only=True)


def test_mixed_step_is_packed_in_two_classes():
    """One-token requests are packed first, the others after them in the order given; wanted rows keep the
    order of the entries; the second class counts its tokens from its own first one."""
    from tiny_transformer_inference_engine_b200.engine.batch import StepEntry
    eng, _ = make(TINY_A, SEEDS["A"], 4, 40)
    mgr, packer = eng.manager, eng.stepper.packer
    spans = {"p": (0, [1, 2, 3, 4, 5]), "a": (9, [6]), "q": (2, [7, 8, 9]), "b": (4, [10])}
    for rid, (start, toks) in spans.items():
        mgr.admit(rid)
        mgr.extend(rid, 0, start + len(toks))
    entries = [StepEntry("p", 0, spans["p"][1], [4, 0]), StepEntry("a", 9, [6], [0]),
               StepEntry("q", 2, spans["q"][1], []), StepEntry("b", 4, [10], [0])]
    ctx = packer.pack(entries)
    assert ctx.token_ids.tolist() == [6, 10, 1, 2, 3, 4, 5, 7, 8, 9]
    assert ctx.positions.tolist() == [9, 4, 0, 1, 2, 3, 4, 2, 3, 4]
    assert ctx.token_seq.tolist() == [0, 1, 2, 2, 2, 2, 2, 3, 3, 3]
    assert ctx.query_start_loc.tolist() == [0, 1, 2, 7, 10]
    assert ctx.seq_lens.tolist() == [10, 5, 5, 5]
    assert ctx.slot_ids.tolist() == [mgr.slot_of[r] for r in ("a", "b", "p", "q")]
    assert ctx.logit_rows.tolist() == [6, 2, 0, 1]                     # p's place 4, p's place 0, a, b
    assert ctx.block_tables[0].tolist()[0][:3] == mgr.table(0, "a")
    single, rest = ctx.classes()
    assert (single.seq_lo, single.seq_hi, single.tok_lo, single.tok_hi, single.max_q_len, single.max_kv_len) == (0, 2, 0, 2, 1, 10)
    assert (rest.seq_lo, rest.seq_hi, rest.tok_lo, rest.tok_hi, rest.max_q_len, rest.max_kv_len) == (2, 4, 2, 10, 5, 5)
    assert single.query_start_loc.tolist() == [0, 1, 2] and rest.query_start_loc.tolist() == [0, 5, 8]
    # a step of one kind is one class: the step itself
    only = packer.pack(entries[1::2])
    assert only.seq_classes is None and len(only.classes()) == 1 and only.classes()[0].tok_hi == 2


def test_requests_added_between_steps():
    """``add_request`` between calls of ``step`` until ``has_unfinished`` says no, on a pool that throws a request out on
    the way: every request's greedy tokens equal plain greedy decoding."""
    from tiny_transformer_inference_engine_b200 import SamplingParams
    cfg = TINY_A
    eng, w = make(cfg, SEEDS["A"], 4, 12)
    g = torch.Generator().manual_seed(3)
    reqs = [(torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist(), new) for n, new in ((9, 12), (17, 10), (3, 14), (20, 8), (5, 5))]
    arrive = [0, 0, 2, 3, 9]
    assert not eng.has_unfinished()
    out, ids, nxt, step = {}, {}, 0, 0
    while nxt < len(reqs) or eng.has_unfinished():
        while nxt < len(reqs) and arrive[nxt] <= step:
            rid = eng.add_request(reqs[nxt][0], SamplingParams(max_new_tokens=reqs[nxt][1], greedy=True, ignore_eos=True))
            ids[rid], out[nxt] = nxt, []
            nxt += 1
        for rid, tok, _ in eng.step():
            out[ids[rid]].append(tok)
        step += 1
        assert step < 500
    assert eng.stats()["preemptions"] > 0 and eng.stats()["finished"] == len(reqs)
    eng.manager.check()
    assert eng.manager.num_free_pages == eng.manager.num_usable_pages
    for i, (prompt, new) in enumerate(reqs):
        toks = list(prompt)
        for _ in range(new):
            toks.append(int(torch.argmax(plain_forward(cfg, w, toks)[-1])))
        assert out[i] == toks[len(prompt):], i
