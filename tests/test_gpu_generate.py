"""Greedy generation through the entry point equals greedy decoding with the plain model;
sampling is reproducible per request whatever shares the batch; CUDA graphs change nothing."""
import pytest
import torch

from plain_model import plain_forward
from tiny_configs import TINY_A, TINY_B, SEEDS, PAGE
from gpu_util import make_engine, requests_for

from tiny_transformer_inference_engine_b200 import SamplingParams, generate_ids

pytestmark = pytest.mark.gpu


def plain_greedy_generate(cfg, w, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        logits = plain_forward(cfg, w, toks)[-1]
        t = int(torch.argmax(logits))
        out.append(t)
        toks.append(t)
        if t == cfg.get("eos_token_id"):
            break
    return out


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_matches_plain(graphs):
    cfg = TINY_A
    eng, w = make_engine(cfg, SEEDS["A"], PAGE["A"], 32, "float32", graphs=graphs, cudagraph_batch_sizes=[1, 2, 4])
    reqs = requests_for(cfg, (5, 17, 33), 3)
    outs = eng.generate(list(reqs.values()), SamplingParams(max_new_tokens=16, greedy=True))
    for prompt, out in zip(reqs.values(), outs):
        assert out == plain_greedy_generate(cfg, w, prompt, 16)
    assert eng.manager.num_free_pages == eng.manager.num_usable_pages
    one = generate_ids(eng, reqs["r1"], 16, greedy=True)
    assert one == outs[1]
    assert generate_ids(eng, reqs["r1"], 0) == []
    with pytest.raises(ValueError):
        generate_ids(eng, [], 4)
    with pytest.raises(ValueError):
        generate_ids(eng, reqs["r1"], -1)
    with pytest.raises(ValueError):
        generate_ids(eng, [1] * 60, 10)


def test_sampling_does_not_depend_on_batch():
    cfg = TINY_B
    eng, _ = make_engine(cfg, SEEDS["B"], PAGE["B"], 80, "float32", budget=16)
    reqs = list(requests_for(cfg, (1, 9, 40, 71), 4).values())
    params = [SamplingParams(max_new_tokens=24, temperature=0.8, seed=100 + i, ignore_eos=True) for i in range(4)]
    together = eng.generate(reqs, params)
    alone = [eng.generate([r], [p])[0] for r, p in zip(reqs, params)]
    assert all(len(o) == 24 for o in together)
    assert together == alone
    assert eng.manager.num_free_pages == eng.manager.num_usable_pages


def test_graph_replays_match_whole_prompts_bfloat16():
    """Captured decode steps in bfloat16 against the same engine without graphs running every request whole.
    Requests of different lengths end at different steps (the batch shrinks and changes its graph bucket; the
    longest context leaves first, then the next, so the context bucket of the graphs changes too),
    contexts cross page boundaries while steps are replayed (the incremental repacking of a steady decode
    step), and with 16 heads of size 64 on one kv head both decode attention kernels run inside graphs: the
    kernels of a graph are planned for the longest context, 4,096 keys, which is the tcgen05 kernel with
    split keys; the eager steps of the short requests take the cluster form."""
    from trace_util import run_steps, whole, worst_relative
    from gpu_util import TOL
    cfg = dict(architecture="mqa_gpt", vocab_size=300, d_model=1024, num_layers=2, num_heads=16, num_kv_heads=1,
               hidden_size=320, max_seq_len=4096, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False,
               eos_token_id=None, dtype="bfloat16")
    g = torch.Generator().manual_seed(5)
    prefix = {"a": 2300, "b": 40, "c": 700, "d": 9}
    tail = {"a": 12, "b": 70, "c": 33, "d": 50}
    reqs = {r: torch.randint(0, 300, (prefix[r] + tail[r],), generator=g).tolist() for r in prefix}
    eager, w = make_engine(cfg, 3, 64, 80, "bfloat16", max_seqs=4, budget=4096, graphs=False)
    ref = run_steps(eager, whole(reqs))
    expected = {r: [ref[(r, i)] for i in range(len(t))] for r, t in reqs.items()}
    steps = [{"entries": [{"id": r, "tokens": t[:prefix[r]], "want": [prefix[r] - 1]}], "end": []} for r, t in reqs.items()]
    fed = dict(prefix)
    while fed:
        entries = [{"id": r, "tokens": reqs[r][fed[r]:fed[r] + 1], "want": [0]} for r in fed]
        for r in fed:
            fed[r] += 1
        end = [r for r in fed if fed[r] == len(reqs[r])]
        steps.append({"entries": entries, "end": end})
        for r in end:
            del fed[r]
    graphs, _ = make_engine(cfg, 3, 64, 80, "bfloat16", max_seqs=4, budget=4096, graphs=True, weights=w, cudagraph_batch_sizes=[1, 2, 4])
    got = run_steps(graphs, steps)
    assert graphs.stats()["step_graph_replays"] == 70 - 4              # 70 decode steps; the four that met a new bucket ran eagerly
    assert {k[:2] for k in graphs.stepper._graphs} == {(4, 4096), (4, 2048), (2, 512), (1, 512)}
    assert {graphs.ops.attention_plan(torch.bfloat16, 4, 16, 1, 64, 1, n, 64)[:2] for n in (300, 4096)} == {("tc", 3), ("tc", 32)}
    worst, where = worst_relative(got, expected)
    assert worst < TOL["bfloat16"], (worst, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pipelined_decode_changes_nothing(dtype):
    """Launching the next captured decode step before the host has read the last one's tokens gives the same
    tokens as reading every step first: requests that end by length and by EOS (which the host learns one
    step late: the step already in flight for them is dropped), requests that arrive while others decode,
    and every page back at the end."""
    cfg = dict(TINY_A, max_seq_len=1100, eos_token_id=None)
    lens, news = (505, 17, 33, 9, 21, 40), (30, 12, 25, 40, 6, 18)      # the first one crosses 512 keys: another context bucket of graphs
    prompts = list(requests_for(cfg, lens, 9).values())
    params = [SamplingParams(max_new_tokens=n, temperature=1.3, seed=40 + i) for i, n in enumerate(news)]
    # the EOS id is chosen from what an engine without one generates: the ninth token of the fourth request
    probe, _ = make_engine(cfg, SEEDS["A"], PAGE["A"], 80, dtype, max_seqs=4, budget=64, graphs=True, cudagraph_batch_sizes=[1, 2, 4])
    cfg = dict(cfg, eos_token_id=probe.generate(prompts[3:4], params[3:4])[0][8])
    del probe
    outs, ends = [], []
    for pipelined in (False, True):
        eng, _ = make_engine(cfg, SEEDS["A"], PAGE["A"], 80, dtype, max_seqs=4, budget=64, graphs=True, cudagraph_batch_sizes=[1, 2, 4])
        eng.engine_config.pipelined_decode = pipelined
        got = {}
        rids = [eng.add_request(p, q) for p, q in zip(prompts[:4], params[:4])]
        calls = 0
        while eng.scheduler.has_work or eng._inflight is not None:
            for rid, tok, done in eng.step():
                got.setdefault(rid, []).append(tok)
            calls += 1
            if calls == 7:                                                          # two more arrive while the first four decode
                rids += [eng.add_request(p, q) for p, q in zip(prompts[4:], params[4:])]
            assert calls < 400
        assert eng.manager.num_free_pages == eng.manager.num_usable_pages
        eng.manager.check()
        outs.append([got[r] for r in rids])
        ends.append([eng._requests[r].finish_reason for r in rids])
        if pipelined:
            assert eng.stats()["step_graph_replays"] > 20
            assert {k[1] for k in eng.stepper._graphs} >= {512, 1100}
    assert outs[0] == outs[1]
    assert ends[0] == ends[1]
    assert any(e == "eos" for e in ends[0]) and any(e == "length" for e in ends[0])
    for o, n in zip(outs[0], news):
        assert 1 <= len(o) <= n
