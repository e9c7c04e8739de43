"""Schedules and paths that only show through the whole engine, each against the plain model (never against
another path of the engine): prompts long enough for the two-tile tensor-core attention kernel and its key
split; preemption by recompute on a pool that is too small; captured decode steps with the sampler inside the
graph and the next step launched ahead of the host, in bfloat16 at head size 128; the 16-token-budget sampled
workload token by token against the plain sampler; and the bounded waits' failure path."""
import struct

import pytest
import torch

from plain_model import plain_forward
from plain_ops import PlainOps, uniform_from_state
from tiny_configs import TINY_A, TINY_B, SEEDS, PAGE
from gpu_util import make_engine, requests_for, TOL
import trace_util as tu

from tiny_transformer_inference_engine_b200 import SamplingParams

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(plain_forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


# ------------------------------------------------------------------------------------------ long prompts
LONG = {
    # 8 and 16 heads of 128 on one kv head; 64 heads of 64 on two
    "h128": dict(architecture="mqa_gpt", vocab_size=160, d_model=1024, num_layers=2, num_heads=8, num_kv_heads=1,
                 hidden_size=192, max_seq_len=2688, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, dtype="float32"),
    "h128w": dict(architecture="mqa_gpt", vocab_size=150, d_model=2048, num_layers=1, num_heads=16, num_kv_heads=1,
                  hidden_size=128, max_seq_len=2688, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, dtype="float32"),
    "h64": dict(architecture="mqa_gpt", vocab_size=130, d_model=4096, num_layers=1, num_heads=64, num_kv_heads=2,
                hidden_size=64, max_seq_len=2688, rope_theta=50000.0, rms_norm_eps=1e-6, bias=False, dtype="float32"),
}


@pytest.mark.parametrize("name,page", [("h128", 64), ("h128", 16), ("h128w", 64), ("h64", 64)])
def test_long_prompts_reach_the_tensor_core_kernels(name, page):
    """A 2,048-token portion (the two-tile kernel where its row tiles fill half of the GPU, else the one-tile kernel), a
    512-token portion behind it (its key range cut over CTAs, then the merge), the rest, decoded tokens beside another
    request's portion, and a prompt taken whole: bfloat16 logits at every position against the plain model."""
    cfg = LONG[name]
    g = torch.Generator().manual_seed(5)
    a = torch.randint(0, cfg["vocab_size"], (2640,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab_size"], (2300,), generator=g).tolist()
    steps = [
        {"entries": [{"id": "a", "tokens": a[:2048], "want": [0, 1, 777, 2047]}], "end": []},
        {"entries": [{"id": "a", "tokens": a[2048:2560], "want": list(range(0, 512, 37)) + [511]}], "end": []},
        {"entries": [{"id": "a", "tokens": a[2560:2600], "want": list(range(40))}], "end": []},
    ]
    # a's last 40 tokens one by one, all but the last beside a portion of b
    cuts = [0, 300, 812, 1100] + list(range(1132, 2300, 32))[:35] + [2300]           # 39 portions
    for i in range(40):
        entries, end = [{"id": "a", "tokens": a[2600 + i:2601 + i], "want": [0]}], []
        if i + 1 < len(cuts):
            lo, hi = cuts[i], cuts[i + 1]
            entries.insert(0, {"id": "b", "tokens": b[lo:hi], "want": [0, hi - lo - 1]})
            end += ["b"] if hi == len(b) else []
        steps.append({"entries": entries, "end": end + (["a"] if i == 39 else [])})
    steps.append({"entries": [{"id": "c", "tokens": b[:2300], "want": [5, 1000, 2299]}], "end": ["c"]})
    pages = tu.max_live_tokens(steps) // page + 3
    eng, w = make_engine(cfg, 9, page, pages, "bfloat16", max_seqs=4, budget=4096)
    plans = []
    inner = eng.ops.attention_plan
    eng.ops.attention_plan = lambda *args, **kw: plans.append(inner(*args, **kw)) or plans[-1]
    try:
        got = tu.run_steps(eng, steps)
    finally:
        eng.ops.attention_plan = inner
    assert eng.ops.tc_error() == 0
    kinds = {(k, n > 1) for k, n, _ in plans}
    # with 8 heads the row tiles of a portion fill less than half of the GPU: the one-tile kernel takes the long portion
    # uncut and the shorter ones behind it with their key range cut over CTAs; with 64 heads the long portions run uncut
    # on the two-tile kernel
    if name in ("h64", "h128w"):
        assert ("tcpp", False) in kinds, kinds
    else:
        assert ("tc", False) in kinds and (("tc", True) in kinds or ("tcpp", True) in kinds), kinds
    exp = {"a": plain_forward(cfg, w, a), "b": plain_forward(cfg, w, b)}
    exp["c"] = exp["b"]
    bad = tu.first_wrong(got, exp, TOL["bfloat16"])
    assert bad is None, f"first wrong place {bad}"


# ------------------------------------------------------------------------------------------ preemption
def test_preemption_by_recompute_on_the_gpu():
    """A pool so small that running requests are thrown out and prefilled again: greedy tokens in float32 equal
    plain greedy decoding; sampled tokens equal those of the same requests on a pool with room for all."""
    cfg = TINY_A
    reqs = list(requests_for(cfg, (5, 17, 30, 9), 3).values())
    new = 24
    eng, w = make_engine(cfg, SEEDS["A"], 4, 28, "float32", max_seqs=4, budget=16, graphs=True, cudagraph_batch_sizes=[1, 2, 4])
    outs = eng.generate(reqs, SamplingParams(max_new_tokens=new, greedy=True, ignore_eos=True))
    assert eng.stats()["preemptions"] > 0
    eng.manager.check()
    assert eng.manager.num_free_pages == eng.manager.num_usable_pages
    for prompt, out in zip(reqs, outs):
        assert out == plain_greedy(cfg, w, prompt, new)
    params = [SamplingParams(max_new_tokens=new, temperature=0.9, top_k=40, seed=50 + i, ignore_eos=True) for i in range(4)]
    before = eng.stats()["preemptions"]
    tight = eng.generate(reqs, params)
    assert eng.stats()["preemptions"] > before
    roomy, _ = make_engine(cfg, SEEDS["A"], 4, 80, "float32", max_seqs=4, budget=16, weights=w)
    assert tight == roomy.generate(reqs, params) and roomy.stats()["preemptions"] == 0
    eng.manager.check()
    assert eng.manager.num_free_pages == eng.manager.num_usable_pages


def test_requests_arriving_between_steps_with_everything_switched_on():
    """The continuous loop as a caller drives it: ``add_request`` between calls of ``step`` until ``has_unfinished`` says
    no, with captured decode steps, repeated layouts replayed, the next step launched ahead of the read and a pool that
    forces a request out now and then.  Twenty requests arrive at random steps; every one's greedy tokens equal plain
    greedy decoding (float32), and the pool is whole at the end."""
    import random
    cfg = TINY_B
    rng = random.Random(11)
    g = torch.Generator().manual_seed(11)
    reqs, arrive, t = [], [], 0
    for i in range(20):
        n = rng.choice([1, 2, 3, 7, 16, 17, 33, 40, 64, 71])
        reqs.append((torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist(), rng.randint(1, 24)))
        arrive.append(t)
        t += rng.choice([0, 0, 1, 2, 5, 9])
    eng, w = make_engine(cfg, SEEDS["B"], PAGE["B"], 18, "float32", max_seqs=4, budget=24, graphs=True, cudagraph_batch_sizes=[1, 2, 4])
    assert eng.engine_config.pipelined_decode and eng.engine_config.capture_repeated_steps
    out, ids, nxt, step = {}, {}, 0, 0
    while nxt < len(reqs) or eng.has_unfinished():
        while nxt < len(reqs) and arrive[nxt] <= step:
            rid = eng.add_request(reqs[nxt][0], SamplingParams(max_new_tokens=reqs[nxt][1], greedy=True, ignore_eos=True))
            ids[rid], out[nxt] = nxt, []
            nxt += 1
        if eng.has_unfinished():
            for rid, tok, _ in eng.step():
                out[ids[rid]].append(tok)
        step += 1
        assert step < 5000
    st = eng.stats()
    assert st["preemptions"] > 0 and st["step_graph_replays"] > 0 and st["finished"] == 20
    eng.manager.check()
    assert eng.manager.num_free_pages == eng.manager.num_usable_pages
    for i, (prompt, n) in enumerate(reqs):
        assert out[i] == plain_greedy(cfg, w, prompt, n), i


# ------------------------------------------------------------------------------------------ graphs, sampler in the graph, pipelining
@pytest.mark.parametrize("pipelined", [True, False])
def test_captured_pipelined_decode_in_bfloat16_against_the_plain_model(pipelined):
    """Head size 128, bfloat16, decode steps replayed from graphs with the sampling kernel inside and the next step
    launched before the host has read this one's tokens.  Requests end at different steps (the batch bucket
    changes), one context crosses 512 keys (the context bucket changes) and every request crosses pages.  Every
    generated token must be a maximum of the plain model's logits for the tokens before it, within the bfloat16
    tolerance of the row."""
    cfg = dict(architecture="mqa_gpt", vocab_size=211, d_model=256, num_layers=2, num_heads=2, num_kv_heads=1,
               hidden_size=320, max_seq_len=640, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, dtype="float32")
    from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig
    from tiny_transformer_inference_engine_b200.weights import random_tensors
    mc = ModelConfig.from_dict(cfg)
    w = random_tensors(mc, 21, std=0.08, perturb_norms=True)
    ec = EngineConfig(dtype="bfloat16", device=DEV, use_cuda_graphs=True, pipelined_decode=pipelined,
                      cache=CacheConfig(block_size=16, num_gpu_blocks=120),
                      sched=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=512, cudagraph_batch_sizes=[1, 2, 4]))
    eng = Engine(mc, w, ec)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 211, (n,), generator=g).tolist() for n in (490, 60, 200)]
    new = [48, 20, 33]
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=n, greedy=True, ignore_eos=True) for n in new])
    assert eng.stepper.counters["graph_replays"] >= 40
    assert {k[0] for k in eng.stepper._graphs} == {1, 2, 4}                                                   # batch buckets
    assert {k[1] for k in eng.stepper._graphs} == {512, 640}                                                   # context buckets
    assert eng.ops.tc_error() == 0
    for prompt, out, n in zip(prompts, outs, new):
        assert len(out) == n
        logits = plain_forward(cfg, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= TOL["bfloat16"] * float(row.abs().max()), (len(prompt), i)


# ------------------------------------------------------------------------------------------ sampled workload, token by token
def test_sampled_tokens_equal_the_plain_sampler_token_by_token():
    """BASELINE's second tiny workload: four prompts prefilled under a 16-token budget beside the decoded tokens of
    the others, temperature 0.8, 24 tokens, float32.  Every token equals the one the plain sampler draws from the
    plain model's logits with the request's own random stream."""
    cfg = TINY_B
    eng, w = make_engine(cfg, SEEDS["B"], PAGE["B"], 80, "float32", budget=16)
    reqs = list(requests_for(cfg, (1, 9, 40, 71), 4).values())
    params = [SamplingParams(max_new_tokens=24, temperature=0.8, seed=100 + i, ignore_eos=True) for i in range(4)]
    outs = eng.generate(reqs, params)
    assert eng.stats()["steps"] > 24                                   # portions and decoded tokens were mixed
    plain = PlainOps()
    for prompt, out, p in zip(reqs, outs, params):
        toks = list(prompt)
        for draw, tok in enumerate(out):
            row = plain_forward(cfg, w, toks)[-1]
            probs = plain.filtered_probs(row, p.temperature, p.top_k, p.top_p)
            u = uniform_from_state(p.seed & 0xFFFFFFFF, p.seed >> 32, draw)
            cdf = torch.cumsum(probs, 0)
            x = u * float(cdf[-1])
            want = min(int(torch.searchsorted(cdf, torch.tensor(x, dtype=cdf.dtype), right=True)), int((probs > 0).nonzero().max()))
            if want != tok:
                # a draw that lands within rounding of a boundary of the distribution may fall on either side of it
                lo, hi = min(want, tok), max(want, tok)
                assert abs(x - float(cdf[lo])) < 1e-5 and float(cdf[hi - 1] - cdf[lo]) < 1e-5, (len(prompt), draw, want, tok)
            toks.append(tok)


# ------------------------------------------------------------------------------------------ command line with a model folder
def test_command_line_with_a_model_folder(tmp_path):
    import json, os, subprocess, sys
    from tiny_transformer_inference_engine_b200 import ModelConfig
    from tiny_transformer_inference_engine_b200.weights import write_random_model
    from safetensors.torch import load_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = write_random_model(ModelConfig.from_dict(TINY_A), 31, str(tmp_path / "model"), perturb_norms=True)
    w = load_file(os.path.join(folder, "model.safetensors"))
    prompts = [[1, 2, 3], [9, 8, 7, 6, 5, 200, 100]]
    cmd = [sys.executable, "-m", "tiny_transformer_inference_engine_b200", "--model", folder, "--tokens", "9", "--greedy",
           "--dtype", "float32", "--num-gpu-blocks", "16", "--ignore-eos"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    run = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [json.loads(l) for l in run.stdout.strip().split("\n")]
    assert [l["prompt_ids"] for l in lines] == prompts
    for l in lines:
        assert l["generated_ids"] == plain_greedy(TINY_A, w, l["prompt_ids"], 9)


# ------------------------------------------------------------------------------------------ bounded waits
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    from tiny_transformer_inference_engine_b200.ops import get_ops, KernelError
    import ctypes
    ops = get_ops(DEV)
    assert ops.tc_error() == 0
    # the host side alone: a failure word set, the next check raises and clears it
    ops._tc_words[0] = 3
    with pytest.raises(KernelError, match="gave up waiting"):
        ops.check_tc()
    assert not ops._tc_words.any()
    ops.check_tc()
    # the device side: a wait with a limit of about a millisecond on a barrier nobody arrives at
    fn = ops.lib.ttie_attn_tc_wait_selftest
    fn.argtypes, fn.restype = [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops._check(fn(2_000_000, 7, gave_up.data_ptr(), torch.cuda.current_stream().cuda_stream), "wait self-test")
    torch.cuda.synchronize()
    assert int(gave_up) == 1                                           # the kernel returned by itself, its wait having run out
    assert int(ops._tc_words[1]) == 7                                  # ... and left its code in the host's mirror
    with pytest.raises(KernelError, match="code 107"):
        ops.check_tc()
    assert ops.tc_error() == 0 and not ops._tc_words.any()
    with pytest.raises(KernelError, match="limit"):
        ops._check(fn(0, 7, gave_up.data_ptr(), None), "wait self-test")
    # the context is whole: a tensor-core attention launch right after it is right
    from test_gpu_kernels import attention_case, rel
    out, exp, _, _ = attention_case(ops, "bfloat16", 8, 1, 128, 64, [(300, 300), (700, 1)], plan=("tc", 1, 0))
    assert rel(out, exp) < 1.2e-2 and ops.tc_error() == 0


# ------------------------------------------------------------------------------------------ sizes refused when the engine is built
def test_sizes_the_kernels_do_not_take_are_refused_at_construction():
    from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig
    from tiny_transformer_inference_engine_b200.ops import KernelError
    import tiny_transformer_inference_engine_b200.weights as weights
    small = dict(TINY_A, d_model=40, num_heads=4)                      # head size 10
    wide = dict(TINY_A, d_model=640, num_heads=2)                      # head size 320
    calls = []
    inner = weights.loader.place
    weights.loader.place = lambda *a, **k: calls.append(1) or inner(*a, **k)
    try:
        for cfg, what in ((small, "head size 10"), (wide, "head size 320")):
            with pytest.raises(KernelError, match=what):
                Engine(ModelConfig.from_dict(cfg), {}, EngineConfig(dtype="float32", device=DEV))
    finally:
        weights.loader.place = inner
    assert not calls                                                   # refused before any weight was looked at


# ------------------------------------------------------------------------------------------ repeated step layouts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_step_layouts_are_replayed_from_graphs(dtype):
    """A long prompt fed in equal portions beside two decoding requests: from its second occurrence on, the step's
    layout is captured and replayed.  Logits at every wanted place against the plain model; the requests' lengths,
    pages and tokens differ from replay to replay, a page edge and a context bucket are crossed on the way."""
    cfg = dict(architecture="mqa_gpt", vocab_size=211, d_model=256, num_layers=2, num_heads=2, num_kv_heads=1,
               hidden_size=320, max_seq_len=2600, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, dtype="float32")
    eng, w = make_engine(cfg, 13, 16, 260, dtype, max_seqs=4, budget=64, graphs=True, cudagraph_batch_sizes=[1, 2, 4])
    assert eng.stepper.capture_repeated
    g = torch.Generator().manual_seed(6)
    a = torch.randint(0, 211, (2400,), generator=g).tolist()
    b = torch.randint(0, 211, (60,), generator=g).tolist()
    c = torch.randint(0, 211, (45,), generator=g).tolist()
    steps = [{"entries": [{"id": "b", "tokens": b[:20], "want": [19]}, {"id": "c", "tokens": c[:5], "want": [4]}], "end": []}]
    for i in range(40):                                              # portions of 48 tokens of a: contexts 48 .. 1920, beside one token of b and of c
        steps.append({"entries": [{"id": "a", "tokens": a[48 * i:48 * (i + 1)], "want": [0, 47]},
                                  {"id": "b", "tokens": b[20 + i:21 + i], "want": [0]},
                                  {"id": "c", "tokens": c[5 + i:6 + i], "want": [0]}],
                      "end": (["b", "c"] if i == 39 else [])})
    for i in range(10):                                              # then a alone in the same portions, across the 2,048-key bucket
        steps.append({"entries": [{"id": "a", "tokens": a[1920 + 48 * i:1920 + 48 * (i + 1)], "want": [47]}], "end": ["a"] if i == 9 else []})
    got = tu.run_steps(eng, steps)
    st = eng.stepper.counters
    assert st["step_graphs_captured"] == 3 and st["step_graph_replays"] == 38 + 0 + 6, st     # (a's portions alone: two context buckets, met 2 and 8 times)
    exp = {"a": plain_forward(cfg, w, a), "b": plain_forward(cfg, w, b), "c": plain_forward(cfg, w, c)}
    bad = tu.first_wrong(got, exp, TOL[dtype])
    assert bad is None, f"first wrong place {bad}"
    # no more graphs are kept than allowed, and a layout that never comes again is never captured
    assert len(eng.stepper._step_graphs) <= eng.stepper.max_step_graphs
