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
