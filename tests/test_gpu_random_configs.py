"""Configurations drawn at random: head sizes in steps of 16 up to 256, any number of heads and groups, widths and
vocabularies that are no power of two, every page size the cache takes.  Each runs a mixed schedule (up to four live
requests, portions beside decoded tokens, pages used again) in 32-bit and in bfloat16 against the plain model."""
import random

import pytest
import torch

from plain_model import plain_forward
import trace_util as tu
from gpu_util import make_engine, TOL

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    head = 16 * rng.randint(1, 16)
    kv = rng.choice([1, 1, 2, 3])
    heads = kv * rng.randint(1, 9 if head <= 128 else 4)
    cfg = dict(architecture="mqa_gpt", vocab_size=rng.randint(40, 2100), d_model=heads * head, num_layers=rng.randint(1, 3),
               num_heads=heads, num_kv_heads=kv, hidden_size=8 * rng.randint(3, 80), max_seq_len=rng.choice([96, 200, 333]),
               rope_theta=rng.choice([1e4, 5e5, 2.5e4]), rms_norm_eps=rng.choice([1e-5, 1e-6, 3e-4]), bias=rng.random() < 0.4,
               eos_token_id=None, dtype="float32")
    page = rng.choice([4, 8, 16, 32, 64, 128])
    lens = [rng.randint(1, cfg["max_seq_len"]) for _ in range(5)]
    return cfg, page, lens, rng.randint(0, 1 << 30)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_a_random_configuration(seed, dtype):
    cfg, page, lens, wseed = draw(seed)
    g = torch.Generator().manual_seed(wseed)
    reqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
    steps = tu.mixed(reqs, seed=seed)
    pages = tu.max_live_tokens(steps, rounding=page) // page + 1
    eng, w = make_engine(cfg, wseed, page, pages, dtype)
    exp = {rid: plain_forward(cfg, w, toks) for rid, toks in reqs.items()}
    got = tu.run_steps(eng, steps)
    assert eng.ops.tc_error() == 0
    bad = tu.first_wrong(got, exp, TOL[dtype])
    worst, where = tu.worst_relative(got, exp)
    assert bad is None, f"{cfg} page {page}: first wrong place {bad}; worst {worst} at {where}"
