"""Replay on the GPU through the engine's own cache and kernels, in 32-bit and in bfloat16:
each request whole; most of it in one step and the last 32 tokens one by one; in portions of
changing size down to two tokens; mixed, up to four live requests with so few pages that they
are used again.  All compared with the plain model."""
import pytest
import torch

from plain_model import plain_forward
from tiny_configs import TINY_A, TINY_B, TINY_C, SEEDS, PAGE
import trace_util as tu
from gpu_util import make_engine, requests_for, TOL

pytestmark = pytest.mark.gpu

CASES = [("A", TINY_A, (5, 17, 33, 64, 48, 21)), ("B", TINY_B, (1, 9, 40, 71, 128, 100)),
         ("C", TINY_C, (300, 640, 77, 513, 130))]
MODES = {"whole": tu.whole, "decode": tu.prefill_then_decode, "portions": tu.portions, "mixed": tu.mixed}
_expected = {}


def expected_for(name, cfg, w, reqs):
    if name not in _expected:
        _expected[name] = {rid: plain_forward(cfg, w, toks) for rid, toks in reqs.items()}
    return _expected[name]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("name,cfg,lens", CASES)
def test_replay(name, cfg, lens, mode, dtype):
    reqs = requests_for(cfg, lens, 5)
    steps = MODES[mode](reqs)
    pages = tu.max_live_tokens(steps) // PAGE[name] + 1
    eng, w = make_engine(cfg, SEEDS[name], PAGE[name], pages, dtype)
    exp = expected_for(name, cfg, w, reqs)
    got = tu.run_steps(eng, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    bad = tu.first_wrong(got, exp, TOL[dtype])
    worst, where = tu.worst_relative(got, exp)
    assert bad is None, f"first wrong place {bad}; worst {worst} at {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decode(dtype):
    """The first tokens of a sequence one by one from an empty cache, and long decoding."""
    cfg, name = TINY_C, "C"
    reqs = requests_for(cfg, (400,), 9)
    toks = reqs["r0"]
    steps = [{"entries": [{"id": "r0", "tokens": toks[i:i + 1], "want": [0]}], "end": ["r0"] if i == len(toks) - 1 else []}
             for i in range(len(toks))]
    eng, w = make_engine(cfg, SEEDS[name], PAGE[name], 640 // PAGE[name] + 1, dtype)
    exp = {"r0": plain_forward(cfg, w, toks)}
    got = tu.run_steps(eng, steps)
    bad = tu.first_wrong(got, exp, TOL[dtype])
    assert bad is None, f"first wrong place {bad}"
