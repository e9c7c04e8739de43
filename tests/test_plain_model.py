"""The plain implementation against the committed logits of the reference's own classes, and
its own consistency (float64 vs float32, sampling filters)."""
import os

import pytest
import torch

from plain_model import (plain_forward, plain_rope, plain_rope_tables, plain_top_k, plain_top_p,
                         plain_sample_probs, plain_greedy, plain_attention)
from plain_ops import PlainOps, philox4x32
from tiny_transformer_inference_engine_b200.config import ModelConfig
from tiny_transformer_inference_engine_b200.weights import random_tensors

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_logits.pt")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_equals_reference_logits(name):
    rec = torch.load(GOLDEN)[name]
    cfg = rec["config"]
    w = random_tensors(ModelConfig.from_dict(cfg), rec["seed"], perturb_norms=True)
    for prompt, ref in zip(rec["prompts"], rec["logits"]):
        mine = plain_forward(cfg, w, prompt)
        assert ((mine - ref).abs().max() / ref.abs().max()).item() < 2e-6


def test_float64_agrees():
    rec = torch.load(GOLDEN)["B"]
    cfg = rec["config"]
    w = random_tensors(ModelConfig.from_dict(cfg), rec["seed"], perturb_norms=True)
    p = rec["prompts"][2]
    a, b = plain_forward(cfg, w, p), plain_forward(cfg, w, p, dtype=torch.float64)
    assert ((a.double() - b).abs().max() / b.abs().max()).item() < 1e-5


def test_rope_pairs():
    x = torch.arange(8.0).view(1, 1, 8)
    cos, sin = plain_rope_tables(8, [3], 10000.0)
    y = plain_rope(x, cos, sin)
    th = 3.0 * 1.0 / (10000.0 ** (torch.arange(0, 8, 2).float() / 8))
    assert torch.allclose(y[0, 0, 2], x[0, 0, 2] * th[1].cos() - x[0, 0, 3] * th[1].sin())
    assert torch.allclose(y[0, 0, 3], x[0, 0, 2] * th[1].sin() + x[0, 0, 3] * th[1].cos())
    z = plain_rope(x, cos, sin, style="half")
    assert torch.allclose(z[0, 0, 1], x[0, 0, 1] * th[1].cos() - x[0, 0, 5] * th[1].sin())


def test_attention_is_causal_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 2, 4), torch.randn(6, 1, 4), torch.randn(6, 1, 4)
    o = plain_attention(q, k, v, 0.5)
    assert torch.allclose(o[0, 0], v[0, 0])                       # the first token sees only itself
    v2 = v.clone(); v2[5] += 1.0
    assert torch.equal(plain_attention(q, k, v2, 0.5)[:5], o[:5])  # a later key changes nothing earlier
    ow = plain_attention(q, k, v, 0.5, window=1)
    assert torch.allclose(ow[:, 0], v[:, 0])


def test_sampling_filters():
    # the reference's own test cases in spirit (tests/test_sampling.py:6-58)
    logits = torch.tensor([[1.0, 3.0, 2.0, 3.0, 0.0]])
    assert plain_greedy(logits).item() == 1
    k2 = plain_top_k(logits, 2)
    assert torch.isfinite(k2).sum() == 2 and torch.isfinite(plain_top_k(logits, 3)).sum() == 3
    assert torch.equal(plain_top_k(logits, 0), logits) and torch.equal(plain_top_p(logits, 1.0), logits)
    probs = torch.tensor([[0.5, 0.3, 0.15, 0.05]]).log()
    kept = torch.isfinite(plain_top_p(probs, 0.7))
    assert kept.tolist() == [[True, True, False, False]]          # the token that crosses 0.7 stays
    assert torch.isfinite(plain_top_p(probs, 0.01)).tolist() == [[True, False, False, False]]
    p = plain_sample_probs(torch.tensor([[0.0, 1.0, 2.0]]), temperature=0.5, top_k=2)
    assert p[0, 0] == 0 and torch.allclose(p.sum(), torch.tensor(1.0))
    # the stand-in's filter equals the reference's order of operations when there are no ties
    row = torch.randn(200, generator=torch.Generator().manual_seed(1))
    a = PlainOps.filtered_probs(row, 0.7, 50, 0.9).float()
    b = plain_sample_probs(row[None], 0.7, 50, 0.9)[0]
    assert torch.allclose(a, b, atol=1e-6)


def test_philox_known_answer():
    # Random123 known-answer test for philox4x32-10
    assert philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert philox4x32([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
