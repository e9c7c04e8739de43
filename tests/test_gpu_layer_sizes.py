"""Logits at the layer sizes of the Llama-2-7B-with-one-kv-head configuration (width 4096, 32 heads of
128, SwiGLU 11008, vocabulary 32000; two layers so that the plain model stays quick), random weights:
float32 to 1e-4 and bfloat16, whole, in portions and decoded, against the plain model."""
import pytest
import torch

from plain_model import plain_forward
import trace_util as tu
from gpu_util import make_engine, TOL

from tiny_transformer_inference_engine_b200 import ModelConfig
from tiny_transformer_inference_engine_b200.weights import random_tensors

pytestmark = pytest.mark.gpu

CFG = dict(architecture="mqa_gpt", vocab_size=32000, d_model=4096, num_layers=2, num_heads=32, num_kv_heads=1,
           hidden_size=11008, max_seq_len=512, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, eos_token_id=None)
_cache = {}


def setup():
    if not _cache:
        w = random_tensors(ModelConfig.from_dict(CFG), 1, perturb_norms=True)
        g = torch.Generator().manual_seed(2)
        reqs = {"a": torch.randint(0, 32000, (150,), generator=g).tolist(), "b": torch.randint(0, 32000, (70,), generator=g).tolist()}
        _cache.update(w=w, reqs=reqs, exp={r: plain_forward(CFG, w, t) for r, t in reqs.items()})
    return _cache["w"], _cache["reqs"], _cache["exp"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "decode", "mixed"])
def test_layer_sizes(dtype, mode):
    w, reqs, exp = setup()
    steps = {"whole": tu.whole, "decode": tu.prefill_then_decode, "mixed": tu.mixed}[mode](reqs)
    eng, _ = make_engine(CFG, 1, 64, tu.max_live_tokens(steps) // 64 + 1, dtype, weights=w, budget=512)
    got = tu.run_steps(eng, steps)
    bad = tu.first_wrong(got, exp, TOL[dtype])
    worst, where = tu.worst_relative(got, exp)
    assert bad is None, f"first wrong place {bad}; worst {worst} at {where}"


OTHER = {
    # Falcon-7B widths in Llama style: 71 heads (no power of two) of 64, width 4544, vocabulary 65024
    "falcon": dict(architecture="mqa_gpt", vocab_size=65024, d_model=4544, num_layers=1, num_heads=71, num_kv_heads=1,
                   hidden_size=18176, max_seq_len=256, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False, eos_token_id=None),
    # Gemma-2B sizes: 8 heads of 256, width 2048, vocabulary 256000
    "gemma": dict(architecture="mqa_gpt", vocab_size=256000, d_model=2048, num_layers=1, num_heads=8, num_kv_heads=1,
                  hidden_size=16384, max_seq_len=256, rope_theta=10000.0, rms_norm_eps=1e-6, bias=False, eos_token_id=None),
}


@pytest.mark.parametrize("name", list(OTHER))
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_other_layer_sizes(name, dtype):
    """One layer at the Falcon-7B and Gemma-2B layer sizes: a prompt in portions, then decoded tokens."""
    cfg = OTHER[name]
    w = random_tensors(ModelConfig.from_dict(cfg), 3, perturb_norms=True)
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, cfg["vocab_size"], (90,), generator=g).tolist()
    exp = {"a": plain_forward(cfg, w, toks)}
    steps = [{"entries": [{"id": "a", "tokens": toks[:70], "want": [0, 33, 69]}], "end": []}]
    steps += [{"entries": [{"id": "a", "tokens": toks[i:i + 1], "want": [0]}], "end": ["a"] if i == 89 else []} for i in range(70, 90)]
    eng, _ = make_engine(cfg, 3, 16, 8, dtype, weights=w, budget=128)
    got = tu.run_steps(eng, steps)
    bad = tu.first_wrong(got, exp, TOL[dtype])
    assert bad is None, f"first wrong place {bad}"
