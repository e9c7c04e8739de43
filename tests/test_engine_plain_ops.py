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
