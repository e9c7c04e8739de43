import torch

from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig
from tiny_transformer_inference_engine_b200.weights import random_tensors

TOL = {"float32": 1e-4, "bfloat16": 4e-2}


def make_engine(cfg, seed, page, pages, dtype, max_seqs=4, budget=64, graphs=False, weights=None, **kw):
    mc = ModelConfig.from_dict(cfg)
    w = weights if weights is not None else random_tensors(mc, seed, perturb_norms=True)
    ec = EngineConfig(dtype=dtype, device="cuda:0", use_cuda_graphs=graphs,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                      sched=SchedulerConfig(max_num_seqs=max_seqs, max_num_batched_tokens=budget, **kw))
    return Engine(mc, w, ec), w


def requests_for(cfg, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
