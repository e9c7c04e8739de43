"""Random-weights mode: writes a model folder from a configuration and a seed.

Every matrix, embedding and bias is N(0, std) from a CPU ``torch.Generator`` seeded
with ``seed``, drawn in the sorted order of the tensor names so that the same
(config, seed) always gives the same bits; integer tables follow the rule their ``ParamSpec`` names; norm weights are ``1 + N(0, std)`` when
``perturb_norms`` is set (so a test sees the norm weight act) and 1 otherwise, which
is the reference's initialisation (models/rmsnorm.py:9).
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..config import ModelConfig
from ..registry import model_spec

_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def random_tensors(config: ModelConfig, seed: int, std: float = 0.02, perturb_norms: bool = False,
                   store_dtype: str = "float32", device="cpu") -> Dict[str, torch.Tensor]:
    """``device="cpu"`` (the default) gives bits that depend only on (config, seed); another
    device draws there with that device's generator - quicker for models of billions of
    parameters, and different bits."""
    from ..models.model import Model
    model = Model(model_spec(config))
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    dt = _STORE[store_dtype]
    out = {}
    specs = model.param_specs()
    for name in sorted(specs):
        ps = specs[name][2]
        if ps.storage == "table":
            # integer tables: uniform in [0, high), or 0, 1, 2, ... along the last dimension, or zeros
            if ps.init == "randint" and ps.high:
                t = torch.randint(0, int(ps.high), ps.shape, generator=gen, device=device)
            elif ps.init == "arange":
                t = torch.arange(ps.shape[-1], device=device).expand(ps.shape)
            elif ps.init == "zeros":
                t = torch.zeros(ps.shape, dtype=torch.int64, device=device)
            else:
                raise ValueError(f"integer table {name}: its ParamSpec must say init='randint' (with high=), 'arange' or 'zeros'")
            out[name] = t.to(torch.int32).contiguous()
            continue
        if ps.init == "normal":
            t = torch.randn(ps.shape, generator=gen, dtype=torch.float32, device=device) * std
        elif ps.init == "ones":
            t = torch.ones(ps.shape, dtype=torch.float32, device=device)
            if perturb_norms:
                t = t + torch.randn(ps.shape, generator=gen, dtype=torch.float32, device=device) * std
        else:
            t = torch.zeros(ps.shape, dtype=torch.float32, device=device)
        # vectors keep 32-bit storage (they are few and their precision matters)
        out[name] = t.to(torch.float32 if ps.storage == "vector" else dt).contiguous()
    return out


def write_random_model(config: ModelConfig, seed: int, folder: str, std: float = 0.02,
                       perturb_norms: bool = False, store_dtype: str = "float32") -> str:
    """Writes ``config.json`` and ``model.safetensors`` into ``folder``; returns ``folder``."""
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    tensors = random_tensors(config, seed, std, perturb_norms, store_dtype)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"seed": str(int(seed))})
    return folder
