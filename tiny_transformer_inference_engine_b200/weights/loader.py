"""Weights from safetensors, found by tensor name.

The reference loads a ``torch.save`` dict with ``load_state_dict(strict=True)``
(inference.py:87,109), stripping the ``_orig_mod.`` prefix that ``torch.compile``
leaves (inference.py:87, serving/paged_model.py:78).  Here a model folder holds
``config.json`` and one or more ``*.safetensors``; every tensor the model's parts
declare is looked up by name, and all problems (missing, unexpected, wrong shape,
wrong kind of dtype) are gathered into ONE error.

Storage rules: matrices are cast to the compute dtype (bfloat16 for a bfloat16 run);
a vector (norm weight) stored in 32-bit stays 32-bit; integer tables become int32.
A float32 run widens everything to 32-bit.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, List

import torch

_PREFIXES_TO_STRIP = ("_orig_mod.",)


class WeightError(RuntimeError):
    """Lists every missing, unexpected and mis-shaped tensor of a model folder."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_dtype):
        self.folder, self.missing, self.unexpected = folder, missing, unexpected
        self.wrong_shape, self.wrong_dtype = wrong_shape, wrong_dtype
        lines = [f"weights in {folder} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(f"{n} {list(s)}" for n, s in missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(f"{n} {list(s)}" for n, s in unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " +
                         ", ".join(f"{n} has {list(g)}, expected {list(e)}" for n, g, e in wrong_shape))
        if wrong_dtype:
            lines.append(f"  wrong dtype ({len(wrong_dtype)}): " +
                         ", ".join(f"{n} is {g}, expected {e}" for n, g, e in wrong_dtype))
        super().__init__("\n".join(lines))


def _strip(name: str) -> str:
    for p in _PREFIXES_TO_STRIP:
        name = name.replace(p, "")
    return name


def read_safetensors(folder: str) -> Dict[str, torch.Tensor]:
    """All tensors of the folder's safetensors files, on the CPU, as stored."""
    from safetensors import safe_open
    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors file in {folder}")
    out: Dict[str, torch.Tensor] = {}
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as f:
            for key in f.keys():
                name = _strip(key)
                if name in out:
                    raise RuntimeError(f"tensor {name!r} appears twice in {folder}")
                out[name] = f.get_tensor(key)
    return out


def place(stored: Dict[str, torch.Tensor], specs, compute_dtype: torch.dtype, device, folder="<memory>"):
    """Checks ``stored`` against ``specs`` (name -> (part, rel, ParamSpec)) and returns the
    tensors on ``device`` in the storage class each spec asks for."""
    missing, unexpected, wrong_shape, wrong_dtype = [], [], [], []
    for name, (_, _, ps) in specs.items():
        if name not in stored:
            missing.append((name, ps.shape))
            continue
        t = stored[name]
        if tuple(t.shape) != tuple(ps.shape):
            wrong_shape.append((name, tuple(t.shape), tuple(ps.shape)))
        if ps.storage == "table":
            if t.dtype.is_floating_point:
                wrong_dtype.append((name, str(t.dtype), "an integer type"))
        elif not t.dtype.is_floating_point:
            wrong_dtype.append((name, str(t.dtype), "a floating type"))
    for name, t in stored.items():
        if name not in specs:
            unexpected.append((name, tuple(t.shape)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(folder, sorted(missing), sorted(unexpected), sorted(wrong_shape), sorted(wrong_dtype))

    placed = {}
    for name, (_, _, ps) in specs.items():
        t = stored[name]
        if ps.storage == "table":
            t = t.to(torch.int32)
        elif ps.storage == "vector":
            # stored in 32-bit stays so; narrower storage is widened only for a 32-bit run
            if compute_dtype == torch.float32 or t.dtype == torch.float32:
                t = t.to(torch.float32)
            else:
                t = t.to(compute_dtype)
        else:
            t = t.to(compute_dtype)
        placed[name] = t.to(device).contiguous()
    return placed


def load_folder(folder: str, specs, compute_dtype: torch.dtype, device):
    return place(read_safetensors(folder), specs, compute_dtype, device, folder)
