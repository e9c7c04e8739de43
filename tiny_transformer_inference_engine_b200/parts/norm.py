"""RMSNorm with the residual add fused in.

Formula of the reference (models/rmsnorm.py:12-18): ``x32 = float(x)``,
``y = x32 * rsqrt(mean(x32**2) + eps)``, ``out = (y * float(w)).to(dtype)`` -
eps inside the square root, weight multiplied in 32-bit before the cast.  The
reference fixes eps in code (models/rmsnorm.py:7) and never passes
``ModelConfig.rms_norm_eps``; here eps is this part's parameter.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Norm, ParamSpec
from ..registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, prefix: str, dim: int, eps: float):
        super().__init__(prefix)
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.dim,), storage="vector", init="ones")}

    def load(self, params):
        self.weight = params["weight"]

    def validate(self, ops, dtype, page_size):
        check = getattr(ops, "check_norm", None)
        if check is not None:
            check(dtype, self.dim)

    def add_norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = torch.empty(resid.shape, dtype=self.dtype, device=resid.device)
        self.ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)
        return out

    def norm_rows(self, resid, delta, rows, num_rows) -> torch.Tensor:
        out = torch.empty((num_rows, self.dim), dtype=self.dtype, device=resid.device)
        if num_rows:
            self.ops.rmsnorm_rows(resid, delta, rows, num_rows, self.weight, self.eps, out)
        return out
