"""Dense SwiGLU feed-forward.

Reference (models/mlp.py:17-32): ``down(silu(gate(x)) * up(x))`` with
``silu(g) = g * sigmoid(g)`` evaluated in 32-bit (kernels/fused_swiglu/kernel.py:20-25),
three linears with bias iff ``bias``.  ``gate`` and ``up`` are fused at load into one
matrix ``[2F, d]`` (gate rows first) so one product feeds the activation kernel.
The width ``F`` is this part's parameter.
"""
from __future__ import annotations

import torch

from .base import FeedForward, ParamSpec, StepContext
from ..registry import register_part


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, prefix: str, d_model: int, hidden: int, bias: bool = False):
        super().__init__(prefix)
        self.d_model, self.hidden, self.bias = int(d_model), int(hidden), bool(bias)
        self.w_gu = self.b_gu = self.w_down = self.b_down = None

    def param_specs(self):
        d, F = self.d_model, self.hidden
        specs = {"gate_proj.weight": ParamSpec((F, d)), "up_proj.weight": ParamSpec((F, d)),
                 "down_proj.weight": ParamSpec((d, F))}
        if self.bias:
            specs.update({"gate_proj.bias": ParamSpec((F,)), "up_proj.bias": ParamSpec((F,)),
                          "down_proj.bias": ParamSpec((d,))})
        return specs

    def load(self, params):
        self.w_gu = torch.cat([params["gate_proj.weight"], params["up_proj.weight"]], dim=0).contiguous()
        self.w_down = params["down_proj.weight"].contiguous()
        if self.bias:
            self.b_gu = torch.cat([params["gate_proj.bias"], params["up_proj.bias"]], dim=0).contiguous()
            self.b_down = params["down_proj.bias"].contiguous()

    def product_weights(self):
        return [self.w_down]                     # (gate/up beyond 8 rows is the library's product plus the activation kernel)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = self.ops.linear_swiglu(x, self.w_gu, self.b_gu, self.hidden)        # [T, F]
        return self.ops.linear(act, self.w_down, self.b_down, partial_ok=True)
