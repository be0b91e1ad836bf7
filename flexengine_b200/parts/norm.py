"""RMSNorm fused with the residual add.

y = w * (x * rsqrt(mean(x^2) + eps)), statistics and product in float32
(src/flexengine/inference/kernels/rmsnorm.py:24-32; called at
src/flexengine/inference/models/qwen2.py:67-71,97,130,134).  The residual stream is
float32; the pending branch output is added in the same kernel.
"""
from __future__ import annotations

import torch

from .base import Norm, register_norm


class RMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.hidden_size,), "vector")}

    def forward(self, ctx, residual, delta, rows=None, upcoming=None):
        return ctx.ops.add_rmsnorm(residual, delta, self.weight, self.eps, ctx.dtype, rows, upcoming=upcoming)

    def following(self, ctx, residual):
        # a decode step in bfloat16 on kernels that can: the product before this norm adds to the residual and
        # starts the norm, the product after it finishes it
        ops = ctx.ops
        if (getattr(ops, "FUSES_RESIDUAL_NORM", False) and ctx.dtype == torch.bfloat16
                and ctx.num_tokens <= ops.FUSED_NORM_MAX_ROWS and type(self).forward is RMSNorm.forward):
            return (residual, self.weight, self.eps)
        return None


register_norm("rmsnorm", RMSNorm)
