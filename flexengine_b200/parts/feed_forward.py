"""Dense SwiGLU feed-forward: down( silu(gate(h)) * up(h) ).

Formula: tests/unit/test_synthetic_qwen.py:30-36 of the reference (its product code
calls the module opaquely, src/flexengine/inference/models/qwen2.py:130).  gate and up
are held as one [2I, H] matrix so that one product feeds the activation kernel.
"""
from __future__ import annotations

from .base import FeedForward, register_feed_forward


class SwiGLU(FeedForward):
    takes_prenormed = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.gate_up_weight = None
        self.down_weight = None

    def parameter_shapes(self) -> dict:
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_up.weight": ((2 * i, h), "matrix"), "down.weight": ((h, i), "matrix")}

    def reads_first(self):
        return self.gate_up_weight

    def forward(self, ctx, h, follow=None):
        act = ctx.ops.linear_swiglu(h, self.gate_up_weight, self.intermediate_size)
        if follow is not None:
            return ctx.ops.linear(act, self.down_weight, follow=follow)
        return ctx.ops.linear(act, self.down_weight)


register_feed_forward("swiglu", SwiGLU)
