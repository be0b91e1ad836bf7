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

    def forward(self, ctx, h, follow=None, upcoming=None):
        if follow is None and upcoming is None:
            return ctx.ops.linear(ctx.ops.linear_swiglu(h, self.gate_up_weight, self.intermediate_size), self.down_weight)
        # a decode step on kernels that take the hints: each product is told which matrix is streamed after it
        act = ctx.ops.linear_swiglu(h, self.gate_up_weight, self.intermediate_size, upcoming=self.down_weight)
        return ctx.ops.linear(act, self.down_weight, follow=follow, upcoming=upcoming)


register_feed_forward("swiglu", SwiGLU)
