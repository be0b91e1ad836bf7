"""Vocabulary head: float32 logits of the rows that are wanted.

logits = x_last lm_head.weight^T, no bias (src/flexengine/inference/models/qwen2.py:131-136); tied
embeddings bind ``weight`` to the embedding table's storage.
"""
from __future__ import annotations

from .base import Head, register_head


class LinearHead(Head):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def forward(self, ctx, h):
        return ctx.ops.linear(h, self.weight, None, out_float32=True)


register_head("linear", LinearHead)
