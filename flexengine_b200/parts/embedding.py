"""Token embedding: the residual stream starts as the rows of a table.

x = embed_tokens.weight[ids] over the step's flattened tokens
(src/flexengine/inference/models/qwen2.py:90,94).  The stream is float32 whatever the table's dtype.
"""
from __future__ import annotations

from .base import Embedding, register_embedding


class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def forward(self, ctx):
        return ctx.ops.embedding(ctx.token_ids, self.weight)


register_embedding("token_table", TokenEmbedding)
