"""Choosing the next token from logits, for a batch of requests at once.

Greedy at temperature 0, otherwise temperature and optional top-k with a per-request
random stream (src/flexengine/engine/sampling/sampler.py:7-22; per-request seeds
src/flexengine/engine/runtime.py:112-116).  The reference draws on the CPU with one
``torch.Generator`` per request; here the draw is a kernel keyed by (request seed, number
of the draw), which gives the same property: a request's tokens do not depend on what
else is in the batch or on how the scheduler cut the work.
"""
from __future__ import annotations

import torch


def validate_sampling(temperature: float, top_k: int) -> None:
    if temperature < 0 or top_k < 0:
        raise ValueError("temperature and top_k must be >= 0")


class Sampler:
    def __init__(self, ops=None):
        if ops is None:
            from .. import ops as cuda_ops
            ops = cuda_ops
        self.ops = ops

    def sample(self, logits: torch.Tensor, temperatures, top_ks, seeds, draws) -> list:
        """logits float32 [R, V]; the other arguments are sequences of length R.  Returns R token ids."""
        if logits.dim() != 2 or logits.shape[0] != len(temperatures):
            raise ValueError("Expected logits [requests, vocab]")
        for t, k in zip(temperatures, top_ks):
            validate_sampling(t, k)
        dev = logits.device
        temperature = torch.tensor(list(temperatures), dtype=torch.float32, device=dev)
        top_k = torch.tensor(list(top_ks), dtype=torch.int32, device=dev)
        seed = torch.tensor(list(seeds), dtype=torch.int64, device=dev)
        draw = torch.tensor(list(draws), dtype=torch.int64, device=dev)
        return self.ops.sample(logits, temperature, top_k, seed, draw).tolist()
