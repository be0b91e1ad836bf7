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
        self._zeros = {}

    def sample(self, logits: torch.Tensor, temperatures, top_ks, seeds, draws) -> list:
        """logits float32 [R, V]; the other arguments are sequences of length R.  Returns R token ids."""
        return self.sample_on_device(logits, temperatures, top_ks, seeds, draws).tolist()

    def sample_on_device(self, logits: torch.Tensor, temperatures, top_ks, seeds, draws) -> torch.Tensor:
        """As ``sample`` but the token ids stay where the logits are (int32 [R]); nothing waits for the device."""
        if logits.dim() != 2 or logits.shape[0] != len(temperatures):
            raise ValueError("Expected logits [requests, vocab]")
        for t, k in zip(temperatures, top_ks):
            validate_sampling(t, k)
        dev = logits.device
        n = len(temperatures)
        if all(t == 0.0 for t in temperatures):
            # greedy rows need no parameters: zeros kept on the device, no copy per step
            key = (str(dev), n)
            if key not in self._zeros:
                self._zeros[key] = (torch.zeros(n, dtype=torch.float32, device=dev),
                                    torch.zeros(n, dtype=torch.int32, device=dev),
                                    torch.zeros(n, dtype=torch.int64, device=dev))
            temperature, top_k, zero64 = self._zeros[key]
            return self.ops.sample(logits, temperature, top_k, zero64, zero64)
        # one host buffer, one copy: [temperature bits | top_k | seed lo, hi | draw lo, hi] as 64-bit words
        packed = torch.empty((4, n), dtype=torch.int64, pin_memory=dev.type == "cuda")
        packed[0] = torch.tensor(list(temperatures), dtype=torch.float32).view(torch.int32).to(torch.int64)
        packed[1] = torch.tensor(list(top_ks), dtype=torch.int64)
        packed[2] = torch.tensor(list(seeds), dtype=torch.int64)
        packed[3] = torch.tensor(list(draws), dtype=torch.int64)
        on_dev = packed.to(dev, non_blocking=True)
        temperature = on_dev[0].to(torch.int32).view(torch.float32)
        top_k = on_dev[1].to(torch.int32)
        return self.ops.sample(logits, temperature, top_k, on_dev[2].contiguous(), on_dev[3].contiguous())
