"""Timing on the device: CUDA events on the launching stream, a synchronize on both sides."""
from __future__ import annotations

import time

import torch


class Timer:
    """Collects wall-clock windows of its timed regions, for the clock sampler to pick its samples from."""

    def __init__(self, ops):
        self.ops = ops
        self.windows = []

    def timed(self, fn, count: int):
        """(milliseconds per call, kernels of this package launched) over ``count`` calls of ``fn(i)``."""
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall = time.time()
        launches = self.ops.launches
        start.record()
        for i in range(count):
            fn(i)
        end.record()
        torch.cuda.synchronize()
        self.windows.append((wall, time.time()))
        return start.elapsed_time(end) / max(count, 1), self.ops.launches - launches
