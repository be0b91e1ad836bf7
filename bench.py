#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen2.5-7B shape, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...] [--kernels]

The measurements themselves are a program of the package (``flexengine bench``, flexengine_b200/bench/); this file
is its entry point at the root of the checkout: it points it at the measured peaks beside it and gives it the
reference arm (``--impl reference``: the unmodified reference under baseline/_ref, see baseline/reference_arm.py),
which is no part of the package.  One JSON line on standard output.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def reference_arm(args) -> int:
    from baseline import reference_arm as arm
    return arm.main(args)


def main() -> int:
    from flexengine_b200.bench import main as bench_main
    argv = sys.argv[1:]
    peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if "--peaks" not in argv and os.path.isfile(peaks):
        argv = argv + ["--peaks", peaks]
    return bench_main(argv, reference_arm=reference_arm)


if __name__ == "__main__":
    sys.exit(main())
