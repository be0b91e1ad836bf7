"""``flexengine bench``: the measurements of this engine as a program of the package.

    flexengine bench [--workload decode|serve-1.5b|long-14b|lengths] [--steps K] [--warmup W] [--kernels] ...

``decode`` (the default) is the headline: decode tokens per second on the Qwen2.5-7B shape at batch 8 after
2,048-token prompts, with prefill, end-to-end, roofline and batch 1 / 64 beside it; ``--kernels`` adds a table of the
step's kernels with their achieved fraction of the measured peaks.  The other two workloads drive the whole engine
(scheduler, page pool, CUDA graphs, overlapped steps) on the 1.5B and 14B shapes.  Every run prints ONE JSON line.
The reference measures over HTTP (src/flexengine/research/benchmark/runner.py:26-105) and in process
(src/flexengine/research/profiling/engine.py:35-46); these run in process, on seeded random token ids.
"""
from __future__ import annotations

import argparse


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="flexengine bench", description="Measure the engine on one GPU; prints one JSON line")
    p.add_argument("--workload", choices=["decode", "serve-1.5b", "long-14b", "lengths"], default="decode")
    p.add_argument("--shape", choices=["7b", "1.5b", "14b"], default="7b",
                   help="the model shape of the decode workload (the headline is 7b)")
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64, help="timed decode steps (decode workload)")
    p.add_argument("--warmup", type=int, default=16,
                   help="untimed steps before the timed ones (after a prompt the first dozen decode steps run a few percent slow)")
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (both numbers are reported)")
    p.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64 and the mixed step")
    p.add_argument("--kernels", action="store_true", help="add the per-kernel table (decode workload)")
    p.add_argument("--profile", choices=["decode", "prefill", "mixed"], default=None,
                   help="run one step between cudaProfilerStart/Stop and exit (for a profiler started with the region off)")
    p.add_argument("--policy", choices=["fcfs", "decode_first", "slo_aware", "adaptive"], default="fcfs")
    p.add_argument("--cuda-graph", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--peaks", default=None, help="JSON file of measured peaks (default: MEASURED_PEAKS.json in the working directory)")
    return p


def main(argv=None, reference_arm=None) -> int:
    """``reference_arm``: a callable(args) -> int that runs the reference instead (``--impl reference``); the package
    itself holds none."""
    args = build_parser().parse_args(argv)
    if args.gpus != 1:
        print(f"this engine runs on one GPU: it has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    if args.impl == "reference":
        if reference_arm is None:
            print('{"impl": "reference", "unavailable": "no reference arm was given to this entry point"}')
            return 0
        return reference_arm(args)
    if args.workload == "serve-1.5b":
        from .serving import serve_small
        return serve_small(args)
    if args.workload == "long-14b":
        from .serving import long_context
        return long_context(args)
    if args.workload == "lengths":
        from .lengths import run as run_lengths
        return run_lengths(args)
    from .headline import run
    return run(args)
