"""Trace replay: feed given token ids through a model step by step and write the logits.

Nothing is sampled.  The program drives the framework's own loader, model, step function,
cache manager and kernels, the ones generation uses; it has no forward pass of its own.
Steps come as JSON lines on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian float32
[wanted, vocab].  After every step a line ``done <step>`` is printed and flushed.
(The reference has no token-level replay; its nearest analogue is the in-process step loop
of src/flexengine/research/profiling/engine.py:35-46.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 4


def build_runner(model_dir: str, dtype: str, max_tokens: int, device: str = "cuda:0", ops=None,
                 page_size: int = PAGE_SIZE, max_requests: int = MAX_LIVE_REQUESTS):
    from ..cache.manager import CacheManager
    from ..weights.loader import load_model
    from .step import ModelRunner
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    _typed, plan, model = load_model(model_dir, dtype, device)
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    # the pool holds exactly what the live requests may hold at any time, so pages are used again
    pages = max(1, -(-int(max_tokens) // page_size))
    cache = CacheManager(plan.cache_groups, pages, page_size, max_requests, torch_dtype, device)
    return ModelRunner(model, cache, ops=ops)


def replay(runner, lines, out_dir: str, report=None) -> int:
    """Run every step read from ``lines``.  Returns the number of steps run."""
    from .step import StepEntry
    os.makedirs(out_dir, exist_ok=True)
    count = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step_no = record["step"]
        entries = [StepEntry(str(e["id"]), [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in record.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits is not None and logits.numel():
                data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step_no}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step_no}.f32"))
            if runner.device.type == "cuda":
                runner.ops.check_status(runner.device)
        for rid in record.get("end", []):
            runner.finish(str(rid))
        count += 1
        if report is not None:
            report(step_no)
    return count


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description="Replay token ids step by step and write logits")
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="the most tokens that live requests hold at any time; the page pool is made for exactly "
                             "this many, in pages of 16 tokens, so pages are used again (a caller that rounds each "
                             "request up to a multiple of 64 has counted enough)")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    runner = build_runner(args.model, args.dtype, args.max_tokens, args.device)

    def report(step_no):
        sys.stdout.write(f"done {step_no}\n")
        sys.stdout.flush()

    replay(runner, sys.stdin, args.out, report)
    return 0
