"""Decode and prefill on the 7B shape at further context lengths and batch sizes than the headline run.

Decode: a step from the CUDA graph at batch 1, 8 and 64 with 2,048, 8,192 and 32,768 tokens of context each (batch 64
up to 8,192; the
cache is reserved and committed without running the prompts: it holds zeros, and the time of a step does not depend on
the values); bytes are every weight once and the live requests' keys and values.  Prefill: one prompt of 512 to
32,768 tokens in one step; flops count the causal attention.  One JSON line, every point flat under ``points``.
"""
from __future__ import annotations

import json

from .clocks import ClockSampler, load_peaks
from .shapes import PAGE, SEVEN_B, decode_bytes, flat_config, prefill_flops
from .timing import Timer

DECODE_CONTEXTS = (2048, 8192, 32768)
DECODE_BATCHES = (1, 8, 64)
PREFILL_LENGTHS = (512, 2048, 8192, 32768)
MAX_CACHED_TOKENS = 600_000        # 34 GB of keys and values on this shape: batch 64 is not run at 32,768 tokens


def run(args) -> int:
    import torch
    from .. import ops
    from ..cache import CacheManager
    from ..engine import ModelRunner, StepEntry
    from ..weights import random_model

    dev = "cuda:0"
    peaks, peak_source = load_peaks(args.peaks)
    cfg = dict(SEVEN_B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    _typed, plan, model = random_model(cfg, 0, "bfloat16", dev)
    timer = Timer(ops)
    sampler = ClockSampler()
    sampler.start()
    gen = torch.Generator().manual_seed(0)
    vocab = cfg["vocab_size"]
    points = {}
    steps, warmup = max(8, args.steps // 2), max(3, min(args.warmup, 8))

    for ctx in DECODE_CONTEXTS:
        limit = ctx + 64
        for batch in DECODE_BATCHES:
            if batch * ctx > MAX_CACHED_TOKENS:
                continue
            cache = CacheManager(plan.cache_groups, batch * (-(-limit // PAGE)), PAGE, batch, torch.bfloat16, dev)
            runner = ModelRunner(model, cache)
            if args.cuda_graph:
                runner.enable_decode_graphs(batch, limit)
            rids = [f"c{ctx}b{batch}r{i}" for i in range(batch)]
            for rid in rids:
                cache.reserve(rid, ctx)
                cache.commit(rid, ctx)
            feed = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()

            def one(i, base=0):
                runner.step([StepEntry(rid, [feed[base + i][j]], [0]) for j, rid in enumerate(rids)])
            for w in range(warmup):
                one(w)
            ms, _ = timer.timed(lambda i: one(i, warmup), steps)
            mean_ctx = ctx + warmup + (steps + 1) / 2.0
            gbs = decode_bytes(cfg, batch, mean_ctx) / (ms / 1e3) / 1e9
            key = f"decode_b{batch}_ctx{ctx}"
            points[key + "_ms"] = round(ms, 4)
            points[key + "_tok_s"] = round(batch / (ms / 1e3), 1)
            points[key + "_hbm_frac"] = round(gbs / peaks["hbm_gbs"], 4)
            del runner, cache
            torch.cuda.empty_cache()

    for length in PREFILL_LENGTHS:
        cache = CacheManager(plan.cache_groups, -(-length // PAGE) + 1, PAGE, 1, torch.bfloat16, dev)
        runner = ModelRunner(model, cache)
        ids = torch.randint(0, vocab, (length,), generator=gen).tolist()

        def once(i):
            runner.step([StepEntry(f"p{length}_{i}", ids, [length - 1])])
            runner.finish(f"p{length}_{i}")
        for w in range(2):
            once(-1 - w)
        ms, _ = timer.timed(once, 3)
        flops = prefill_flops(cfg, length)
        points[f"prefill_{length}_ms"] = round(ms, 3)
        points[f"prefill_{length}_tok_s"] = round(length / (ms / 1e3), 1)
        points[f"prefill_{length}_tensor_frac"] = round(flops / (ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)
        del runner, cache
        torch.cuda.empty_cache()

    ops.check_status(torch.device(dev))
    sampler.stop()
    headline = points["decode_b8_ctx32768_tok_s"]
    line = {"metric": "decode tokens/s (Qwen2.5-7B shape, batch 8, 32,768 tokens of context)", "value": headline,
            "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random token ids, random weights N(0, 0.02), a cache of zeros",
            "impl": "ours",
            "config": flat_config(cfg, model="Qwen2.5-7B shape", layers_full=full_layers, kv_page=PAGE, parallelism="single GPU",
                                  cuda_graph=bool(args.cuda_graph), peaks=peak_source),
            "points": points, "clocks": sampler.summary(timer.windows)}
    print(json.dumps(line))
    return 0
