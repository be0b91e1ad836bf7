"""The headline workload: decode and prefill throughput on the Qwen2.5-7B shape with random bfloat16 weights.

``value`` is decoded tokens per second at batch 8 (a step = one decode step of every live request at a context of
about 2,048 tokens, CUDA events around K steps); ``e2e`` is the same through ``Engine.step`` (host token ids in,
sampled token ids out, every step); ``prefill`` is one 2,048-token prompt in one step; ``roofline`` is the decode
step's unavoidable HBM traffic over its time; ``points`` holds decode at batch 1 and 64 and a mixed step.  The
weights (15 GB) are larger than L2, so every step streams them from HBM again.
"""
from __future__ import annotations

import json

from .clocks import ClockSampler, load_peaks
from .shapes import CONTEXT_LEN, PAGE, PROMPT_LEN, SHAPES, decode_bytes, flat_config, prefill_flops
from .timing import Timer

MIXED_PORTION, MIXED_AFTER, MIXED_DECODERS = 128, 3072, 7


def run(args) -> int:
    import torch
    from .. import ops
    from ..cache import CacheManager
    from ..config import EngineConfig
    from ..engine import ModelRunner, StepEntry
    from ..engine.runtime import Engine
    from ..weights import random_model

    dev = "cuda:0"
    peaks, peak_source = load_peaks(args.peaks)
    cfg = dict(SHAPES[args.shape])
    shape_name = f"Qwen2.5-{args.shape.upper()} shape"
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    torch.manual_seed(0)
    _typed, plan, model = random_model(cfg, seed=0, dtype="bfloat16", device=dev)
    gen = torch.Generator().manual_seed(1)
    vocab = cfg["vocab_size"]
    sampler = ClockSampler().start()
    timer = Timer(ops)

    def prompt():
        return torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist()

    max_batch = max(args.batch, 64 if not args.skip_points else args.batch)
    cache = CacheManager(plan.cache_groups, max_batch * CONTEXT_LEN // PAGE, PAGE, max_batch, torch.bfloat16, dev)
    runner = ModelRunner(model, cache)
    if args.cuda_graph:
        runner.enable_decode_graphs(max_batch, CONTEXT_LEN)
    zeros = {}

    def greedy(logits):
        n = logits.shape[0]
        if n not in zeros:
            zeros[n] = (torch.zeros(n, device=dev), torch.zeros(n, dtype=torch.int32, device=dev),
                        torch.zeros(n, dtype=torch.int64, device=dev))
        t, k, z = zeros[n]
        return ops.sample(logits, t, k, z, z)

    # ---- prefill: one 2,048-token prompt in one step ----------------------------------------------
    prompt_ids = prompt()

    def prefill_once(i):
        rid = f"p{i}"
        greedy(runner.step([StepEntry(rid, prompt_ids, [PROMPT_LEN - 1])]))
        runner.finish(rid)

    # ---- decode at a batch size ----------------------------------------------------------------------
    def decode(batch, steps, warmup):
        rids = [f"d{batch}_{i}" for i in range(batch)]
        for rid in rids:                                   # 2,048-token prompts, prefilled for real
            runner.step([StepEntry(rid, prompt(), [])])
        feed = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()

        def one(i, base=0):
            greedy(runner.step([StepEntry(rid, [feed[base + i][j]], [0]) for j, rid in enumerate(rids)]))
        for w in range(warmup):
            one(w)
        ms, launches = timer.timed(lambda i: one(i, warmup), steps)
        ctx = PROMPT_LEN + warmup + (steps + 1) / 2.0
        for rid in rids:
            runner.finish(rid)
        return ms, launches, ctx

    # ---- a mixed step: a portion of a prompt late in its context beside decoded tokens ----------------
    def mixed(count, hook=None):
        """``count`` timed steps of 128 prompt tokens after 3,072 cached ones beside seven decoded tokens at 2,048.
        The cache holds zeros for what came before: the step's time does not depend on values."""
        rids = [f"m{i}" for i in range(MIXED_DECODERS)]
        for rid in rids:
            cache.reserve(rid, PROMPT_LEN)
            cache.commit(rid, PROMPT_LEN)
        portion = torch.randint(0, vocab, (MIXED_PORTION,), generator=gen).tolist()

        def one(i):
            cache.reserve("long", MIXED_AFTER)
            cache.commit("long", MIXED_AFTER)
            greedy(runner.step([StepEntry("long", portion, [])] + [StepEntry(rid, [i + 1], [0]) for rid in rids]))
            runner.finish("long")
        for w in range(3):
            one(w)
        if hook:
            return hook(one)
        ms, _ = timer.timed(one, count)
        for rid in rids:
            runner.finish(rid)
        return ms

    warmup = max(args.warmup, 3)
    if args.profile:
        # for a profiler started with --profile-from-start off: only one step is captured
        def captured(fn):
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            fn()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        if args.profile == "mixed":
            mixed(0, lambda one: captured(lambda: one(5)))
        elif args.profile == "prefill":
            for w in range(3):
                prefill_once(-1 - w)
            captured(lambda: prefill_once(100))
        else:
            rids = [f"x{i}" for i in range(args.batch)]
            for rid in rids:
                cache.reserve(rid, PROMPT_LEN)
                cache.commit(rid, PROMPT_LEN)            # the cache holds zeros: timing does not depend on values
            for i in range(3):
                greedy(runner.step([StepEntry(rid, [i + 1], [0]) for rid in rids]))
            captured(lambda: greedy(runner.step([StepEntry(rid, [7], [0]) for rid in rids])))
        sampler.stop()
        print(json.dumps({"profiled": args.profile, "batch": args.batch}))
        return 0

    for w in range(3):
        prefill_once(-1 - w)
    prefill_ms, _ = timer.timed(prefill_once, 5)
    flops = prefill_flops(cfg, PROMPT_LEN)
    prefill = {"value": PROMPT_LEN / (prefill_ms / 1e3), "tokens": PROMPT_LEN, "ms": prefill_ms,
               "frac": flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12)}

    ms, launches, ctx = decode(args.batch, args.steps, warmup)
    value = args.batch / (ms / 1e3)
    achieved = decode_bytes(cfg, args.batch, ctx) / (ms / 1e3) / 1e9
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, _, pctx = decode(b, max(4, args.steps // 2), warmup)
            points[f"decode_b{b}"] = b / (pms / 1e3)
            points[f"decode_b{b}_hbm_frac"] = decode_bytes(cfg, b, pctx) / (pms / 1e3) / 1e9 / peaks["hbm_gbs"]
        # tokens a second of a step that brings 128 prompt tokens after 3,072 beside seven decoded tokens
        points["mixed_128_after_3072_plus_7"] = (MIXED_PORTION + MIXED_DECODERS) / (mixed(8) / 1e3)

    kernels = None
    if args.kernels:
        from .kernels import kernel_table
        kernels = kernel_table(model, cfg, args.batch, PROMPT_LEN, peaks, timer)

    # ---- the same through the Python entry point: host tokens in, sampled tokens out, every step -----
    del runner, cache
    torch.cuda.empty_cache()
    engine = Engine.from_model(model, EngineConfig(
        model=f"random-{args.shape}-shape", device=dev, dtype="bfloat16", max_model_len=CONTEXT_LEN, max_num_seqs=args.batch,
        max_num_batched_tokens=PROMPT_LEN, prefill_chunk_size=PROMPT_LEN, kv_block_size=PAGE,
        kv_num_blocks=args.batch * CONTEXT_LEN // PAGE, max_output_tokens=4096, max_waiting=max(64, args.batch),
        scheduler_policy="fcfs", trace_steps=False, cuda_graph=args.cuda_graph))
    requests = [engine.submit(prompt(), max_tokens=warmup + args.steps + args.batch + 8) for _ in range(args.batch)]
    while any(len(r.generated_ids) < warmup for r in requests):
        engine.step()
    engine.drain()
    before = [len(r.generated_ids) for r in requests]
    h2d0 = engine.runner.h2d_bytes

    def engine_step(i):
        # the engine launches a step before it has read the tokens of the one before; the last timed step
        # is followed by the read of its own tokens, so K steps and K reads lie inside the timed region
        engine.step()
        if i == args.steps - 1:
            engine.drain()
    e2e_ms, _ = timer.timed(engine_step, args.steps)
    h2d = (engine.runner.h2d_bytes - h2d0) / args.steps
    if engine.fault:
        raise RuntimeError(engine.fault)
    assert all(len(r.generated_ids) == n + args.steps for r, n in zip(requests, before)), "a timed step was not a full decode step"
    for r in requests:
        engine.cancel(r.request_id)
    e2e = {"value": args.batch / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 * (args.batch + 1)}      # tokens and the status word
    ops.check_status(dev)
    sampler.stop()

    line = {
        "metric": f"decode tokens/s ({shape_name}, batch {args.batch}, 2,048-token prompts)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "config": flat_config(cfg, model=shape_name, layers_full=full_layers, global_batch=args.batch,
                              seq_len=CONTEXT_LEN, prompt_len=PROMPT_LEN, kv_page=PAGE, parallelism="single GPU",
                              cuda_graph=bool(args.cuda_graph), l2=f"inputs larger than L2 ({decode_bytes(cfg, 0, 0) / 1e9:.0f} GB of weights per step)",
                              peaks=peak_source),
        "e2e": e2e,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"]},
        "points": points,
        "gpu_launches": launches,
        "clocks": sampler.summary(timer.windows),
    }
    if kernels is not None:
        line["kernels"] = kernels
    print(json.dumps(line))
    return 0
