#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen2.5-7B shape, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line: ``value`` is decoded tokens per second at batch 8 (a step = one decode step of
every live request at a context of about 2,048 tokens, timed with CUDA events around K steps);
``e2e`` is the same through the engine's Python entry point (host token ids in, sampled token
ids out, every step); ``prefill`` is one 2,048-token prompt in one step; ``roofline`` is the
decode step's unavoidable HBM traffic over its time; ``points`` holds decode at batch 1 and 64.
Weights (15 GB) are larger than L2, so every step streams them from HBM again.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEVEN_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=3584,
               num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
               vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768,
               tie_word_embeddings=False, use_sliding_window=False, hidden_act="silu", eos_token_id=None)
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            flat = {}
            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat.setdefault("bf16_tflops_sustained", flat["bf16_tflops"])
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        def pump():
            for line in self.proc.stdout:
                self.samples.append((time.time(), [p.strip() for p in line.split(",")]))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        picked = [s for t, s in self.samples if any(a <= t <= b for a, b in windows)] or [s for _, s in self.samples]
        clocks, reasons, max_mhz = [], set(), None
        for s in picked:
            try:
                clocks.append(float(s[0]))
                max_mhz = float(s[1])
            except (ValueError, IndexError):
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_mhz,
                "reasons": sorted(reasons), "samples": len(picked)}


def linear_params(cfg):
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kd = cfg["num_key_value_heads"] * cfg["head_dim"]
    return cfg["num_hidden_layers"] * ((qd + 2 * kd) * h + qd * h + 3 * h * i)


def decode_bytes(cfg, batch, ctx):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    h, v = cfg["hidden_size"], cfg["vocab_size"]
    kd = cfg["num_key_value_heads"] * cfg["head_dim"]
    weights = 2 * (linear_params(cfg) + v * h) + 2 * batch * h           # matrices + lm head + embedding rows
    kv = batch * ctx * 2 * kd * cfg["num_hidden_layers"] * 2
    return weights + kv


def prefill_flops(cfg, tokens):
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    attention = cfg["num_hidden_layers"] * 2 * 2 * qd * tokens * (tokens + 1) / 2     # causal QK^T and PV
    return 2.0 * linear_params(cfg) * tokens + attention + 2.0 * cfg["vocab_size"] * cfg["hidden_size"]


def run_ours(args):
    import torch
    from flexengine_b200 import ops
    from flexengine_b200.cache import CacheManager
    from flexengine_b200.config import EngineConfig
    from flexengine_b200.engine import ModelRunner, StepEntry
    from flexengine_b200.engine.runtime import Engine
    from flexengine_b200.weights import random_model

    dev = "cuda:0"
    peaks, peak_source = load_peaks()
    cfg = dict(SEVEN_B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    torch.manual_seed(0)
    _typed, plan, model = random_model(cfg, seed=0, dtype="bfloat16", device=dev)
    gen = torch.Generator().manual_seed(1)
    vocab = cfg["vocab_size"]
    sampler = ClockSampler()
    sampler.start()
    windows = []

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

    def timed(fn, count):
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.time()
        launches0 = ops.launches
        start.record()
        for i in range(count):
            fn(i)
        end.record()
        torch.cuda.synchronize()
        windows.append((wall0, time.time()))
        return start.elapsed_time(end) / count, ops.launches - launches0

    # ---- prefill: one 2,048-token prompt in one step ----------------------------------------------
    def prefill_once(i):
        rid = f"p{i}"
        logits = runner.step([StepEntry(rid, prompt_ids, [PROMPT_LEN - 1])])
        greedy(logits)
        runner.finish(rid)
    prompt_ids = prompt()
    if args.profile != "decode":
        for w in range(max(args.warmup, 3)):
            prefill_once(-1 - w)
    prefill_ms, _ = timed(prefill_once, 3 if not args.profile else 0) if not args.profile else (1.0, 0)
    flops = prefill_flops(cfg, PROMPT_LEN)
    prefill = {"value": PROMPT_LEN / (prefill_ms / 1e3), "tokens": PROMPT_LEN, "ms": prefill_ms,
               "frac": flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12)}

    # ---- decode at a batch size ----------------------------------------------------------------------
    def decode(batch, steps, warmup):
        rids = [f"d{batch}_{i}" for i in range(batch)]
        for rid in rids:                                   # 2,048-token prompts, prefilled for real
            runner.step([StepEntry(rid, prompt(), [])])
        feed = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()
        def one(i, base=0):
            logits = runner.step([StepEntry(rid, [feed[base + i][j]], [0]) for j, rid in enumerate(rids)])
            greedy(logits)
        for w in range(warmup):
            one(w)
        ms, launches = timed(lambda i: one(i, warmup), steps)
        ctx = PROMPT_LEN + warmup + (steps + 1) / 2.0
        for rid in rids:
            runner.finish(rid)
        return ms, launches, ctx

    # ---- a mixed step: a portion of a prompt late in its context beside decoded tokens ----------------
    MIXED_PORTION, MIXED_AFTER, MIXED_DECODERS = 128, 3072, 7

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
            entries = [StepEntry("long", portion, [])] + [StepEntry(rid, [i + 1], [0]) for rid in rids]
            greedy(runner.step(entries))
            runner.finish("long")
        for w in range(3):
            one(w)
        if hook:
            return hook(one)
        ms, _ = timed(one, count)
        for rid in rids:
            runner.finish(rid)
        return ms

    warmup = max(args.warmup, 3)
    if args.profile == "mixed":
        def capture(one):
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            one(5)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        mixed(0, capture)
        sampler.stop()
        print(json.dumps({"profiled": args.profile}))
        return 0
    if args.profile:
        # for a profiler started with --profile-from-start off: only this region is captured
        if args.profile == "prefill":
            torch.cuda.profiler.start()
            prefill_once(100)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        else:
            rids = [f"x{i}" for i in range(args.batch)]
            for rid in rids:
                cache.reserve(rid, PROMPT_LEN)
                cache.commit(rid, PROMPT_LEN)            # the cache holds zeros: timing does not depend on values
            for i in range(3):
                greedy(runner.step([StepEntry(rid, [i + 1], [0]) for rid in rids]))
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            greedy(runner.step([StepEntry(rid, [7], [0]) for rid in rids]))
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        sampler.stop()
        print(json.dumps({"profiled": args.profile, "batch": args.batch}))
        return 0
    ms, launches, ctx = decode(args.batch, args.steps, warmup)
    value = args.batch / (ms / 1e3)
    achieved = decode_bytes(cfg, args.batch, ctx) / (ms / 1e3) / 1e9
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, _, _ = decode(b, max(4, args.steps // 2), 3)
            points[f"decode_b{b}"] = b / (pms / 1e3)
        # tokens a second of a step that brings 128 prompt tokens after 3,072 beside seven decoded tokens
        points["mixed_128_after_3072_plus_7"] = (MIXED_PORTION + MIXED_DECODERS) / (mixed(8) / 1e3)

    # ---- the same through the Python entry point: host tokens in, sampled tokens out, every step -----
    del runner, cache
    torch.cuda.empty_cache()
    engine = Engine.from_model(model, EngineConfig(
        model="random-7b-shape", device=dev, dtype="bfloat16", max_model_len=CONTEXT_LEN, max_num_seqs=args.batch,
        max_num_batched_tokens=PROMPT_LEN, prefill_chunk_size=PROMPT_LEN, kv_block_size=PAGE,
        kv_num_blocks=args.batch * CONTEXT_LEN // PAGE, max_output_tokens=4096, max_waiting=max(64, args.batch),
        scheduler_policy="fcfs", trace_steps=False, cuda_graph=args.cuda_graph))
    requests = [engine.submit(prompt(), max_tokens=warmup + args.steps + args.batch + 8) for _ in range(args.batch)]
    while any(len(r.generated_ids) < warmup for r in requests):
        engine.step()
    engine.drain()
    before = [len(r.generated_ids) for r in requests]
    h2d0 = getattr(engine.runner, "h2d_bytes", 0)

    def engine_step(i):
        # the engine launches a step before it has read the tokens of the one before; the last timed step
        # is followed by the read of its own tokens, so K steps and K reads lie inside the timed region
        engine.step()
        if i == args.steps - 1:
            engine.drain()
    e2e_ms, _ = timed(engine_step, args.steps)
    h2d = (getattr(engine.runner, "h2d_bytes", 0) - h2d0) / args.steps
    if engine.fault:
        raise RuntimeError(engine.fault)
    assert all(len(r.generated_ids) == n + args.steps for r, n in zip(requests, before)), "a timed step was not a full decode step"
    for r in requests:
        engine.cancel(r.request_id)
    e2e = {"value": args.batch / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 * args.batch}
    ops.check_status(dev)
    sampler.stop()

    line = {
        "metric": "decode tokens/s (Qwen2.5-7B shape, batch 8, 2,048-token prompts)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random token ids, random weights N(0, 0.02)",
        "impl": "ours",
        "config": {"model": "Qwen2.5-7B shape", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
                   "global_batch": args.batch, "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN, "kv_page": PAGE,
                   "parallelism": "single GPU", "cuda_graph": bool(args.cuda_graph),
                   "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": peak_source},
        "e2e": e2e,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"]},
        "points": points,
        "gpu_launches": launches,
        "clocks": sampler.summary(windows),
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    from baseline import reference_arm
    return reference_arm.main(args)


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=16)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (named in config)")
    p.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    p.add_argument("--profile", choices=["decode", "prefill", "mixed"], default=None,
                   help="run one decode step, one prefill or one mixed step between cudaProfilerStart/Stop and exit")
    p.add_argument("--cuda-graph", action=argparse.BooleanOptionalAction, default=True)
    args = p.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
