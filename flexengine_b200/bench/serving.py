"""Two whole-engine workloads, through ``Engine.generate`` / ``Engine.step`` with host tokens in and out.

``serve-1.5b``: the Qwen2.5-1.5B shape, 64 concurrent requests with prompts of 16 to 1,024 random tokens and 256
output tokens each, chunked prefill under a 2,048-token budget.  ``long-14b``: the Qwen2.5-14B shape, 32 requests
with 8,192-token prompts and 128 greedy tokens each, the page pool sized to fill what memory the weights leave.
Both follow the in-process loop of the reference's profiler (src/flexengine/research/profiling/engine.py:35-46):
submit, step until every request has ended, report.  Wall-clock time with a synchronize on both sides: the host
is part of what is measured.
"""
from __future__ import annotations

import json
import time

from .clocks import ClockSampler, load_peaks
from .shapes import SHAPES, decode_bytes, flat_config, kv_bytes_per_token, prefill_flops


def _line(metric, value, unit, cfg, config, extra, sampler, windows):
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random token ids, random weights N(0, 0.02)",
            "impl": "ours", "config": flat_config(cfg, parallelism="single GPU", **config)}
    line.update(extra)
    line["clocks"] = sampler.summary(windows)
    return line


def serve_small(args) -> int:
    import torch
    from .. import ops
    from ..config import EngineConfig
    from ..engine.runtime import Engine
    from ..weights import random_model

    dev = "cuda:0"
    peaks, peak_source = load_peaks(args.peaks)
    cfg = dict(SHAPES["1.5b"])
    requests, outputs, budget, limit = 64, 256, 2048, 2048
    _typed, _plan, model = random_model(cfg, 0, "bfloat16", dev)
    engine = Engine.from_model(model, EngineConfig(
        model="random-1.5b-shape", device=dev, dtype="bfloat16", max_model_len=limit, max_num_seqs=requests,
        max_num_batched_tokens=budget, prefill_chunk_size=budget, kv_block_size=16, kv_num_blocks=requests * limit // 16,
        max_output_tokens=512, max_waiting=2 * requests, scheduler_policy=args.policy, trace_steps=False,
        cuda_graph=args.cuda_graph))
    gen = torch.Generator().manual_seed(3)
    sampler = ClockSampler().start()
    windows, runs = [], []
    for trial in range(max(1, args.warmup // 3) + 1):            # the first pass warms libraries and allocator up
        lengths = torch.randint(16, 1025, (requests,), generator=gen).tolist()
        prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
        steps0, launches0 = engine.step_index, ops.launches
        torch.cuda.synchronize()
        wall = time.time()
        t0 = time.perf_counter()
        outs = engine.generate(prompts, max_tokens=outputs)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        windows = [(wall, time.time())]
        made = sum(len(o.token_ids) for o in outs)
        runs.append(dict(seconds=seconds, prompt_tokens=sum(lengths), output_tokens=made, steps=engine.step_index - steps0,
                         launches=ops.launches - launches0))
    ops.check_status(dev)
    sampler.stop()
    last = runs[-1]
    mean_ctx = last["prompt_tokens"] / requests + outputs / 2
    floor_ms = decode_bytes(cfg, requests, mean_ctx) / (peaks["hbm_gbs"] * 1e9) * 1e3
    extra = {"steps": last["steps"], "warmup": len(runs) - 1, "ms_per_step": last["seconds"] * 1e3 / max(last["steps"], 1),
             "e2e": {"value": last["output_tokens"] / last["seconds"], "unit": "output tokens/s",
                     "h2d_bytes_per_step": None, "d2h_bytes_per_step": None, "note": "the timed region is Engine.generate itself"},
             "total_tokens_per_s": (last["output_tokens"] + last["prompt_tokens"]) / last["seconds"], "seconds": last["seconds"],
             "prompt_tokens": last["prompt_tokens"], "output_tokens": last["output_tokens"],
             "preemptions": engine.preemption_count, "pages_in_use_after": engine.cache.used_pages,
             "roofline": {"bound": "hbm", "unit": "ms per decode step of 64", "peak": floor_ms,
                          "achieved": last["seconds"] * 1e3 / max(last["steps"], 1),
                          "frac": floor_ms / (last["seconds"] * 1e3 / max(last["steps"], 1)),
                          "note": "all steps, prompt portions included, against the floor of a pure decode step"},
             "gpu_launches": last["launches"]}
    print(json.dumps(_line("output tokens/s (Qwen2.5-1.5B shape, 64 requests, prompts 16-1,024, 256 outputs, budget 2,048)",
                           last["output_tokens"] / last["seconds"], "tokens/s", cfg,
                           dict(model="Qwen2.5-1.5B shape", layers_full=cfg["num_hidden_layers"], global_batch=requests,
                                seq_len=limit, token_budget=budget, kv_page=16, policy=args.policy,
                                cuda_graph=bool(args.cuda_graph), peaks=peak_source), extra, sampler, windows)))
    return 0


def long_context(args) -> int:
    import torch
    from .. import ops
    from ..config import EngineConfig
    from ..engine.request import TERMINAL
    from ..engine.runtime import Engine
    from ..weights import random_model

    dev = "cuda:0"
    peaks, peak_source = load_peaks(args.peaks)
    cfg = dict(SHAPES["14b"])
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    batch, prompt_len, outputs = 32, 8192, 128
    _typed, _plan, model = random_model(cfg, 0, "bfloat16", dev)
    engine = Engine.from_model(model, EngineConfig(
        model="random-14b-shape", device=dev, dtype="bfloat16", max_model_len=prompt_len + outputs + 16, max_num_seqs=batch,
        max_num_batched_tokens=prompt_len, prefill_chunk_size=prompt_len, kv_block_size=16, kv_num_blocks=0,
        kv_memory_fraction=0.9, max_output_tokens=512, max_waiting=2 * batch, scheduler_policy="fcfs", trace_steps=False,
        cuda_graph=args.cuda_graph))
    pages = engine.cache.total_pages
    engine.generate([[1, 2, 3] * 1000], max_tokens=4)              # warms libraries, scratch and allocator up
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab_size"], (prompt_len,), generator=gen).tolist() for _ in range(batch)]
    sampler = ClockSampler().start()
    requests = [engine.submit(p, max_tokens=outputs) for p in prompts]
    launches0 = ops.launches
    torch.cuda.synchronize()
    wall0, t0 = time.time(), time.perf_counter()
    prefill_steps = 0
    while any(r.in_prefill or not r.generated_ids for r in requests):
        engine.step()
        prefill_steps += 1
    engine.drain()
    torch.cuda.synchronize()
    wall1, t1 = time.time(), time.perf_counter()
    decode_steps = 0
    while any(r.state not in TERMINAL for r in requests):
        if not engine.step():
            break
        decode_steps += 1
    engine.drain()
    torch.cuda.synchronize()
    wall2, t2 = time.time(), time.perf_counter()
    if engine.fault:
        raise RuntimeError(engine.fault)
    ops.check_status(dev)
    sampler.stop()
    made = sum(len(r.generated_ids) for r in requests)
    decode_ms = (t2 - t1) * 1e3 / max(decode_steps, 1)
    step_bytes = decode_bytes(cfg, batch, prompt_len + outputs / 2)
    prefill_rate = prefill_flops(cfg, prompt_len) * batch / (t1 - t0)
    extra = {"steps": decode_steps, "warmup": 1, "ms_per_step": decode_ms,
             "e2e": {"value": (made - batch) / (t2 - t1), "unit": "tokens/s", "h2d_bytes_per_step": None,
                     "d2h_bytes_per_step": 4 * (batch + 1), "note": "the timed region is Engine.step itself"},
             "prefill": {"value": batch * prompt_len / (t1 - t0), "tokens": prompt_len, "ms": (t1 - t0) * 1e3 / batch,
                         "frac": prefill_rate / (peaks["bf16_tflops_sustained"] * 1e12)},
             "roofline": {"bound": "hbm", "achieved": step_bytes / (decode_ms / 1e3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                          "frac": step_bytes / (decode_ms / 1e3) / 1e9 / peaks["hbm_gbs"]},
             "output_tokens": made, "preemptions": engine.preemption_count, "pages_in_use_after": engine.cache.used_pages,
             "gpu_launches": ops.launches - launches0}
    print(json.dumps(_line("decode tokens/s (Qwen2.5-14B shape, batch 32, 8,192-token prompts, 128 greedy tokens)",
                           (made - batch) / (t2 - t1), "tokens/s", cfg,
                           dict(model="Qwen2.5-14B shape", layers_full=full_layers, global_batch=batch, seq_len=prompt_len + outputs,
                                prompt_len=prompt_len, kv_page=16, kv_pages=pages, kv_bytes_per_token=kv_bytes_per_token(cfg),
                                cuda_graph=bool(args.cuda_graph), peaks=peak_source), extra, sampler,
                           [(wall0, wall1), (wall1, wall2)])))
    return 0
