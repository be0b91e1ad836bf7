"""Kernel by kernel: what each operation of a decode step and of a prefill step reads or computes, how long it
takes, and what fraction of the machine's measured peak that is.

Every operation is timed where it runs in serving: inside a replayed CUDA graph (decode) or launched back to back
(prefill), once per layer of the model, each layer with its own weights and its own cache, so that what a kernel
reads comes from HBM and not from a cache the previous repetition warmed (a 7B model's layers hold 13 GB, L2 126 MB).
"""
from __future__ import annotations

import torch


def _time_graph(fn, reps: int = 5) -> float:
    """Milliseconds of one replay of ``fn`` captured into a CUDA graph (a warm-up run outside the graph first)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        fn()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps


def _time_eager(fn, reps: int = 3) -> float:
    fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps


def kernel_table(model, cfg: dict, batch: int, context: int, peaks: dict, timer=None) -> dict:
    """{"decode": [...], "prefill": [...]}: one row per operation with its time per layer in microseconds, the bytes
    it has to read (decode) or the flops it does (prefill), and the fraction of the measured peak."""
    from .. import ops
    from ..cache import CacheManager
    from ..engine import ModelRunner, StepEntry

    dev = model.device
    plan = model.plan
    layers = len(model.blocks)
    h, inter, vocab = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    page = 16
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rows = {"decode": [], "prefill": []}

    def decode_row(name, ms_total, bytes_each, count=layers):
        us = ms_total * 1e3 / count
        rows["decode"].append({"kernel": name, "us": round(us, 2), "mbytes": round(bytes_each / 1e6, 2),
                               "gbs": round(bytes_each / (us * 1e-6) / 1e9, 1) if bytes_each else None,
                               "frac_hbm": round(bytes_each / (us * 1e-6) / hbm, 3) if bytes_each else None})

    def prefill_row(name, ms_total, flops_each, count=layers):
        us = ms_total * 1e3 / count
        rows["prefill"].append({"kernel": name, "us": round(us, 1), "gflop": round(flops_each / 1e9, 1),
                                "tflops": round(flops_each / (us * 1e-6) / 1e12, 1) if flops_each else None,
                                "frac_tensor": round(flops_each / (us * 1e-6) / tensor, 3) if flops_each else None})

    # ---- decode: ``batch`` requests of one token each at ``context`` cached tokens ------------------------------
    cache = CacheManager(plan.cache_groups, batch * (context // page + 2), page, batch, torch.bfloat16, dev)
    runner = ModelRunner(model, cache)
    rids = [f"k{i}" for i in range(batch)]
    for rid in rids:
        cache.reserve(rid, context + 1)
        cache.commit(rid, context)                        # the cache holds zeros: time does not depend on values
    ctx = runner.build_context([StepEntry(rid, [1], [0]) for rid in rids])
    torch.cuda.synchronize()
    group = ctx.groups[0]
    blocks = model.blocks
    residual = torch.randn(batch, h, device=dev)
    delta = torch.randn(batch, h, device=dev).to(torch.bfloat16)
    hidden = torch.randn(batch, h, device=dev).to(torch.bfloat16)
    heads_out = torch.randn(batch, nq * d, device=dev).to(torch.bfloat16)
    act = torch.randn(batch, inter, device=dev).to(torch.bfloat16)
    qkv = torch.randn(batch, (nq + 2 * nkv) * d, device=dev).to(torch.bfloat16)
    bf = 2

    def each_layer(fn):
        def run():
            for l in range(layers):
                fn(l, blocks[l])
        return run

    # the forms a decode step runs: the product that ends a branch adds to the residual and begins the next norm, the
    # product that reads the norm finishes it (no norm kernel between them)
    eps = blocks[0].input_norm.eps
    began = ops.linear(heads_out, blocks[0].mixer.out_weight, follow=(residual, blocks[0].post_mixer_norm.weight, eps))
    fused = isinstance(began, ops.Prenormed)
    normed = began if fused else hidden

    def project(l, b):
        m = b.mixer
        inv_freq, rot = m.position.rotary_table(dev)
        k_cache, v_cache = group.kv_slot(l)
        ops.qkv_projection(normed, m.qkv_weight, m.qkv_bias, ctx.positions, inv_freq, rot, group.slot_mapping, k_cache, v_cache,
                           nq, nkv, d, page)

    def attend(l, b):
        k_cache, v_cache = group.kv_slot(l)
        ops.paged_attention(qkv, k_cache, v_cache, group.block_table, ctx, nq, nkv, d, page, b.mixer.scale, 0)

    def end_branch(x, weight_of, norm_of):
        def run(l, b):
            ops.linear(x, weight_of(b), follow=(residual, norm_of(b).weight, eps))
        return run

    decode_row("norm as a kernel (first layer and final norm only)", _time_graph(each_layer(
        lambda l, b: ops.add_rmsnorm(residual, delta, b.input_norm.weight, b.input_norm.eps, torch.bfloat16))), 0)
    decode_row("qkv projection: norm scale, bias, rotary, cache write", _time_graph(each_layer(project)), (nq + 2 * nkv) * d * h * bf)
    decode_row("decode attention (splits merged in the cluster)", _time_graph(each_layer(attend)), batch * (context + 1) * 2 * nkv * d * bf)
    decode_row("output projection + residual add + norm begun", _time_graph(each_layer(
        end_branch(heads_out, lambda b: b.mixer.out_weight, lambda b: b.post_mixer_norm))), nq * d * h * bf)
    decode_row("gate/up projection: norm scale, SwiGLU", _time_graph(each_layer(
        lambda l, b: ops.linear_swiglu(normed, b.feed_forward.gate_up_weight, inter))), 2 * inter * h * bf)
    decode_row("down projection + residual add + norm begun", _time_graph(each_layer(
        end_branch(act, lambda b: b.feed_forward.down_weight, lambda b: b.input_norm))), inter * h * bf)
    logits = ops.linear(hidden, model.lm_head, None, out_float32=True)
    decode_row("vocabulary projection (once a step)", _time_graph(
        lambda: ops.linear(hidden, model.lm_head, None, out_float32=True)), vocab * h * bf, count=1)
    zeros = (torch.zeros(batch, device=dev), torch.zeros(batch, dtype=torch.int32, device=dev), torch.zeros(batch, dtype=torch.int64, device=dev))
    decode_row("greedy sampling (once a step)", _time_graph(lambda: ops.sample(logits, zeros[0], zeros[1], zeros[2], zeros[2])),
               batch * vocab * 4, count=1)
    for rid in rids:
        runner.finish(rid)
    del cache, runner, ctx, group

    # ---- prefill: one prompt of ``context`` tokens ---------------------------------------------------------------
    T = context
    cache = CacheManager(plan.cache_groups, T // page + 2, page, 1, torch.bfloat16, dev)
    runner = ModelRunner(model, cache)
    cache.reserve("p", T)
    ctx = runner.build_context([StepEntry("p", [1] * T, [T - 1])])
    group = ctx.groups[0]
    residual = torch.randn(T, h, device=dev)
    delta = torch.randn(T, h, device=dev).to(torch.bfloat16)
    hidden = torch.randn(T, h, device=dev).to(torch.bfloat16)
    heads_out = torch.randn(T, nq * d, device=dev).to(torch.bfloat16)
    act = torch.randn(T, inter, device=dev).to(torch.bfloat16)
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=dev).to(torch.bfloat16)
    normed = hidden
    prefill_row("norm (residual add + RMSNorm)", _time_eager(each_layer(
        lambda l, b: ops.add_rmsnorm(residual, delta, b.input_norm.weight, b.input_norm.eps, torch.bfloat16))), 0)
    prefill_row("qkv projection, bias + rotary + cache write", _time_eager(each_layer(project)), 2.0 * T * (nq + 2 * nkv) * d * h)
    prefill_row("prefill attention", _time_eager(each_layer(attend)), 4.0 * nq * d * T * (T + 1) / 2)
    prefill_row("output projection", _time_eager(each_layer(lambda l, b: ops.linear(heads_out, b.mixer.out_weight))), 2.0 * T * nq * d * h)
    prefill_row("gate/up projection + SwiGLU", _time_eager(each_layer(
        lambda l, b: ops.linear_swiglu(hidden, b.feed_forward.gate_up_weight, inter))), 2.0 * T * 2 * inter * h)
    prefill_row("down projection", _time_eager(each_layer(lambda l, b: ops.linear(act, b.feed_forward.down_weight))), 2.0 * T * inter * h)
    runner.finish("p")
    ops.check_status(dev)
    return rows
