"""The reference arm of bench.py: the unmodified reference, installed under ``baseline/_ref``
(``pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy of the reference>``),
driven through its own public API: ``Qwen2Adapter.from_pretrained`` and ``Engine.submit`` / ``Engine.step``.

Nothing of flexengine_b200 is on this path.  The reference loads a Hugging Face model folder and a tokenizer, so
this file first writes both to a scratch folder with plain PyTorch and the ``safetensors`` / ``tokenizers``
libraries: random bfloat16 weights N(0, 0.02) of the Qwen2.5-7B shape in per-layer shards, and a word-level tokenizer
whose words are ``<id>``, so that a prompt of given token ids can be handed over as the string the reference's
``submit`` wants.  The metric and its configuration are those of the other arm: decode tokens per second at batch 8
after 2,048-token prompts, context limit 4,096, page size 16, bfloat16; ``materialized`` attention (the backend of
the reference's own published numbers) and the reference's own CUDA graphs for decode steps (its stock
``cuda_graph=True`` path, src/flexengine/engine/runtime.py:44-49,216-240, captured for batch buckets 1, 2, 4, 8), unless
``--no-cuda-graph`` is given.
If any step cannot be done here the arm prints ``{"impl": "reference", "unavailable": "<why>"}`` and exits 0.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:300]}))
    return 0


def write_model_folder(folder: str, cfg: dict, seed: int = 0) -> None:
    """config.json, sharded safetensors with an index, and a word-level tokenizer."""
    import torch
    from safetensors.torch import save_file
    from tokenizers import Tokenizer, models, pre_tokenizers

    os.makedirs(folder, exist_ok=True)
    hf = dict(cfg)
    hf.update({"torch_dtype": "bfloat16", "attention_dropout": 0.0, "initializer_range": 0.02, "use_cache": True,
               "bos_token_id": None, "eos_token_id": None, "sliding_window": None, "max_window_layers": cfg["num_hidden_layers"]})
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(hf, f)
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev).manual_seed(seed)
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kd = cfg["num_key_value_heads"] * cfg["head_dim"]

    def normal(*shape, mean=0.0, std=0.02):
        return (torch.randn(*shape, generator=gen, device=dev) * std + mean).to(torch.bfloat16).cpu()

    weight_map = {}

    def shard(name: str, tensors: dict) -> None:
        save_file(tensors, os.path.join(folder, name), metadata={"format": "pt"})
        for key in tensors:
            weight_map[key] = name

    shard("model-embed.safetensors", {"model.embed_tokens.weight": normal(v, h)})
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shard(f"model-layer-{l:03d}.safetensors", {
            p + "input_layernorm.weight": normal(h, mean=1.0, std=0.01),
            p + "post_attention_layernorm.weight": normal(h, mean=1.0, std=0.01),
            p + "self_attn.q_proj.weight": normal(qd, h), p + "self_attn.q_proj.bias": normal(qd),
            p + "self_attn.k_proj.weight": normal(kd, h), p + "self_attn.k_proj.bias": normal(kd),
            p + "self_attn.v_proj.weight": normal(kd, h), p + "self_attn.v_proj.bias": normal(kd),
            p + "self_attn.o_proj.weight": normal(h, qd),
            p + "mlp.gate_proj.weight": normal(i, h), p + "mlp.up_proj.weight": normal(i, h),
            p + "mlp.down_proj.weight": normal(h, i)})
    shard("model-head.safetensors", {"model.norm.weight": normal(h, mean=1.0, std=0.01), "lm_head.weight": normal(v, h)})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)

    tok = Tokenizer(models.WordLevel({f"<{t}>": t for t in range(v)}, unk_token="<0>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "model_max_length": 1 << 20}, f)


def main(args) -> int:
    if not os.path.isdir(os.path.join(REF, "flexengine")):
        return unavailable("the reference is not installed under baseline/_ref")
    sys.path.insert(0, ROOT)
    # sizes of the workload and the nvidia-smi sampler: plain Python shared with the other arm, no model or kernel code
    from flexengine_b200.bench.clocks import ClockSampler
    from flexengine_b200.bench.shapes import CONTEXT_LEN, PAGE, PROMPT_LEN, SEVEN_B, flat_config
    folder = None
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        sys.path.insert(0, REF)
        from flexengine.engine.config import EngineConfig
        from flexengine.engine.runtime import Engine
        from flexengine.inference.models.qwen2 import Qwen2Adapter

        cfg = dict(SEVEN_B)
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        batch, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
        need = 2 * (cfg["num_hidden_layers"] * 233e6 + 2 * cfg["vocab_size"] * cfg["hidden_size"]) * 1.1
        base = tempfile.gettempdir()
        if shutil.disk_usage(base).free < need:
            return unavailable(f"not enough scratch space in {base} for the model folder the reference loads")
        folder = tempfile.mkdtemp(prefix="reference_model_")
        write_model_folder(folder, cfg)
        adapter = Qwen2Adapter.from_pretrained(folder, device="cuda:0", dtype="bfloat16", attention_backend="materialized")
        engine = Engine(EngineConfig(
            model=folder, device="cuda:0", dtype="bfloat16", max_model_len=CONTEXT_LEN, max_num_seqs=batch,
            max_num_batched_tokens=PROMPT_LEN, prefill_chunk_size=PROMPT_LEN, max_waiting=max(64, batch),
            kv_block_size=PAGE, kv_num_blocks=batch * CONTEXT_LEN // PAGE, attention_backend="materialized",
            max_output_tokens=512, trace_steps=False, cuda_graph=bool(args.cuda_graph)), adapter)
        gen = torch.Generator().manual_seed(1)
        sampler = ClockSampler()
        sampler.start()

        def prompt():
            return " ".join(f"<{t}>" for t in torch.randint(0, cfg["vocab_size"], (PROMPT_LEN,), generator=gen).tolist())

        requests = [engine.submit(prompt(), max_tokens=warmup + steps + batch + 8) for _ in range(batch)]
        # prefill: the first step runs the first request's whole prompt (token budget = prompt length)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.step()
        torch.cuda.synchronize()
        prefill_ms = (time.perf_counter() - t0) * 1e3
        while any(len(r.generated_ids) < warmup for r in requests):
            if not engine.step():
                raise RuntimeError(f"the reference engine stopped: {engine.fault}")
        before = [len(r.generated_ids) for r in requests]
        torch.cuda.synchronize()
        w0 = time.time()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            engine.step()
        end.record()
        torch.cuda.synchronize()
        windows = [(w0, time.time())]
        ms = start.elapsed_time(end) / steps
        if engine.fault:
            raise RuntimeError(engine.fault)
        if not all(len(r.generated_ids) == n + steps for r, n in zip(requests, before)):
            raise RuntimeError("a timed step of the reference was not a full decode step")
        sampler.stop()
        graph_stats = engine.graph_manager.stats() if getattr(engine, "graph_manager", None) is not None else {}
        engine.stop()
        value = batch / (ms / 1e3)
        print(json.dumps({
            "impl": "reference", "metric": "decode tokens/s (Qwen2.5-7B shape, batch 8, 2,048-token prompts)",
            "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: random token ids, random weights N(0, 0.02)",
            "config": flat_config(cfg, model="Qwen2.5-7B shape", layers_full=SEVEN_B["num_hidden_layers"],
                                  global_batch=batch, seq_len=CONTEXT_LEN, prompt_len=PROMPT_LEN, kv_page=PAGE,
                                  parallelism="single GPU", cuda_graph=bool(args.cuda_graph),
                                  attention_backend="materialized"),
            "e2e": {"value": value, "unit": "tokens/s", "note": "the reference's API is host tokens in and out; same run"},
            "prefill": {"value": PROMPT_LEN / (prefill_ms / 1e3), "tokens": PROMPT_LEN, "ms": prefill_ms,
                        "note": "the reference's first step, cold"},
            "reference_graphs": {k: graph_stats.get(k) for k in ("captures", "replays", "fallbacks")},
            "clocks": sampler.summary(windows)}))
        return 0
    except Exception as ex:  # noqa: BLE001 - whatever keeps the reference from running is reported, not raised
        return unavailable(f"{type(ex).__name__}: {ex}")
    finally:
        if folder:
            shutil.rmtree(folder, ignore_errors=True)
