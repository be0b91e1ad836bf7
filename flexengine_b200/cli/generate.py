"""``flexengine generate``: model folder in, generated tokens out.

Engine options carry the reference's names and meanings (src/flexengine/serving/cli/server.py:7-54):
--model, --policy, --token-budget, --prefill-chunk-size, --block-size, --num-blocks,
--max-model-len, --max-num-seqs, --trace-dir, --[no-]cuda-graph; like there, each one
overrides the matching ``FLEX_*`` variable (src/flexengine/engine/config.py:64-86).
Sampling options are those of a request (src/flexengine/engine/runtime.py:89): --max-tokens,
--temperature, --top-k, --seed.
"""
from __future__ import annotations

import argparse
import json
import sys


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="flexengine generate", description="Generate tokens with the engine")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--random-weights", action="store_true",
                   help="ignore model.safetensors: draw seeded random weights for config.json on the device")
    p.add_argument("--weights-seed", type=int, default=0)
    p.add_argument("--prompt", action="append", default=[], help="text prompt (needs tokenizer.json in the folder)")
    p.add_argument("--prompt-ids", action="append", default=[], help="token ids, comma or space separated")
    p.add_argument("--max-tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--dtype", choices=["bfloat16", "bf16", "float32", "fp32"], default=None)
    p.add_argument("--device", default=None)
    p.add_argument("--policy", choices=["fcfs", "decode_first", "slo_aware", "adaptive"], default=None)
    p.add_argument("--trace-dir", default=None)
    p.add_argument("--token-budget", type=int, default=None)
    p.add_argument("--prefill-chunk-size", type=int, default=None)
    p.add_argument("--block-size", type=int, default=None)
    p.add_argument("--num-blocks", type=int, default=None)
    p.add_argument("--max-model-len", type=int, default=None)
    p.add_argument("--max-num-seqs", type=int, default=None)
    p.add_argument("--cuda-graph", action=argparse.BooleanOptionalAction, default=None)
    return p


def engine_config_from_args(args):
    from ..config.engine_config import EngineConfig
    return EngineConfig.from_env(
        model=args.model, dtype=args.dtype, device=args.device, scheduler_policy=args.policy,
        trace_dir=args.trace_dir, max_num_batched_tokens=args.token_budget,
        prefill_chunk_size=args.prefill_chunk_size, kv_block_size=args.block_size, kv_num_blocks=args.num_blocks,
        max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs, cuda_graph=args.cuda_graph)


def load_tokenizer(model_dir: str):
    """A tokenizer for text prompts when the folder has ``tokenizer.json`` (the ``tokenizers``
    package); random-weight folders have none and take token ids."""
    import os
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    from tokenizers import Tokenizer

    class _Wrapped:
        bos_token_id = None

        def __init__(self, tok):
            self.tok = tok

        def encode(self, text, add_special_tokens=False):
            return self.tok.encode(text, add_special_tokens=add_special_tokens).ids

        def decode(self, ids, skip_special_tokens=True, clean_up_tokenization_spaces=False):
            return self.tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    return _Wrapped(Tokenizer.from_file(path))


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from ..config.model_config import read_config_json
    from ..engine.runtime import Engine
    from ..weights.loader import load_model, random_model
    config = engine_config_from_args(args)
    prompts = list(args.prompt)
    for text in args.prompt_ids:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    if not prompts:
        print("give at least one --prompt or --prompt-ids", file=sys.stderr)
        return 2
    tokenizer = load_tokenizer(args.model)
    if args.random_weights:
        _typed, _plan, model = random_model(read_config_json(args.model), args.weights_seed, config.dtype, config.device)
    else:
        _typed, _plan, model = load_model(args.model, config.dtype, config.device)
    engine = Engine.from_model(model, config, tokenizer=tokenizer)
    outputs = engine.generate(prompts, max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                              seed=args.seed)
    for out in outputs:
        print(json.dumps({"request_id": out.request_id, "prompt_tokens": len(out.prompt_ids),
                          "token_ids": out.token_ids, "text": out.text, "finish_reason": out.finish_reason}))
    return 0
