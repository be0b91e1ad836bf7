"""``flexengine random-model``: write config.json and model.safetensors from a configuration and a seed."""
from __future__ import annotations

import argparse
import json


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="flexengine random-model")
    p.add_argument("--config", required=True, help="a config.json to take the architecture and sizes from")
    p.add_argument("--out", required=True, help="folder to write")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    args = p.parse_args(argv)
    from ..weights.random_init import write_random_model
    with open(args.config, "r", encoding="utf8") as f:
        config = json.load(f)
    print(write_random_model(config, args.out, args.seed, args.dtype))
    return 0
