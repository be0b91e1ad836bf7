"""Random weights from a configuration and a seed.

The reference has no such mode in product code; its tests build random modules under
``torch.manual_seed`` (tests/unit/test_synthetic_qwen.py:91-92).  Here every checkpoint
tensor gets its own generator seeded from (seed, tensor name), so any subset can be
regenerated alone, and the statistics come from the plan (``ModelPlan.init``).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config.registry import resolve
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{int(seed)}:{name}".encode("utf8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def _rule(plan, name: str):
    init = plan.init or {}
    for suffix, rule in (init.get("suffix") or {}).items():
        if name.endswith(suffix):
            return rule
    return init.get("default", ("normal", 0.0, 0.02))


def random_tensor(plan, name: str, shape, seed: int, dtype=torch.bfloat16, device="cpu") -> torch.Tensor:
    """The tensor ``name`` of the random checkpoint (seed, plan): drawn in float32, cast to ``dtype``."""
    kind, mean, std = _rule(plan, name)
    if kind != "normal":
        raise ValueError(f"unknown init rule {kind!r}")
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    rows = shape[0] if len(shape) else 1
    out = torch.empty(shape, dtype=dtype, device=device)
    # draw big matrices in row slabs so that the float32 staging stays small
    slab = max(1, (1 << 26) // max(1, out.numel() // max(rows, 1)))
    if out.dim() < 2 or rows <= slab:
        out.copy_(torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std + mean)
    else:
        for r0 in range(0, rows, slab):
            r1 = min(rows, r0 + slab)
            out[r0:r1].copy_(torch.randn((r1 - r0,) + tuple(shape[1:]), generator=gen, device=device,
                                         dtype=torch.float32) * std + mean)
    return out


def checkpoint_tensors(plan):
    """[(name, shape)] of every tensor a checkpoint of this plan holds, in binding order."""
    out = []
    for b in plan.bindings:
        for s in b.sources:
            out.append((s.name, tuple(s.shape)))
    return out


def write_random_model(config: dict, out_dir: str, seed: int = 0, dtype: str = "bfloat16") -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` with seeded random weights."""
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    _typed, plan = resolve(config)
    os.makedirs(out_dir, exist_ok=True)
    cfg = dict(config)
    cfg["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf8") as f:
        json.dump(cfg, f, indent=2)
    tensors = checkpoint_tensors(plan)
    shapes = dict(tensors)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      [(n, s, torch_dtype) for n, s in tensors],
                      lambda n: random_tensor(plan, n, shapes[n], seed, torch_dtype),
                      metadata={"format": "pt", "seed": seed})
    return out_dir
