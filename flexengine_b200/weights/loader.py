"""Binding checkpoint tensors to a model by name.

Precision rule: in bfloat16 mode matrices stay bfloat16 (float16 is converted), a matrix
stored in 32-bit stays 32-bit (its product then runs in float32), norm weights and
biases are held in float32 (lossless from bfloat16), integer tables become int32; in
float32 mode every floating tensor is float32.  All mismatches between what the plan
needs and what the files hold are reported in ONE error: missing, unexpected, wrong shape,
wrong dtype.  (The reference delegates loading to ``from_pretrained``,
src/flexengine/inference/models/qwen2.py:51-65.)
"""
from __future__ import annotations

import torch

from ..config.model_config import read_config_json
from ..config.registry import resolve
from ..parts.model import DecoderModel
from .random_init import random_tensor
from .safetensors_io import DTYPES, CheckpointReader

FLOAT_STORED = ("BF16", "F16", "F32")
INT_STORED = ("I32", "I64")
COMPUTE_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class CheckpointError(ValueError):
    """The checkpoint does not fit the model; the message lists every problem."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, other=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype, self.other = list(wrong_shape), list(wrong_dtype), list(other)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got, want in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}, expected one of {list(want)}")
        lines += [f"  {o}" for o in self.other]
        super().__init__("\n".join(lines))


def check_against_plan(plan, entries: dict) -> None:
    """``entries``: {name: object with .shape and .dtype (safetensors dtype string)}."""
    wanted = {}
    kinds = {}
    for b in plan.bindings:
        for s in b.sources:
            wanted[s.name] = tuple(s.shape)
            kinds[s.name] = b.kind
    missing = sorted(set(wanted) - set(entries), key=_natural)
    unexpected = sorted(set(entries) - set(wanted), key=_natural)
    wrong_shape, wrong_dtype = [], []
    for name in sorted(set(wanted) & set(entries), key=_natural):
        e = entries[name]
        if tuple(e.shape) != wanted[name]:
            wrong_shape.append((name, tuple(e.shape), wanted[name]))
        allowed = INT_STORED if kinds[name] == "int" else FLOAT_STORED
        if e.dtype not in allowed:
            wrong_dtype.append((name, e.dtype, allowed))
    other = []
    for b in plan.bindings:
        if b.alias_of is not None:
            other += [f"{name} is present although {b.why or 'the plan binds its target to another tensor'}"
                      for name in b.absent if name in entries]
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise CheckpointError(missing, unexpected, wrong_shape, wrong_dtype, other)


def _natural(name: str):
    return [(0, int(p), "") if p.isdigit() else (1, 0, p) for p in name.split(".")]


def _held_dtype(kind: str, stored: list, compute: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if kind == "vector" or compute == torch.float32:
        return torch.float32
    if any(s == "F32" for s in stored):
        return torch.float32          # stored in 32-bit: stays so
    return torch.bfloat16


def _bind_all(plan, compute: torch.dtype, device, fetch, stored_dtype) -> DecoderModel:
    model = DecoderModel(plan)
    shapes = model.parameter_shapes()
    tensors = {}
    problems = []
    for b in plan.bindings:
        if b.alias_of is not None:
            continue
        if b.target not in shapes:
            problems.append(f"binding target {b.target} is not a parameter of the model")
            continue
        want_shape, kind = shapes[b.target]
        held = _held_dtype(kind, [stored_dtype(s.name) for s in b.sources], compute)
        rows = sum(s.shape[0] for s in b.sources)
        full_shape = (rows,) + tuple(b.sources[0].shape[1:])
        if tuple(full_shape) != tuple(want_shape):
            problems.append(f"binding {b.target}: sources give {full_shape}, the part wants {tuple(want_shape)}")
            continue
        out = torch.empty(full_shape, dtype=held, device=device)
        r = 0
        for s in b.sources:
            out[r:r + s.shape[0]].copy_(fetch(s.name, s.shape), non_blocking=False)
            r += s.shape[0]
        tensors[b.target] = out
    for b in plan.bindings:
        if b.alias_of is not None:
            tensors[b.target] = tensors[b.alias_of]
    unbound = sorted(str(t) for t in set(shapes) - set(tensors))
    if unbound:
        problems.append("model parameters without a binding: " + ", ".join(unbound))
    if problems:
        raise CheckpointError([], [], [], [], problems)
    model.bind(tensors, compute, torch.device(device))
    return model


def load_model(model_dir: str, dtype: str = "bfloat16", device="cuda:0"):
    """Model folder -> (typed config, plan, DecoderModel with weights on ``device``)."""
    compute = COMPUTE_DTYPES[dtype]
    typed, plan = resolve(read_config_json(model_dir))
    reader = CheckpointReader(model_dir)
    check_against_plan(plan, reader.entries)
    try:
        model = _bind_all(plan, compute, device, lambda name, _shape: reader.read(name),
                          lambda name: reader.entries[name].dtype)
    finally:
        reader.close()
    return typed, plan, model


def random_model(config: dict, seed: int = 0, dtype: str = "bfloat16", device="cuda:0",
                 stored_dtype: str = "bfloat16"):
    """The model that ``write_random_model(config, ..., seed)`` would describe, generated on
    ``device`` without touching disk (values differ from the on-disk variant, which is drawn
    by the CPU generator, unless ``device`` is the CPU)."""
    compute = COMPUTE_DTYPES[dtype]
    typed, plan = resolve(config)
    stored = {"bfloat16": torch.bfloat16, "float32": torch.float32}[stored_dtype]
    code = {torch.bfloat16: "BF16", torch.float32: "F32"}[stored]
    model = _bind_all(plan, compute, device,
                      lambda name, shape: random_tensor(plan, name, shape, seed, stored, device),
                      lambda name: code)
    return typed, plan, model
