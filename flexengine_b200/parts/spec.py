"""Data that describes a model as an arrangement of parts.

A model is a :class:`ModelPlan`: a list of layers (each a mixer, a feed-forward, a
norm kind and a block arrangement, chosen layer by layer), the order in which the
layers run (data too: an entry may name a layer twice, or read the cache another
entry wrote), the cache groups the mixers need, and the tensors to bind by name.
The reference hard-wires one decoder loop (src/flexengine/inference/models/qwen2.py:95-130);
here the same loop is the interpretation of a plan.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence


@dataclass(frozen=True)
class PartSpec:
    """A part kind (a key of one of the part registries) and its parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class CacheGroupSpec:
    """What one group of layers needs from the cache manager.

    kind "full":   paged keys/values, every key kept.
    kind "window": paged keys/values, only the last ``window`` keys are visible; pages
                   that the window has passed are given back.
    kind "state":  a fixed-size per-request slot (``state_shape`` elements of ``state_dtype``),
                   zeroed at admission.
    ``slots`` is the number of cache slots in the group (one per run entry that writes).
    ``page_size``: tokens per page of this group; 0 takes the engine's ``kv_block_size``.
    ``chunk_granularity``: portions of a prompt that do not end it must be multiples of this many
    tokens (a mixer whose state advances in blocks); the scheduler rounds to the least common
    multiple over the groups.
    """
    name: str
    kind: str
    slots: int
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: tuple = ()
    state_dtype: str = "float32"
    page_size: int = 0
    chunk_granularity: int = 1

    def __post_init__(self):
        if self.page_size < 0 or self.chunk_granularity < 1:
            raise ValueError("page_size must be >= 0 and chunk_granularity >= 1")
        if self.kind not in ("full", "window", "state"):
            raise ValueError(f"unknown cache group kind {self.kind!r}")
        if self.kind == "window" and self.window <= 0:
            raise ValueError("a window group needs window > 0")


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which parts it is made of.  ``block`` names the arrangement."""
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec
    block: str = "prenorm"


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order.

    ``layer`` indexes ``ModelPlan.layers`` (the same layer may appear more than once).
    ``cache_group``/``cache_slot`` say where this run's mixer keeps what it remembers;
    ``write_cache=False`` makes it read what another entry wrote into that slot.
    """
    layer: int
    cache_group: int = 0
    cache_slot: int = 0
    write_cache: bool = True


@dataclass(frozen=True)
class WeightSource:
    """A tensor in the checkpoint, by name, with the shape it must have."""
    name: str
    shape: tuple


@dataclass(frozen=True)
class WeightBinding:
    """Where checkpoint tensors go.

    ``target`` is ("embedding"|"final_norm"|"lm_head", local) or ("layer", i, part, local)
    with part in {"mixer", "feed_forward", "norm"}.  Several sources are concatenated
    along dim 0 in the given order.  ``alias_of`` binds the target to another target's
    storage instead (tied embeddings); then ``sources`` is empty, and ``absent`` may name
    checkpoint tensors whose presence contradicts the alias (``why`` says what they contradict).
    ``kind`` is "matrix" (kept in the compute dtype, bfloat16 or as stored when 32-bit),
    "vector" (norm weights and biases; held in float32, which is lossless) or
    "int" (integer tables, int32).
    """
    target: tuple
    sources: tuple = ()
    alias_of: tuple | None = None
    kind: str = "matrix"
    absent: tuple = ()
    why: str = ""


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Sequence[LayerSpec]
    run: Sequence[RunEntry]
    cache_groups: Sequence[CacheGroupSpec]
    final_norm: PartSpec
    bindings: Sequence[WeightBinding]
    # how the residual stream starts and how logits are made of it; None: a token table and a
    # bias-free vocabulary product of the plan's sizes
    embedding: PartSpec | None = None
    head: PartSpec | None = None
    eos_token_ids: tuple = ()
    bos_token_id: int | None = None
    # statistics of random initialisation, by binding kind / local name
    init: Mapping[str, Any] = field(default_factory=dict)

    def validate(self) -> None:
        for e in self.run:
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"run entry names layer {e.layer}, plan has {len(self.layers)}")
            if not (0 <= e.cache_group < len(self.cache_groups)):
                raise ValueError(f"run entry names cache group {e.cache_group}")
            g = self.cache_groups[e.cache_group]
            if not (0 <= e.cache_slot < g.slots):
                raise ValueError(f"run entry names slot {e.cache_slot} of group {g.name!r} with {g.slots} slots")
        written = {(e.cache_group, e.cache_slot) for e in self.run if e.write_cache}
        for e in self.run:
            if not e.write_cache and (e.cache_group, e.cache_slot) not in written:
                raise ValueError("a run entry reads a cache slot that no entry writes")
