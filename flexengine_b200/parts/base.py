"""Interfaces of the parts a layer is put together from, and their registries.

A part knows its own sizes and constants (constructor parameters) and nothing about
the model it sits in.  Kinds are looked up by name, so that a test or another
architecture can add a mixer, feed-forward, norm, position encoding or block
arrangement with ``register_*`` and no change to this package.

Interfaces
----------
Every part:      ``parameter_shapes() -> {local name: (shape, kind)}`` with kind in
                 {"matrix", "vector", "int"}; ``bind({local name: tensor})``.
Mixer:           ``cache_need() -> dict | None`` (what cache group it needs) and
                 ``forward(ctx, h, entry) -> delta [T, hidden]``.  A mixer that keeps per-request
                 state reads and writes ``ctx.groups[g].state(slot)[ctx.state_slots[r]]`` for request r.
                 **A state slot below 0 is a padding request** (a batch padded to a fixed shape for a
                 CUDA graph): the mixer touches no state for it, and what it returns for its rows is
                 never read.  The same holds for cache slot -1 in ``slot_mapping``: nothing is written.
                 Under CUDA graphs the slots must be taken from the device tensors (``ctx.state_slots``),
                 not from their host copies, whose values a captured graph would keep for good.
FeedForward:     ``forward(ctx, h) -> delta [T, hidden]``.
Norm:            ``forward(ctx, residual, delta, rows=None) -> h``: adds ``delta`` (may be None)
                 to the float32 residual stream in place and returns the normalised rows
                 in the compute dtype; with ``rows`` it reads only those rows and leaves the
                 residual untouched.  ``following(ctx, residual)`` may return what a product needs
                 to do this norm's work in its own epilogue (see "a norm that follows" below).
PositionEncoding: ``rotary_table(device)`` -> (inv_freq float32 [rot/2], rot) for the half-split
                 rotation that the mixer's kernel does itself, or None for no rotation there; an
                 encoding of its own overrides ``apply(ctx, q, k)``, which rewrites the query heads
                 q [T, nq, d] and key heads k [T, nkv, d] in place (views of one projection,
                 biases added) before the keys go to the cache; ``ctx.positions`` are the tokens'
                 absolute positions.
Block:           ``forward(ctx, residual, pending, entry) -> pending``: the arrangement of
                 norms, mixer and feed-forward around the residual stream.
A norm that follows: in a decode step a norm is a few kilobytes between products that stream
                 hundreds of megabytes.  A block may therefore hand the part that ends a branch
                 ``follow=(residual, norm weight, eps)`` (only to a ``forward`` that names the
                 parameter): the part may then add its output to the residual itself and return the
                 rows on their way through that norm (``ctx.ops.Prenormed``) instead of its output,
                 or ignore the hint and return its output as ever.  A part whose ``forward`` may be
                 given such rows as its input says so with ``takes_prenormed = True``; others get
                 them materialised.
Embedding:       ``forward(ctx) -> residual``: the float32 residual stream [T, hidden] of the step's
                 tokens (``ctx.token_ids``), which the blocks then add to in place.
Head:            ``forward(ctx, h) -> logits``: float32 [rows, vocab] from the final norm's output
                 rows (the rows whose logits are wanted, nothing else reaches it).
"""
from __future__ import annotations

from typing import Callable

_REGISTRIES: dict[str, dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str, factory: Callable) -> None:
    _REGISTRIES[family][kind] = factory


def register_mixer(kind: str, factory: Callable) -> None:
    _register("mixer", kind, factory)


def register_feed_forward(kind: str, factory: Callable) -> None:
    _register("feed_forward", kind, factory)


def register_norm(kind: str, factory: Callable) -> None:
    _register("norm", kind, factory)


def register_position(kind: str, factory: Callable) -> None:
    _register("position", kind, factory)


def register_block(kind: str, factory: Callable) -> None:
    _register("block", kind, factory)


def register_embedding(kind: str, factory: Callable) -> None:
    _register("embedding", kind, factory)


def register_head(kind: str, factory: Callable) -> None:
    _register("head", kind, factory)


def build_part(family: str, spec):
    """Instantiate ``spec`` (a PartSpec) from the registry of ``family``."""
    table = _REGISTRIES[family]
    if spec.kind not in table:
        raise KeyError(f"unknown {family} kind {spec.kind!r}; known: {sorted(table)}")
    return table[spec.kind](**dict(spec.params))


def block_factory(kind: str) -> Callable:
    table = _REGISTRIES["block"]
    if kind not in table:
        raise KeyError(f"unknown block kind {kind!r}; known: {sorted(table)}")
    return table[kind]


class Part:
    """Common behaviour: declared parameters are bound by local name with a shape check."""

    def parameter_shapes(self) -> dict:
        return {}

    def bind(self, tensors: dict) -> None:
        want = self.parameter_shapes()
        missing = sorted(set(want) - set(tensors))
        extra = sorted(set(tensors) - set(want))
        if missing or extra:
            raise ValueError(f"{type(self).__name__}: missing {missing}, unexpected {extra}")
        for name, (shape, _kind) in want.items():
            if tuple(tensors[name].shape) != tuple(shape):
                raise ValueError(f"{type(self).__name__}.{name}: shape {tuple(tensors[name].shape)}, want {tuple(shape)}")
            setattr(self, name.replace(".", "_"), tensors[name])

    def reads_first(self):
        """The weight matrix this part streams first, or None.  A small kernel that runs before the part in
        a decode step may ask for its start to be brought into L2 (``upcoming`` of the ops)."""
        return None


class Mixer(Part):
    takes_prenormed = False

    def cache_need(self):
        return None

    def forward(self, ctx, h, entry):  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    takes_prenormed = False

    def forward(self, ctx, h):  # pragma: no cover - interface
        raise NotImplementedError


class Norm(Part):
    def forward(self, ctx, residual, delta, rows=None):  # pragma: no cover - interface
        raise NotImplementedError

    def following(self, ctx, residual):
        """(residual, weight, eps) when a product may do this norm's work in its epilogue in this step, else None."""
        return None


class Embedding(Part):
    def forward(self, ctx):  # pragma: no cover - interface
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx, h):  # pragma: no cover - interface
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_table(self, device):
        return None

    def apply(self, ctx, q, k):
        return None

    @property
    def applies_itself(self) -> bool:
        """True when the class brings an ``apply`` of its own: the mixer then projects, lets the encoding
        rewrite queries and keys, and writes the cache afterwards, instead of the fused kernel."""
        return type(self).apply is not PositionEncoding.apply
