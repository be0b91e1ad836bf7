"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

"prenorm" is the reference's decoder layer (src/flexengine/inference/models/qwen2.py:97-130):
    x = x + mixer(norm_in(x));  x = x + feed_forward(norm_post(x)).
The residual stream is float32.  A branch output is not added at once: it is handed on
as ``pending`` and added inside the next norm kernel (fused residual add + norm).
"""
from __future__ import annotations

import inspect

from .base import build_part, register_block


class PreNormBlock:
    part_names = ("input_norm", "mixer", "post_mixer_norm", "feed_forward")

    def __init__(self, layer_spec):
        self.input_norm = build_part("norm", layer_spec.norm)
        self.post_mixer_norm = build_part("norm", layer_spec.norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward)

    def parts(self) -> dict:
        return {name: getattr(self, name) for name in self.part_names}

    def forward(self, ctx, residual, pending, entry):
        # each norm is told which matrix comes next: in a decode step it starts that matrix into L2 meanwhile
        h = _norm(self.input_norm, ctx, residual, pending, self.mixer.reads_first())
        mixed = self.mixer.forward(ctx, h, entry)
        h = _norm(self.post_mixer_norm, ctx, residual, mixed, self.feed_forward.reads_first())
        return self.feed_forward.forward(ctx, h)


def _norm(norm, ctx, residual, delta, upcoming):
    """A norm of another kind need not know the hint: it is passed only to a ``forward`` that names it."""
    takes = getattr(norm, "_takes_upcoming", None)
    if takes is None:
        takes = norm._takes_upcoming = "upcoming" in inspect.signature(norm.forward).parameters
    if takes and upcoming is not None:
        return norm.forward(ctx, residual, delta, upcoming=upcoming)
    return norm.forward(ctx, residual, delta)


register_block("prenorm", PreNormBlock)
