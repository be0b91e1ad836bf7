"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

"prenorm" is the reference's decoder layer (src/flexengine/inference/models/qwen2.py:97-130):
    x = x + mixer(norm_in(x));  x = x + feed_forward(norm_post(x)).
The residual stream is float32.  A branch output is not added at once: it is handed on
as ``pending`` and added inside the next norm kernel (fused residual add + norm).
"""
from __future__ import annotations

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
        h = self.input_norm.forward(ctx, residual, pending)
        mixed = self.mixer.forward(ctx, h, entry)
        h = self.post_mixer_norm.forward(ctx, residual, mixed)
        return self.feed_forward.forward(ctx, h)


register_block("prenorm", PreNormBlock)
