"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

"prenorm" is the reference's decoder layer (src/flexengine/inference/models/qwen2.py:97-130):
    x = x + mixer(norm_in(x));  x = x + feed_forward(norm_post(x)).
The residual stream is float32.  A branch output is not added at once: it is handed on
as ``pending`` and added inside the next norm kernel (fused residual add + norm).
"""
from __future__ import annotations

import inspect

import torch

from .base import build_part, register_block


def _accepts(function, name: str) -> bool:
    """Whether ``function`` names the parameter (looked up once per function)."""
    cache = _accepts.__dict__.setdefault("seen", {})
    key = (getattr(function, "__func__", function), name)
    if key not in cache:
        cache[key] = name in inspect.signature(function).parameters
    return cache[key]


class PreNormBlock:
    part_names = ("input_norm", "mixer", "post_mixer_norm", "feed_forward")
    takes_prenormed = True          # ``pending`` may be rows on their way through this block's input norm

    def __init__(self, layer_spec):
        self.input_norm = build_part("norm", layer_spec.norm)
        self.post_mixer_norm = build_part("norm", layer_spec.norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward)

    def parts(self) -> dict:
        return {name: getattr(self, name) for name in self.part_names}

    def forward(self, ctx, residual, pending, entry, next_norm=None, next_reads=None):
        """``next_norm``: the norm that will read the residual after this block (the next block's input norm), when
        the model knows it: the feed-forward may then begin it (see ``parts.base``, "a norm that follows").
        ``next_reads``: the matrix the next block streams first."""
        if getattr(ctx.ops, "native_layers_usable", None) is not None and ctx.ops.native_layers_usable(ctx):
            done = self._native_forward(ctx, residual, pending, entry)
            if done is not None:
                return done
        h = self._normed(self.input_norm, ctx, residual, pending, self.mixer)
        mixed = self._branch(self.mixer, (ctx, h, entry), ctx, residual, self.post_mixer_norm, self.feed_forward.reads_first())
        h = self._normed(self.post_mixer_norm, ctx, residual, mixed, self.feed_forward)
        return self._branch(self.feed_forward, (ctx, h), ctx, residual, next_norm, next_reads)

    def _native_forward(self, ctx, residual, pending, entry):
        """The whole layer as one call into the kernel library (a step of more than a handful of tokens, outside graph
        capture), when its parts are the ones that call is written for; None otherwise."""
        ops = ctx.ops
        layer = self.__dict__.get("_native")
        if layer is None:
            layer = self._native = self._native_layer(ctx) or False
        group = ctx.groups[entry.cache_group]
        if (layer is False or (pending is not None and not torch.is_tensor(pending)) or group.kind not in ("full", "window")
                or group.storage.dtype != torch.bfloat16):
            return None
        steps = ctx.__dict__.setdefault("_native_steps", {})
        step_key = (entry.cache_group, entry.write_cache, layer.hidden, layer.nq, layer.nkv, layer.d, layer.intermediate, layer.window)
        step = steps.get(step_key)
        if step is None:
            step = steps[step_key] = ops.native_step(ctx, group, layer, residual, entry.write_cache)
        # two buffers take turns: a layer's output is the next layer's pending input
        outs = ctx.__dict__.setdefault("_native_outs", [])
        if not outs:
            outs.extend(torch.empty((residual.shape[0], layer.hidden), dtype=torch.bfloat16, device=residual.device) for _ in range(2))
        out = outs[0] if pending is not outs[0] else outs[1]
        k_cache, v_cache = group.kv_slot(entry.cache_slot)
        return out if ops.layer_forward(layer, step, k_cache, v_cache, pending, out) else None

    def _native_layer(self, ctx):
        from .attention import AttentionMixer
        from .feed_forward import SwiGLU
        from .norm import RMSNorm
        from .position import RotaryHalfSplit
        m, f = self.mixer, self.feed_forward
        if not (type(m) is AttentionMixer and type(f) is SwiGLU and type(self.input_norm) is RMSNorm
                and type(self.post_mixer_norm) is RMSNorm and type(m.position) is RotaryHalfSplit and not m.has_out_bias
                and self.input_norm.eps == self.post_mixer_norm.eps):
            return None
        ops = ctx.ops
        if not ops.NativeLayer.fits(m.qkv_weight, m.out_weight, f.gate_up_weight, f.down_weight):
            return None
        inv_freq, rot = m.position.rotary_table(ctx.device)
        return ops.NativeLayer(self.input_norm.weight, self.post_mixer_norm.weight, self.input_norm.eps, m.qkv_weight, m.qkv_bias,
                               m.out_weight, f.gate_up_weight, f.down_weight, inv_freq, rot, m.num_heads, m.num_kv_heads,
                               m.head_dim, m.scale, m.window)

    @staticmethod
    def _normed(norm, ctx, residual, pending, reader):
        """The input of ``reader``: ``pending`` added to the residual and normalised, or, when the part before has
        begun this very norm already, the rows it left (materialised for a reader that does not take them)."""
        if getattr(pending, "weight", None) is not None and hasattr(pending, "materialize"):
            if pending.weight is not norm.weight:
                raise RuntimeError("a part began a norm that is not the one that follows it")
            return pending if getattr(reader, "takes_prenormed", False) else pending.materialize()
        # the norm is told which matrix comes next: in a decode step it starts that matrix into L2 meanwhile
        return _norm(norm, ctx, residual, pending, reader.reads_first())

    @staticmethod
    def _branch(part, args, ctx, residual, norm_after, upcoming=None):
        follow = None
        if norm_after is not None and _accepts(part.forward, "follow"):
            follow = norm_after.following(ctx, residual)
        if follow is None:
            return part.forward(*args)
        if upcoming is not None and _accepts(part.forward, "upcoming"):
            return part.forward(*args, follow=follow, upcoming=upcoming)
        return part.forward(*args, follow=follow)


def _norm(norm, ctx, residual, delta, upcoming):
    """A norm of another kind need not know the hint: it is passed only to a ``forward`` that names it."""
    if upcoming is not None and _accepts(norm.forward, "upcoming"):
        return norm.forward(ctx, residual, delta, upcoming=upcoming)
    return norm.forward(ctx, residual, delta)


register_block("prenorm", PreNormBlock)
