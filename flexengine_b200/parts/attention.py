"""Causal grouped-query attention over the paged cache.

q = h Wq^T + bq, k, v likewise; rotary encoding of q and k; k, v written to the
request's pages before the scores are taken, so that a portion sees itself; key t is
visible to the query at absolute position p iff t <= p (and t > p - window for a
window group); softmax in float32; query head h reads key/value head h // (nq/nkv);
output projection (src/flexengine/inference/models/qwen2.py:98-129,
src/flexengine/inference/attention/paged.py:18-70).
"""
from __future__ import annotations

import math

from .base import Mixer, build_part, register_mixer
from .spec import PartSpec


class AttentionMixer(Mixer):
    takes_prenormed = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec | dict | None = None, qkv_bias: bool = True, out_bias: bool = False,
                 window: int = 0, scale: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("Invalid GQA head ratio")
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise ValueError(f"head_dim={head_dim}: the attention kernels take head sizes in steps of 16 from 16 to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = \
            int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.has_qkv_bias, self.has_out_bias, self.window = bool(qkv_bias), bool(out_bias), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        if position is None:
            position = PartSpec("none")
        if isinstance(position, dict):
            position = PartSpec(position["kind"], position.get("params", {}))
        self.position = build_part("position", position)
        self.qkv_weight = self.qkv_bias = self.out_weight = self.out_bias = None      # bound by local name

    @property
    def qkv_width(self) -> int:
        return (self.num_heads + 2 * self.num_kv_heads) * self.head_dim

    def parameter_shapes(self) -> dict:
        shapes = {"qkv.weight": ((self.qkv_width, self.hidden_size), "matrix"),
                  "out.weight": ((self.hidden_size, self.num_heads * self.head_dim), "matrix")}
        if self.has_qkv_bias:
            shapes["qkv.bias"] = ((self.qkv_width,), "vector")
        if self.has_out_bias:
            shapes["out.bias"] = ((self.hidden_size,), "vector")
        return shapes

    def reads_first(self):
        return self.qkv_weight

    def cache_need(self):
        return {"kind": "window" if self.window > 0 else "full", "kv_heads": self.num_kv_heads,
                "head_dim": self.head_dim, "window": self.window}

    def forward(self, ctx, h, entry, follow=None, upcoming=None):
        ops = ctx.ops
        group = ctx.groups[entry.cache_group]
        k_cache, v_cache = group.kv_slot(entry.cache_slot)
        slot_mapping = group.slot_mapping if entry.write_cache else None
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        if self.position.applies_itself:
            # an encoding of its own: projection and bias, the encoding on the query and key heads in place,
            # then the keys and values to their cache slots
            qkv = ops.linear(h, self.qkv_weight, self.qkv_bias)
            self.position.apply(ctx, qkv[:, :nq * d].view(-1, nq, d), qkv[:, nq * d:(nq + nkv) * d].view(-1, nkv, d))
            ops.qkv_bias_rope_cache(qkv, None, ctx.positions, None, 0, slot_mapping, k_cache, v_cache, nq, nkv, d,
                                    group.page_size)
        else:
            # projection, bias, rotation and the cache write are one operation (one kernel in decode); a
            # run entry that only reads another entry's cache passes no slot mapping, so nothing is written
            inv_freq, rot = self.position.rotary_table(h.device) or (None, 0)
            qkv = ops.qkv_projection(h, self.qkv_weight, self.qkv_bias, ctx.positions, inv_freq, rot, slot_mapping,
                                     k_cache, v_cache, nq, nkv, d, group.page_size)
        out = ops.paged_attention(qkv, k_cache, v_cache, group.block_table, ctx, self.num_heads,
                                  self.num_kv_heads, self.head_dim, group.page_size, self.scale, self.window,
                                  upcoming=self.out_weight)
        if follow is not None:
            return ops.linear(out, self.out_weight, self.out_bias, follow=follow, upcoming=upcoming)
        return ops.linear(out, self.out_weight, self.out_bias)


register_mixer("attention", AttentionMixer)
