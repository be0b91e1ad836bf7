"""Qwen2 / Qwen2.5 dense decoder as a plan of parts.

Pre-norm RMSNorm, grouped-query attention with biased Q/K/V projections and half-split
rotary encoding, SwiGLU feed-forward, optionally tied embeddings
(src/flexengine/inference/models/qwen2.py:20-136).  Tensor names are the ones the
reference walks as module attributes (qwen2.py:94-135): q/k/v are concatenated into
one [(nq+2nkv)d, H] matrix and gate/up into one [2I, H] matrix at load.
"""
from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..config.registry import register_architecture
from ..parts.spec import (CacheGroupSpec, LayerSpec, ModelPlan, PartSpec, RunEntry, WeightBinding, WeightSource)


def build_qwen2_plan(cfg: Qwen2Config) -> ModelPlan:
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    norm = PartSpec("rmsnorm", {"hidden_size": h, "eps": cfg.rms_norm_eps})
    mixer = PartSpec("attention", {
        "hidden_size": h, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "qkv_bias": True,
        "out_bias": False, "window": 0,
        "position": PartSpec("rope_half_split", {"head_dim": d, "theta": cfg.rope_theta}),
    })
    ffn = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": i})
    layers = [LayerSpec(mixer=mixer, feed_forward=ffn, norm=norm, block="prenorm")
              for _ in range(cfg.num_hidden_layers)]
    run = [RunEntry(layer=l, cache_group=0, cache_slot=l, write_cache=True)
           for l in range(cfg.num_hidden_layers)]
    groups = [CacheGroupSpec(name="attention", kind="full", slots=cfg.num_hidden_layers, kv_heads=nkv, head_dim=d),
              # Qwen2 keeps no fixed-size state; the slot is still assigned to every request.
              CacheGroupSpec(name="state", kind="state", slots=1, state_shape=(0,))]

    def src(name, *shape):
        return WeightSource(name, tuple(shape))

    bindings = [WeightBinding(("embedding", "weight"), (src("model.embed_tokens.weight", v, h),)),
                WeightBinding(("final_norm", "weight"), (src("model.norm.weight", h),), kind="vector")]
    if cfg.tie_word_embeddings:
        bindings.append(WeightBinding(("lm_head", "weight"), alias_of=("embedding", "weight"),
                                      absent=("lm_head.weight",), why="tie_word_embeddings is true"))
    else:
        bindings.append(WeightBinding(("lm_head", "weight"), (src("lm_head.weight", v, h),)))
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        a = p + "self_attn."
        bindings += [
            WeightBinding(("layer", l, "input_norm", "weight"), (src(p + "input_layernorm.weight", h),), kind="vector"),
            WeightBinding(("layer", l, "post_mixer_norm", "weight"),
                          (src(p + "post_attention_layernorm.weight", h),), kind="vector"),
            WeightBinding(("layer", l, "mixer", "qkv.weight"),
                          (src(a + "q_proj.weight", nq * d, h), src(a + "k_proj.weight", nkv * d, h),
                           src(a + "v_proj.weight", nkv * d, h))),
            WeightBinding(("layer", l, "mixer", "qkv.bias"),
                          (src(a + "q_proj.bias", nq * d), src(a + "k_proj.bias", nkv * d),
                           src(a + "v_proj.bias", nkv * d)), kind="vector"),
            WeightBinding(("layer", l, "mixer", "out.weight"), (src(a + "o_proj.weight", h, nq * d),)),
            WeightBinding(("layer", l, "feed_forward", "gate_up.weight"),
                          (src(p + "mlp.gate_proj.weight", i, h), src(p + "mlp.up_proj.weight", i, h))),
            WeightBinding(("layer", l, "feed_forward", "down.weight"), (src(p + "mlp.down_proj.weight", h, i),)),
        ]
    # random initialisation: matrices and biases N(0, 0.02), norm weights 1 + N(0, 0.01)
    init = {"default": ("normal", 0.0, 0.02), "suffix": {"layernorm.weight": ("normal", 1.0, 0.01),
                                                          "model.norm.weight": ("normal", 1.0, 0.01)}}
    sizes = {"vocab_size": v, "hidden_size": h}
    return ModelPlan(architecture=Qwen2Config.ARCHITECTURE, vocab_size=v, hidden_size=h, layers=layers, run=run,
                     cache_groups=groups, final_norm=norm, bindings=bindings,
                     embedding=PartSpec("token_table", sizes), head=PartSpec("linear", sizes),
                     eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id, init=init)


register_architecture(Qwen2Config.ARCHITECTURE, Qwen2Config, build_qwen2_plan)
