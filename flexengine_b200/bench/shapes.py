"""The model shapes the benchmarks run, and the arithmetic of their rooflines.

The shapes are Qwen2.5 configurations as config.json would give them; weights are random.  ``decode_bytes`` is
what a decode step has to read (every weight it uses once, and the cache of the live requests); ``prefill_flops``
what a prompt costs (linear layers, causal attention, the vocabulary product of the one wanted row).
"""
from __future__ import annotations


def _qwen2(layers, hidden, heads, kv_heads, intermediate, vocab, eps, tied):
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=layers, hidden_size=hidden,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=128, intermediate_size=intermediate,
                vocab_size=vocab, rope_theta=1000000.0, rms_norm_eps=eps, max_position_embeddings=32768,
                tie_word_embeddings=tied, use_sliding_window=False, hidden_act="silu", eos_token_id=None)


SHAPES = {
    "7b": _qwen2(28, 3584, 28, 4, 18944, 152064, 1e-6, False),
    "1.5b": _qwen2(28, 1536, 12, 2, 8960, 151936, 1e-6, True),
    "14b": _qwen2(48, 5120, 40, 8, 13824, 152064, 1e-5, False),
}
SEVEN_B = SHAPES["7b"]
PROMPT_LEN = 2048          # the headline workload: prompts of this many tokens ...
CONTEXT_LEN = 4096         # ... under this context limit ...
PAGE = 16                  # ... in pages of this many tokens
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def linear_params(cfg) -> int:
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kd = cfg["num_key_value_heads"] * cfg["head_dim"]
    return cfg["num_hidden_layers"] * ((qd + 2 * kd) * h + qd * h + 3 * h * i)


def kv_bytes_per_token(cfg) -> int:
    return 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * cfg["num_hidden_layers"] * 2


def decode_bytes(cfg, batch, ctx) -> float:
    h, v = cfg["hidden_size"], cfg["vocab_size"]
    weights = 2 * (linear_params(cfg) + v * h) + 2 * batch * h           # matrices + vocabulary matrix + embedding rows
    return weights + batch * ctx * kv_bytes_per_token(cfg)


def prefill_flops(cfg, tokens, start=0) -> float:
    """``tokens`` prompt tokens after ``start`` cached ones, one row of logits."""
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    keys = tokens * start + tokens * (tokens + 1) / 2                       # causal: (query, key) pairs
    attention = cfg["num_hidden_layers"] * 2 * 2 * qd * keys
    return 2.0 * linear_params(cfg) * tokens + attention + 2.0 * cfg["vocab_size"] * cfg["hidden_size"]


def flat_config(cfg, **more) -> dict:
    """The sizes under the short names the benchmark lines use (flat: nested values are lost in the record)."""
    out = {"layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
           "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
           "vocab": cfg["vocab_size"]}
    out.update(more)
    return out
