"""A plain, slow implementation of the Qwen2.5 decoder: whole sequences, no cache, one
function per part, float32 PyTorch on whatever device the weights are on.

It shares no code with ``flexengine_b200``: weights are read with the ``safetensors``
library (not the framework's reader), the configuration is the raw config.json
dictionary.  Every function is written from the reference's formulas and cites them by
the file's path within the reference project.

This file rests on the formulas AND on a one-time comparison with the reference's own code,
which imports on the CPU: ``tests/golden/make_golden.py`` drove the reference's ``Qwen2Adapter``
over tiny fixed-weight models, its own ``FakeRMS`` / ``FakeMLP`` modules on fixed inputs and its
whole synthetic ``FakeQwen``, and committed the outputs; ``tests/test_plain_model.py`` compares
this file with them (the whole model at the reference's bar of 1e-5, the two parts at 1e-6).
"""
from __future__ import annotations

import json
import math
import os

import torch


# ---------------------------------------------------------------------------------------------
# reading a model folder
# ---------------------------------------------------------------------------------------------
def read_model_folder(model_dir: str, device="cpu", keep_dtype: bool = False):
    """config.json as a dict and every tensor of model.safetensors by name, as float32
    (bfloat16 values convert exactly)."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf8") as f:
        config = json.load(f)
    tensors = load_file(os.path.join(model_dir, "model.safetensors"))
    if not keep_dtype:
        tensors = {k: v.to(torch.float32) for k, v in tensors.items()}
    return config, {k: v.to(device) for k, v in tensors.items()}


# ---------------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, in float32.
    src/flexengine/inference/kernels/rmsnorm.py:24-32 (variance = sum(x*x)/H; result =
    values * rsqrt(variance + EPS) * weights); used at src/flexengine/inference/models/qwen2.py:67-71."""
    x = x.float()
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight.float()


def rope_inverse_frequencies(head_dim: int, theta: float, device) -> torch.Tensor:
    """inv_freq = 1 / theta ** (arange(0, d, 2) / d), float32.
    src/flexengine/inference/models/qwen2.py:46."""
    return 1.0 / theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[d/2:], x[:d/2]).  src/flexengine/inference/models/qwen2.py:15-17."""
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [T, heads, d]: x*cos + rotate_half(x)*sin with angles = positions[:,None] * inv_freq[None,:],
    emb = cat(angles, angles).  src/flexengine/inference/models/qwen2.py:73-77."""
    freqs = positions.float().unsqueeze(1) * inv_freq.unsqueeze(0)
    emb = torch.cat([freqs, freqs], dim=-1)
    cos, sin = emb.cos().unsqueeze(1), emb.sin().unsqueeze(1)
    return x * cos + rotate_half(x) * sin


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0,
                         scale: float | None = None) -> torch.Tensor:
    """q [T, nq, d], k and v [T, nkv, d] of ONE whole sequence (positions 0..T-1) -> [T, nq, d].
    scores = q.k / sqrt(d); key t visible to query p iff t <= p (and t > p - window when a
    window is given); softmax over keys; query head h reads key/value head h // (nq/nkv)
    (repeat_interleave).  src/flexengine/inference/attention/paged.py:25-35 (mask
    key_pos <= positions, scale 1/sqrt(d), repeat_interleave(ratio)) and :50-70 (the same in float32)."""
    T, nq, d = q.shape
    ratio = nq // k.shape[1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    kh = k.float().repeat_interleave(ratio, dim=1)
    vh = v.float().repeat_interleave(ratio, dim=1)
    scores = torch.einsum("qhd,thd->hqt", q.float(), kh) * scale
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window and window > 0:
        visible = visible & (pos[None, :] > pos[:, None] - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    return torch.einsum("hqt,thd->qhd", weights, vh)


def swiglu_mlp(h: torch.Tensor, gate_w, up_w, down_w) -> torch.Tensor:
    """down( silu(gate(h)) * up(h) ), no biases.
    tests/unit/test_synthetic_qwen.py:30-36 of the reference (the product code calls the
    module opaquely, src/flexengine/inference/models/qwen2.py:130)."""
    gate = h @ gate_w.float().T
    up = h @ up_w.float().T
    return (torch.nn.functional.silu(gate) * up) @ down_w.float().T


def attention_block(h, w, prefix: str, positions, nq, nkv, d, inv_freq, window=0):
    """q/k/v projections with bias, view as heads, rope on q and k, attention, output projection
    without bias.  src/flexengine/inference/models/qwen2.py:98-102,128-129."""
    T = h.shape[0]
    q = (h @ w[prefix + "q_proj.weight"].float().T + w[prefix + "q_proj.bias"].float()).view(T, nq, d)
    k = (h @ w[prefix + "k_proj.weight"].float().T + w[prefix + "k_proj.bias"].float()).view(T, nkv, d)
    v = (h @ w[prefix + "v_proj.weight"].float().T + w[prefix + "v_proj.bias"].float()).view(T, nkv, d)
    q = apply_rope(q, positions, inv_freq)
    k = apply_rope(k, positions, inv_freq)
    o = causal_gqa_attention(q, k, v, window)
    return o.reshape(T, nq * d) @ w[prefix + "o_proj.weight"].float().T


# ---------------------------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------------------------
def config_sizes(config: dict):
    nq = int(config["num_attention_heads"])
    nkv = int(config.get("num_key_value_heads") or nq)
    d = int(config.get("head_dim") or config["hidden_size"] // nq)        # qwen2.py:36
    theta = float(config.get("rope_theta") or 10000.0)                     # qwen2.py:42-45
    return nq, nkv, d, theta, float(config["rms_norm_eps"]), int(config["num_hidden_layers"])


@torch.no_grad()
def forward_logits(config: dict, w: dict, ids) -> torch.Tensor:
    """Logits [len(ids), vocab] at every position of one whole sequence.
    Decoder loop: src/flexengine/inference/models/qwen2.py:94-135 —
    x = embed(ids); per layer: x += o_proj(attn(norm(x))); x += mlp(norm(x)); logits = lm_head(norm(x)).
    Tied embeddings: lm_head shares embed_tokens.weight."""
    nq, nkv, d, theta, eps, layers = config_sizes(config)
    dev = w["model.embed_tokens.weight"].device
    ids = torch.as_tensor(ids, dtype=torch.long, device=dev)
    positions = torch.arange(len(ids), device=dev)
    inv_freq = rope_inverse_frequencies(d, theta, dev)
    x = w["model.embed_tokens.weight"].float()[ids]
    for l in range(layers):
        p = f"model.layers.{l}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        x = x + attention_block(h, w, p + "self_attn.", positions, nq, nkv, d, inv_freq)
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = rms_norm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.float().T


@torch.no_grad()
def greedy_generate(config: dict, w: dict, prompt, count: int) -> list:
    """``count`` greedy tokens after ``prompt``: argmax of the last position's logits, appended,
    the whole sequence run again each time (src/flexengine/engine/sampling/sampler.py:12-13)."""
    ids = list(prompt)
    out = []
    for _ in range(count):
        token = int(forward_logits(config, w, ids)[-1].argmax().item())
        out.append(token)
        ids.append(token)
    return out


# ---------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------
def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int) -> torch.Tensor:
    """The probabilities the reference draws from: softmax(logits / T) over the k largest (all
    when k == 0 or k >= vocab).  src/flexengine/engine/sampling/sampler.py:16-22."""
    x = logits.detach().to(device="cpu", dtype=torch.float32) / temperature
    probs = torch.zeros_like(x)
    if 0 < top_k < x.numel():
        vals, idxs = torch.topk(x, top_k)
        probs[idxs] = torch.softmax(vals, dim=-1)
    else:
        probs = torch.softmax(x, dim=-1)
    return probs
