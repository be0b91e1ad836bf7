"""Plain PyTorch references of every kernel, with the signatures of ``flexengine_b200.ops``.

Two uses: the ``-m gpu`` tests compare each CUDA kernel with its function here, and the
CPU tests hand this module to the engine as its kernel provider, so that the step
function, cache and scheduler are exercised here without a GPU.  Intermediate math is
float32; results are rounded to the dtype the kernel returns.
"""
from __future__ import annotations

import math

import torch


def embedding(token_ids, table):
    return table[token_ids.long()].float()


def carry_tokens(token_ids, rows, sources, previous):
    keep = rows >= 0
    token_ids[rows[keep].long()] = previous[sources[keep].long()].to(token_ids.dtype)


def add_rmsnorm(residual, delta, weight, eps, out_dtype, rows=None, upcoming=None):
    if rows is None:
        if delta is not None:
            residual += delta.float()
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return (x * torch.rsqrt(variance + eps) * weight.float()).to(out_dtype)


def linear(x, w, bias=None, out_float32=False):
    y = x.float() @ w.float().T
    if bias is not None:
        y = y + bias.float()
    return y if out_float32 else y.to(x.dtype)


def swiglu(gate_up, intermediate):
    g = gate_up[:, :intermediate].float()
    u = gate_up[:, intermediate:].float()
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear_swiglu(x, w, intermediate):
    return swiglu(linear(x, w), intermediate)


def qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache,
                        nq, nkv, d, page_size, src=None):
    """``src``: the projection in float32 when it was kept so; else ``qkv`` is rewritten in place."""
    T = qkv.shape[0]
    x = (qkv if src is None else src).float()
    if bias is not None:
        x = x + bias.float()
    x = x.view(T, nq + 2 * nkv, d)
    if inv_freq is not None and rot > 0:
        ang = positions.float()[:, None] * inv_freq.float()[None, :]          # [T, rot/2]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        qk = x[:, :nq + nkv]
        a, b = qk[..., :rot // 2].clone(), qk[..., rot // 2:rot].clone()
        qk[..., :rot // 2] = a * cos - b * sin
        qk[..., rot // 2:rot] = b * cos + a * sin
    out = x.to(qkv.dtype)
    qkv.copy_(out.view(T, -1))
    if slot_mapping is not None:
        slots = slot_mapping.long()
        keep = slots >= 0
        page, off = slots[keep] // page_size, slots[keep] % page_size
        k_cache[page, :, off] = out[keep, nq:nq + nkv]
        v_cache[page, :, off] = out[keep, nq + nkv:]


def qkv_projection(h, w, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size):
    """The product stays float32 until bias and rotation are in: one rounding, whatever the number of rows."""
    product = linear(h, w, out_float32=True)
    qkv = torch.empty(product.shape, dtype=h.dtype, device=h.device)
    qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size,
                        src=product)
    return qkv


def paged_attention(qkv, k_cache, v_cache, block_table, ctx, nq, nkv, d, page_size, scale, window, upcoming=None):
    T = qkv.shape[0]
    out = torch.zeros(T, nq * d, dtype=qkv.dtype, device=qkv.device)
    q_all = qkv[:, :nq * d].float().view(T, nq, d)
    cu = ctx.cu_q.tolist()
    starts = ctx.q_start.tolist()
    ratio = nq // nkv
    for r in range(len(starts)):
        q = q_all[cu[r]:cu[r + 1]]
        n = q.shape[0]
        length = starts[r] + n
        lo = max(0, starts[r] - window + 1) if window > 0 else 0
        lo_page = lo // page_size
        pages = block_table[r, lo_page:-(-length // page_size)].long()
        k = k_cache[pages].float().permute(0, 2, 1, 3).reshape(-1, nkv, d)      # [tokens, nkv, d]
        v = v_cache[pages].float().permute(0, 2, 1, 3).reshape(-1, nkv, d)
        key_pos = torch.arange(lo_page * page_size, lo_page * page_size + k.shape[0], device=q.device)
        q_pos = torch.arange(starts[r], length, device=q.device)
        visible = (key_pos[None, :] <= q_pos[:, None]) & (key_pos[None, :] < length)
        if window > 0:
            visible &= key_pos[None, :] > q_pos[:, None] - window
        kh = k.repeat_interleave(ratio, dim=1)
        vh = v.repeat_interleave(ratio, dim=1)
        scores = torch.einsum("qhd,thd->hqt", q, kh) * scale
        scores = scores.masked_fill(~visible[None], float("-inf"))
        w = torch.softmax(scores, dim=-1)
        w = torch.where(visible[None], w, torch.zeros_like(w))
        o = torch.einsum("hqt,thd->qhd", w, vh)
        out[cu[r]:cu[r + 1]] = o.reshape(n, nq * d).to(qkv.dtype)
    return out


# ---- sampling ----------------------------------------------------------------------------------
MASK64 = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return x ^ (x >> 31)


def uniform_from(seed: int, draw: int) -> float:
    """The uniform number in [0, 1) of request seed ``seed`` at its ``draw``-th sampled token."""
    bits = splitmix64((splitmix64(seed & MASK64) + draw) & MASK64)
    return (bits >> 40) * (1.0 / (1 << 24))


def sample(logits, temperature, top_k, seed, draw):
    """Greedy rows (temperature 0): lowest index of the maximum.  Other rows: x = logits / T; keep
    the k largest (ties by lowest index) when 0 < k < V; p = softmax over the kept; the token is
    the first index whose cumulative probability (in index order) exceeds u * total."""
    R, V = logits.shape
    out = torch.zeros(R, dtype=torch.int32)
    for r in range(R):
        row = logits[r].detach().float().cpu()
        t = float(temperature[r])
        if t == 0.0:
            out[r] = int(torch.nonzero(row == row.max())[0])
            continue
        x = row / t
        k = int(top_k[r])
        keep = torch.ones(V, dtype=torch.bool)
        if 0 < k < V:
            order = torch.sort(x, descending=True, stable=True).indices[:k]
            keep = torch.zeros(V, dtype=torch.bool)
            keep[order] = True
        e = torch.where(keep, torch.exp(x - x[keep].max()), torch.zeros_like(x)).double()
        cum = torch.cumsum(e, 0)
        u = uniform_from(int(seed[r]), int(draw[r]))
        target = u * float(cum[-1])
        idx = int(torch.searchsorted(cum, torch.tensor(target, dtype=torch.float64), right=True))
        idx = min(idx, V - 1)
        while not keep[idx]:
            idx -= 1
        out[r] = idx
    return out.to(logits.device)
