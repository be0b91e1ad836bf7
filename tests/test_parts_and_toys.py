"""Each part alone against the plain implementation, and the generality of the arrangement:
a toy mixer with state of its own, a run order that names a layer twice, and a run entry that
reads another entry's cache; and a second toy architecture whose feed-forward routes tokens to
experts, whose position encoding rotates interleaved pairs and whose norm centres its rows:
all registered, built and stepped from this file alone.

Everything runs on the CPU with the reference kernels and, marked ``gpu``, with the CUDA kernels.
"""
import math
import random
import types
from dataclasses import dataclass

import pytest
import torch

import helpers
import kernel_refs
import plain_model
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import register_architecture
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.parts import (CacheGroupSpec, FeedForward, LayerSpec, Mixer, ModelPlan, Norm, PartSpec,
                                   PositionEncoding, RunEntry, WeightBinding, WeightSource, build_part,
                                   register_feed_forward, register_mixer, register_norm, register_position)
from flexengine_b200.weights import load_model, write_random_model

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]


def provider(device):
    if device == "cpu":
        return kernel_refs
    from flexengine_b200 import ops
    return ops


def fake_ctx(device, dtype, chunks, table=None):
    """A step context for parts that are driven alone: chunks = [(start, n)]."""
    cu = [0]
    for _, n in chunks:
        cu.append(cu[-1] + n)
    ctx = types.SimpleNamespace(ops=provider(device), dtype=dtype, device=torch.device(device))
    ctx.cu_q = torch.tensor(cu, dtype=torch.int32, device=device)
    ctx.q_start = torch.tensor([s for s, _ in chunks], dtype=torch.int32, device=device)
    ctx.token_request = torch.tensor([r for r, (_, n) in enumerate(chunks) for _ in range(n)], dtype=torch.int32, device=device)
    ctx.positions = torch.tensor([p for s, n in chunks for p in range(s, s + n)], dtype=torch.int32, device=device)
    return ctx


# ---- each part alone ----------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
def test_norm_part(device):
    torch.manual_seed(1)
    norm = build_part("norm", PartSpec("rmsnorm", {"hidden_size": 80, "eps": 3e-6}))
    w = (1 + 0.1 * torch.randn(80)).to(device)
    norm.bind({"weight": w})
    residual, delta = torch.randn(6, 80, device=device), torch.randn(6, 80, device=device)
    ctx = fake_ctx(device, torch.float32, [(0, 6)])
    want = plain_model.rms_norm(residual + delta, w, 3e-6)
    got = norm.forward(ctx, residual, delta)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-5)
    rows = torch.tensor([5, 2], dtype=torch.int32, device=device)
    torch.testing.assert_close(norm.forward(ctx, residual, None, rows=rows), want[[5, 2]], atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_feed_forward_part(device):
    torch.manual_seed(2)
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": 48, "intermediate_size": 112}))
    gate, up, down = torch.randn(112, 48) * 0.2, torch.randn(112, 48) * 0.2, torch.randn(48, 112) * 0.2
    ffn.bind({"gate_up.weight": torch.cat([gate, up]).to(device), "down.weight": down.to(device)})
    h = torch.randn(9, 48, device=device)
    got = ffn.forward(fake_ctx(device, torch.float32, [(0, 9)]), h)
    torch.testing.assert_close(got.cpu(), plain_model.swiglu_mlp(h.cpu(), gate, up, down), atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_position_part(device):
    pos = build_part("position", PartSpec("rope_half_split", {"head_dim": 32, "theta": 1e6}))
    inv_freq, rot = pos.rotary_table(device)
    assert rot == 32
    torch.testing.assert_close(inv_freq.cpu(), plain_model.rope_inverse_frequencies(32, 1e6, "cpu"), atol=0, rtol=0)
    assert build_part("position", PartSpec("none")).rotary_table(device) is None


@pytest.mark.parametrize("window", [0, 7])
@pytest.mark.parametrize("device", DEVICES)
def test_attention_mixer_part(device, window):
    """One mixer driven over a paged cache in two portions and a decoded token; compared with the
    plain attention block over the whole sequence."""
    torch.manual_seed(3)
    H, nq, nkv, d, ps = 40, 4, 2, 16, 8
    spec = PartSpec("attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "window": window,
                                  "position": PartSpec("rope_half_split", {"head_dim": d, "theta": 10000.0})})
    mixer = build_part("mixer", spec)
    w = {"q_proj.weight": torch.randn(nq * d, H) * 0.2, "k_proj.weight": torch.randn(nkv * d, H) * 0.2,
         "v_proj.weight": torch.randn(nkv * d, H) * 0.2, "q_proj.bias": torch.randn(nq * d) * 0.1,
         "k_proj.bias": torch.randn(nkv * d) * 0.1, "v_proj.bias": torch.randn(nkv * d) * 0.1,
         "o_proj.weight": torch.randn(H, nq * d) * 0.2}
    mixer.bind({"qkv.weight": torch.cat([w["q_proj.weight"], w["k_proj.weight"], w["v_proj.weight"]]).to(device),
                "qkv.bias": torch.cat([w["q_proj.bias"], w["k_proj.bias"], w["v_proj.bias"]]).to(device),
                "out.weight": w["o_proj.weight"].to(device)})
    need = mixer.cache_need()
    assert need["kind"] == ("window" if window else "full") and need["kv_heads"] == nkv
    T = 21
    h = torch.randn(T, H)
    inv = plain_model.rope_inverse_frequencies(d, 10000.0, "cpu")
    want = plain_model.attention_block(h, w, "", torch.arange(T), nq, nkv, d, inv, window)
    group_spec = CacheGroupSpec("kv", "window" if window else "full", slots=1, kv_heads=nkv, head_dim=d, window=window)
    cache = CacheManager([group_spec], 4, ps, 1, torch.float32, device)
    runner_ctx = ModelRunner.__new__(ModelRunner)                # only build_context is used
    runner_ctx.cache, runner_ctx.ops, runner_ctx.device = cache, provider(device), cache.device
    runner_ctx._ring, runner_ctx._ring_at, runner_ctx.h2d_bytes = [], 0, 0
    runner_ctx.model = types.SimpleNamespace(dtype=torch.float32)
    outs, fed = [], 0
    for n in (9, 11, 1):
        cache.reserve("r", fed + n)
        ctx = runner_ctx.build_context([StepEntry("r", [0] * n, [])])
        outs.append(mixer.forward(ctx, h[fed:fed + n].to(device), RunEntry(0, 0, 0, True)).cpu())
        cache.commit("r", n)
        fed += n
    torch.testing.assert_close(torch.cat(outs), want, atol=2e-5, rtol=2e-5)
    if window:
        assert cache.groups[0].pool.used_pages <= 3               # 21 tokens, window 7: old pages came back


# ---- a toy architecture made of the framework's parts and one mixer of its own ------------------------------
class CumulativeMeanMixer(Mixer):
    """out_i = W . mean(h_0 .. h_i): a causal mixer whose memory is a fixed-size state per request
    (the running sum and the count), kept in a state slot of the cache manager."""

    def __init__(self, hidden_size: int):
        self.hidden_size = hidden_size
        self.proj_weight = None

    def parameter_shapes(self):
        return {"proj.weight": ((self.hidden_size, self.hidden_size), "matrix")}

    def cache_need(self):
        return {"kind": "state", "state_shape": (self.hidden_size + 1,)}

    def forward(self, ctx, h, entry):
        state = ctx.groups[entry.cache_group].state(entry.cache_slot)          # [max_requests, H + 1]
        H = self.hidden_size
        out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        row = 0
        for slot, n in zip(ctx.host_state_slots, ctx.host_lengths):
            x = h[row:row + n].float()
            sums = state[slot, :H] + torch.cumsum(x, 0)
            counts = state[slot, H] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
            out[row:row + n] = sums / counts[:, None]
            if entry.write_cache:
                state[slot, :H] = sums[-1]
                state[slot, H] = counts[-1]
            row += n
        return ctx.ops.linear(out.to(h.dtype), self.proj_weight)


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    eps: float

    @classmethod
    def from_dict(cls, data):
        return cls(int(data["vocab_size"]), int(data["hidden_size"]), float(data["eps"]))


TOY = {"architectures": ["ToyMixedForCausalLM"], "vocab_size": 97, "hidden_size": 48, "eps": 1e-5}
NQ, NKV, D, I = 3, 1, 16, 64


def build_toy_plan(cfg: ToyConfig) -> ModelPlan:
    h, v = cfg.hidden_size, cfg.vocab_size
    norm = PartSpec("rmsnorm", {"hidden_size": h, "eps": cfg.eps})
    attention = PartSpec("attention", {"hidden_size": h, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
                                       "position": PartSpec("rope_half_split", {"head_dim": D, "theta": 500.0})})
    ffn = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": I})
    layers = [LayerSpec(attention, ffn, norm), LayerSpec(PartSpec("toy_cumulative_mean", {"hidden_size": h}), ffn, norm),
              LayerSpec(attention, ffn, norm)]
    # layer 0 writes cache slot 0; the toy layer keeps state; layer 2 READS slot 0 (its own keys are
    # never written); then layer 0 runs a second time with a cache slot of its own
    run = [RunEntry(0, 0, 0, True), RunEntry(1, 1, 0, True), RunEntry(2, 0, 0, False), RunEntry(0, 0, 1, True)]
    groups = [CacheGroupSpec("attention", "full", slots=2, kv_heads=NKV, head_dim=D),
              CacheGroupSpec("running_mean", "state", slots=1, state_shape=(h + 1,))]
    def src(name, *shape):
        return WeightSource(name, tuple(shape))
    bindings = [WeightBinding(("embedding", "weight"), (src("embed.weight", v, h),)),
                WeightBinding(("lm_head", "weight"), alias_of=("embedding", "weight")),
                WeightBinding(("final_norm", "weight"), (src("norm.weight", h),), kind="vector")]
    for l, layer in enumerate(layers):
        p = f"layers.{l}."
        bindings += [WeightBinding(("layer", l, "input_norm", "weight"), (src(p + "norm1.weight", h),), kind="vector"),
                     WeightBinding(("layer", l, "post_mixer_norm", "weight"), (src(p + "norm2.weight", h),), kind="vector"),
                     WeightBinding(("layer", l, "feed_forward", "gate_up.weight"), (src(p + "gate.weight", I, h), src(p + "up.weight", I, h))),
                     WeightBinding(("layer", l, "feed_forward", "down.weight"), (src(p + "down.weight", h, I),))]
        if layer.mixer.kind == "attention":
            bindings += [WeightBinding(("layer", l, "mixer", "qkv.weight"), (src(p + "q.weight", NQ * D, h), src(p + "k.weight", NKV * D, h), src(p + "v.weight", NKV * D, h))),
                         WeightBinding(("layer", l, "mixer", "qkv.bias"), (src(p + "q.bias", NQ * D), src(p + "k.bias", NKV * D), src(p + "v.bias", NKV * D)), kind="vector"),
                         WeightBinding(("layer", l, "mixer", "out.weight"), (src(p + "o.weight", h, NQ * D),))]
        else:
            bindings.append(WeightBinding(("layer", l, "mixer", "proj.weight"), (src(p + "proj.weight", h, h),)))
    init = {"default": ("normal", 0.0, 0.15), "suffix": {"norm1.weight": ("normal", 1.0, 0.05), "norm2.weight": ("normal", 1.0, 0.05),
                                                           "norm.weight": ("normal", 1.0, 0.05)}}
    return ModelPlan("ToyMixedForCausalLM", v, h, layers, run, groups, norm, bindings, init=init)


register_mixer("toy_cumulative_mean", CumulativeMeanMixer)
register_architecture("ToyMixedForCausalLM", ToyConfig, build_toy_plan)


def toy_reference(w: dict, ids) -> torch.Tensor:
    """The toy model over one whole sequence, from the plain implementation's parts."""
    T = len(ids)
    eps = TOY["eps"]
    pos = torch.arange(T)
    inv = plain_model.rope_inverse_frequencies(D, 500.0, "cpu")
    x = w["embed.weight"][torch.tensor(ids)]

    def rename(l):
        p = f"layers.{l}."
        return {"q_proj.weight": w[p + "q.weight"], "k_proj.weight": w[p + "k.weight"], "v_proj.weight": w[p + "v.weight"],
                "q_proj.bias": w[p + "q.bias"], "k_proj.bias": w[p + "k.bias"], "v_proj.bias": w[p + "v.bias"],
                "o_proj.weight": w[p + "o.weight"]}

    def ffn(l, x):
        p = f"layers.{l}."
        h = plain_model.rms_norm(x, w[p + "norm2.weight"], eps)
        return x + plain_model.swiglu_mlp(h, w[p + "gate.weight"], w[p + "up.weight"], w[p + "down.weight"])

    def qkv(l, h):
        m = rename(l)
        q = (h @ m["q_proj.weight"].T + m["q_proj.bias"]).view(T, NQ, D)
        k = (h @ m["k_proj.weight"].T + m["k_proj.bias"]).view(T, NKV, D)
        v = (h @ m["v_proj.weight"].T + m["v_proj.bias"]).view(T, NKV, D)
        return plain_model.apply_rope(q, pos, inv), plain_model.apply_rope(k, pos, inv), v

    # run 0: layer 0, its keys and values are remembered
    h = plain_model.rms_norm(x, w["layers.0.norm1.weight"], eps)
    q, k0, v0 = qkv(0, h)
    x = ffn(0, x + plain_model.causal_gqa_attention(q, k0, v0).reshape(T, -1) @ w["layers.0.o.weight"].T)
    # run 1: the toy mixer
    h = plain_model.rms_norm(x, w["layers.1.norm1.weight"], eps)
    mean = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
    x = ffn(1, x + mean @ w["layers.1.proj.weight"].T)
    # run 2: layer 2's queries over the keys and values of run 0
    h = plain_model.rms_norm(x, w["layers.2.norm1.weight"], eps)
    q, _, _ = qkv(2, h)
    x = ffn(2, x + plain_model.causal_gqa_attention(q, k0, v0).reshape(T, -1) @ w["layers.2.o.weight"].T)
    # run 3: layer 0 again, with keys and values of its own
    h = plain_model.rms_norm(x, w["layers.0.norm1.weight"], eps)
    q, k, v = qkv(0, h)
    x = ffn(0, x + plain_model.causal_gqa_attention(q, k, v).reshape(T, -1) @ w["layers.0.o.weight"].T)
    return plain_model.rms_norm(x, w["norm.weight"], eps) @ w["embed.weight"].T


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("toy"))
    write_random_model(TOY, d, seed=4, dtype="float32")
    return d


@pytest.mark.parametrize("device", DEVICES)
def test_toy_architecture_is_registered_built_and_stepped(toy_dir, device):
    _cfg, plan, model = load_model(toy_dir, "float32", device)
    assert [type(b.mixer).__name__ for b in model.blocks] == ["AttentionMixer", "CumulativeMeanMixer", "AttentionMixer"]
    _, w = plain_model.read_model_folder(toy_dir)
    rng = random.Random(0)
    requests = {f"t{i}": helpers.random_prompt(rng, n, 97) for i, n in enumerate([40, 9, 23, 31, 17])}
    steps = helpers.steps_mixed(requests, rng, live=3, decode_tail=4)
    pages = helpers.peak_pages(steps, 8)
    cache = CacheManager(plan.cache_groups, pages, 8, 3, torch.float32, device)
    runner = ModelRunner(model, cache, ops=provider(device))
    results = helpers.run_steps(runner, steps)
    assert cache.used_pages == 0 and len(cache.free_state_slots) == 3
    for rid, ids in requests.items():
        want = toy_reference(w, ids)
        got = torch.stack([results[(rid, p)] for p in range(len(ids))])
        helpers.assert_logits_close(got, want, "float32", f"toy {rid}")


# ---- a second toy architecture: routed feed-forward, a position encoding and a norm of its own ----------------
class InterleavedRotary(PositionEncoding):
    """Rotation of the pairs (2i, 2i + 1) by position * base^(-2i/d): another pairing than the framework's
    half-split form, so the mixer cannot fuse it and calls ``apply`` before the keys go to the cache."""

    def __init__(self, head_dim: int, base: float):
        self.head_dim, self.base = int(head_dim), float(base)

    def apply(self, ctx, q, k):
        d = self.head_dim
        inv = 1.0 / self.base ** (torch.arange(0, d, 2, dtype=torch.float32, device=q.device) / d)
        ang = ctx.positions.float()[:, None] * inv[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        for x in (q, k):
            even, odd = x[..., 0::2].float(), x[..., 1::2].float()
            new_even, new_odd = even * cos - odd * sin, odd * cos + even * sin       # both before either is written
            x[..., 0::2] = new_even.to(x.dtype)
            x[..., 1::2] = new_odd.to(x.dtype)


class TopTwoExperts(FeedForward):
    """Router logits and softmax in float32, the two best experts per token with weights renormalised to
    one, each expert a two-matrix ReLU network."""

    def __init__(self, hidden_size: int, inner_size: int, experts: int):
        self.hidden_size, self.inner_size, self.experts = int(hidden_size), int(inner_size), int(experts)

    def parameter_shapes(self):
        h, i, e = self.hidden_size, self.inner_size, self.experts
        return {"router.weight": ((e, h), "matrix"), "w_in": ((e, i, h), "matrix"), "w_out": ((e, h, i), "matrix")}

    def forward(self, ctx, h):
        probs = torch.softmax(h.float() @ self.router_weight.float().T, dim=-1)
        top, which = probs.topk(2, dim=-1)
        gate = torch.zeros_like(probs).scatter_(1, which, top / top.sum(-1, keepdim=True))
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        for e in range(self.experts):           # dense over experts: a token's unchosen experts weigh zero
            inner = torch.relu(ctx.ops.linear(h, self.w_in[e]))
            out += gate[:, e:e + 1] * ctx.ops.linear(inner, self.w_out[e]).float()
        return out.to(h.dtype)


class CentredNorm(Norm):
    """(x - mean) / sqrt(var + eps) * weight + bias over the float32 residual stream."""

    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size, self.eps = int(hidden_size), float(eps)

    def parameter_shapes(self):
        return {"weight": ((self.hidden_size,), "vector"), "bias": ((self.hidden_size,), "vector")}

    def forward(self, ctx, residual, delta, rows=None):
        if rows is not None:
            x = residual[rows.long()] + (delta[rows.long()].float() if delta is not None else 0.0)
        else:
            if delta is not None:
                residual += delta.float()
            x = residual
        y = (x - x.mean(-1, keepdim=True)) * torch.rsqrt(x.var(-1, unbiased=False, keepdim=True) + self.eps)
        return (y * self.weight + self.bias).to(ctx.dtype)


@dataclass(frozen=True)
class RoutedConfig:
    vocab_size: int
    width: int
    depth: int
    heads: int
    head_size: int
    inner: int
    experts: int
    rope_base: float
    eps: float

    @classmethod
    def from_dict(cls, data):
        return cls(*(type_(data[name]) for name, type_ in (
            ("vocab_size", int), ("width", int), ("depth", int), ("heads", int), ("head_size", int), ("inner", int),
            ("experts", int), ("rope_base", float), ("eps", float))))


ROUTED = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 61, "width": 40, "depth": 2, "heads": 2,
          "head_size": 16, "inner": 24, "experts": 3, "rope_base": 77.0, "eps": 2e-5}


def build_routed_plan(cfg: RoutedConfig) -> ModelPlan:
    h, v, nq, d = cfg.width, cfg.vocab_size, cfg.heads, cfg.head_size
    norm = PartSpec("toy_centred_norm", {"hidden_size": h, "eps": cfg.eps})
    mixer = PartSpec("attention", {"hidden_size": h, "num_heads": nq, "num_kv_heads": nq, "head_dim": d, "qkv_bias": False,
                                   "position": PartSpec("toy_interleaved_rotary", {"head_dim": d, "base": cfg.rope_base})})
    ffn = PartSpec("toy_top_two_experts", {"hidden_size": h, "inner_size": cfg.inner, "experts": cfg.experts})
    layers = [LayerSpec(mixer, ffn, norm) for _ in range(cfg.depth)]
    run = [RunEntry(l, 0, l, True) for l in range(cfg.depth)]
    groups = [CacheGroupSpec("attention", "full", slots=cfg.depth, kv_heads=nq, head_dim=d)]

    def src(name, *shape):
        return WeightSource(name, tuple(shape))
    bindings = [WeightBinding(("embedding", "weight"), (src("tok.weight", v, h),)),
                WeightBinding(("lm_head", "weight"), (src("out.weight", v, h),)),
                WeightBinding(("final_norm", "weight"), (src("ln_f.weight", h),), kind="vector"),
                WeightBinding(("final_norm", "bias"), (src("ln_f.bias", h),), kind="vector")]
    for l in range(cfg.depth):
        p = f"blocks.{l}."
        for part, short in (("input_norm", "ln1"), ("post_mixer_norm", "ln2")):
            bindings += [WeightBinding(("layer", l, part, "weight"), (src(p + short + ".weight", h),), kind="vector"),
                         WeightBinding(("layer", l, part, "bias"), (src(p + short + ".bias", h),), kind="vector")]
        bindings += [WeightBinding(("layer", l, "mixer", "qkv.weight"), (src(p + "qkv.weight", 3 * nq * d, h),)),
                     WeightBinding(("layer", l, "mixer", "out.weight"), (src(p + "proj.weight", h, nq * d),)),
                     WeightBinding(("layer", l, "feed_forward", "router.weight"), (src(p + "router.weight", cfg.experts, h),)),
                     WeightBinding(("layer", l, "feed_forward", "w_in"), (src(p + "experts.w_in", cfg.experts, cfg.inner, h),)),
                     WeightBinding(("layer", l, "feed_forward", "w_out"), (src(p + "experts.w_out", cfg.experts, h, cfg.inner),))]
    init = {"default": ("normal", 0.0, 0.2), "suffix": {".weight_of_norm": ("normal", 1.0, 0.05)}}
    init["suffix"].update({f"{n}.weight": ("normal", 1.0, 0.05) for n in ("ln1", "ln2", "ln_f")})
    init["suffix"].update({f"{n}.bias": ("normal", 0.0, 0.05) for n in ("ln1", "ln2", "ln_f")})
    init["suffix"]["router.weight"] = ("normal", 0.0, 1.0)
    return ModelPlan("ToyRoutedForCausalLM", v, h, layers, run, groups, norm, bindings, init=init)


register_position("toy_interleaved_rotary", InterleavedRotary)
register_feed_forward("toy_top_two_experts", TopTwoExperts)
register_norm("toy_centred_norm", CentredNorm)
register_architecture("ToyRoutedForCausalLM", RoutedConfig, build_routed_plan)


def routed_reference(w: dict, ids) -> torch.Tensor:
    """The routed toy over one whole sequence, written out plainly: no cache, no parts of the framework."""
    cfg = ROUTED
    T, nq, d, eps = len(ids), cfg["heads"], cfg["head_size"], cfg["eps"]

    def norm(x, name):
        y = (x - x.mean(-1, keepdim=True)) / torch.sqrt(x.var(-1, unbiased=False, keepdim=True) + eps)
        return y * w[name + ".weight"] + w[name + ".bias"]

    def rotate(x):                                            # [T, heads, d], pairs (2i, 2i + 1)
        inv = 1.0 / cfg["rope_base"] ** (torch.arange(0, d, 2, dtype=torch.float32) / d)
        ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = torch.empty_like(x)
        out[..., 0::2] = x[..., 0::2] * cos - x[..., 1::2] * sin
        out[..., 1::2] = x[..., 1::2] * cos + x[..., 0::2] * sin
        return out

    x = w["tok.weight"][torch.tensor(ids)]
    for l in range(cfg["depth"]):
        p = f"blocks.{l}."
        q, k, v = (norm(x, p + "ln1") @ w[p + "qkv.weight"].T).view(T, 3, nq, d).unbind(1)
        x = x + plain_model.causal_gqa_attention(rotate(q), rotate(k), v).reshape(T, -1) @ w[p + "proj.weight"].T
        h = norm(x, p + "ln2")
        probs = torch.softmax(h @ w[p + "router.weight"].T, dim=-1)
        delta = torch.zeros_like(x)
        for t in range(T):
            top, which = probs[t].topk(2)
            for weight, e in zip(top / top.sum(), which.tolist()):
                delta[t] += weight * (torch.relu(h[t] @ w[p + "experts.w_in"][e].T) @ w[p + "experts.w_out"][e].T)
        x = x + delta
    return norm(x, "ln_f") @ w["out.weight"].T


@pytest.fixture(scope="module")
def routed_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("routed"))
    write_random_model(ROUTED, d, seed=9, dtype="float32")
    return d


@pytest.mark.parametrize("device", DEVICES)
def test_routed_toy_with_its_own_feed_forward_position_encoding_and_norm(routed_dir, device):
    _cfg, plan, model = load_model(routed_dir, "float32", device)
    block = model.blocks[0]
    assert type(block.feed_forward).__name__ == "TopTwoExperts" and type(block.mixer.position).__name__ == "InterleavedRotary"
    assert block.mixer.position.applies_itself and type(model.final_norm).__name__ == "CentredNorm"
    _, w = plain_model.read_model_folder(routed_dir)
    rng = random.Random(1)
    requests = {f"m{i}": helpers.random_prompt(rng, n, ROUTED["vocab_size"]) for i, n in enumerate([33, 12, 26, 19])}
    steps = helpers.steps_mixed(requests, rng, live=3, decode_tail=5)
    cache = CacheManager(plan.cache_groups, helpers.peak_pages(steps, 4), 4, 3, torch.float32, device)
    runner = ModelRunner(model, cache, ops=provider(device))
    results = helpers.run_steps(runner, steps)
    assert cache.used_pages == 0
    for rid, ids in requests.items():
        want = routed_reference(w, ids)
        got = torch.stack([results[(rid, p)] for p in range(len(ids))])
        helpers.assert_logits_close(got, want, "float32", f"routed {rid}")
    # the router did route: not every token chose the same pair of experts
    h = torch.randn(50, ROUTED["width"], device=device)
    chosen = (h @ block.feed_forward.router_weight.float().T).topk(2, dim=-1).indices.sort(-1).values
    assert len({tuple(c) for c in chosen.tolist()}) > 1


# ---- a third toy: full attention in one layer, a sliding window in the other, each with pages of its own ----------
@dataclass(frozen=True)
class WindowedConfig:
    vocab_size: int
    hidden_size: int
    window: int

    @classmethod
    def from_dict(cls, data):
        return cls(int(data["vocab_size"]), int(data["hidden_size"]), int(data["window"]))


WINDOWED = {"architectures": ["ToyWindowedForCausalLM"], "vocab_size": 211, "hidden_size": 128, "window": 70}
WQ, WKV, WD, WI = 8, 2, 64, 192           # head size 64 and group 4: portions of 64 queries take the tcgen05 kernel


def build_windowed_plan(cfg: WindowedConfig) -> ModelPlan:
    h, v = cfg.hidden_size, cfg.vocab_size
    norm = PartSpec("rmsnorm", {"hidden_size": h, "eps": 1e-5})
    position = PartSpec("rope_half_split", {"head_dim": WD, "theta": 30000.0})
    def attention(window):
        return PartSpec("attention", {"hidden_size": h, "num_heads": WQ, "num_kv_heads": WKV, "head_dim": WD,
                                      "window": window, "position": position})
    ffn = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": WI})
    layers = [LayerSpec(attention(0), ffn, norm), LayerSpec(attention(cfg.window), ffn, norm)]
    run = [RunEntry(0, 0, 0, True), RunEntry(1, 1, 0, True)]
    groups = [CacheGroupSpec("all_keys", "full", slots=1, kv_heads=WKV, head_dim=WD),
              CacheGroupSpec("recent_keys", "window", slots=1, kv_heads=WKV, head_dim=WD, window=cfg.window)]
    def src(name, *shape):
        return WeightSource(name, tuple(shape))
    bindings = [WeightBinding(("embedding", "weight"), (src("embed.weight", v, h),)),
                WeightBinding(("lm_head", "weight"), alias_of=("embedding", "weight")),
                WeightBinding(("final_norm", "weight"), (src("norm.weight", h),), kind="vector")]
    for l in range(2):
        p = f"layers.{l}."
        bindings += [WeightBinding(("layer", l, "input_norm", "weight"), (src(p + "norm1.weight", h),), kind="vector"),
                     WeightBinding(("layer", l, "post_mixer_norm", "weight"), (src(p + "norm2.weight", h),), kind="vector"),
                     WeightBinding(("layer", l, "feed_forward", "gate_up.weight"), (src(p + "gate.weight", WI, h), src(p + "up.weight", WI, h))),
                     WeightBinding(("layer", l, "feed_forward", "down.weight"), (src(p + "down.weight", h, WI),)),
                     WeightBinding(("layer", l, "mixer", "qkv.weight"), (src(p + "q.weight", WQ * WD, h), src(p + "k.weight", WKV * WD, h), src(p + "v.weight", WKV * WD, h))),
                     WeightBinding(("layer", l, "mixer", "qkv.bias"), (src(p + "q.bias", WQ * WD), src(p + "k.bias", WKV * WD), src(p + "v.bias", WKV * WD)), kind="vector"),
                     WeightBinding(("layer", l, "mixer", "out.weight"), (src(p + "o.weight", h, WQ * WD),))]
    init = {"default": ("normal", 0.0, 0.08), "suffix": {"norm1.weight": ("normal", 1.0, 0.05), "norm2.weight": ("normal", 1.0, 0.05),
                                                           "norm.weight": ("normal", 1.0, 0.05)}}
    return ModelPlan("ToyWindowedForCausalLM", v, h, layers, run, groups, norm, bindings, init=init)


register_architecture("ToyWindowedForCausalLM", WindowedConfig, build_windowed_plan)


def windowed_reference(w: dict, ids) -> torch.Tensor:
    T = len(ids)
    pos = torch.arange(T)
    inv = plain_model.rope_inverse_frequencies(WD, 30000.0, "cpu")
    x = w["embed.weight"].float()[torch.tensor(ids)]
    for l, window in enumerate((0, WINDOWED["window"])):
        p = f"layers.{l}."
        names = {"q_proj.weight": w[p + "q.weight"], "k_proj.weight": w[p + "k.weight"], "v_proj.weight": w[p + "v.weight"],
                 "q_proj.bias": w[p + "q.bias"], "k_proj.bias": w[p + "k.bias"], "v_proj.bias": w[p + "v.bias"],
                 "o_proj.weight": w[p + "o.weight"]}
        x = x + plain_model.attention_block(plain_model.rms_norm(x, w[p + "norm1.weight"].float(), 1e-5), names, "", pos, WQ, WKV, WD, inv, window)
        x = x + plain_model.swiglu_mlp(plain_model.rms_norm(x, w[p + "norm2.weight"].float(), 1e-5), w[p + "gate.weight"].float(),
                                       w[p + "up.weight"].float(), w[p + "down.weight"].float())
    return plain_model.rms_norm(x, w["norm.weight"].float(), 1e-5) @ w["embed.weight"].float().T


@pytest.mark.parametrize("device,dtype", [pytest.param("cpu", "float32", id="cpu"),
                                          pytest.param("cuda:0", "float32", id="gpu-float32", marks=pytest.mark.gpu),
                                          pytest.param("cuda:0", "bfloat16", id="gpu-bfloat16", marks=pytest.mark.gpu)])
def test_windowed_toy_gives_pages_back_and_matches_the_plain_implementation(tmp_path_factory, device, dtype):
    """Long prompts in portions (some of 64 queries and more: the tcgen05 kernel in bfloat16), decoded tails, mixed
    batches; the window group holds only the pages its window still reaches."""
    folder = str(tmp_path_factory.mktemp("windowed"))
    write_random_model(WINDOWED, folder, seed=6, dtype="bfloat16")
    _cfg, plan, model = load_model(folder, dtype, device)
    _, w = plain_model.read_model_folder(folder)
    rng = random.Random(4)
    requests = {f"w{i}": helpers.random_prompt(rng, n, WINDOWED["vocab_size"]) for i, n in enumerate([330, 90, 201])}
    steps = helpers.steps_mixed(requests, rng, live=3, decode_tail=5)
    torch_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    cache = CacheManager(plan.cache_groups, helpers.peak_pages(steps, 8), 8, 3, torch_dtype, device)
    runner = ModelRunner(model, cache, ops=provider(device))
    window_pool = cache.groups[1].pool
    most_window_pages = 0
    results = {}
    for entries, ended in steps:
        out = runner.step([StepEntry(rid, toks, want) for rid, toks, want in entries])
        row = 0
        for rid, toks, want in entries:
            start = cache.tokens_of(rid) - len(toks)
            for place in want:
                results[(rid, start + place)] = out[row].float().cpu()
                row += 1
        most_window_pages = max(most_window_pages, window_pool.used_pages)
        for rid in ended:
            runner.finish(rid)
    assert cache.used_pages == 0
    # three live requests never hold more than their windows' worth (and the portion in flight) in the window group
    assert most_window_pages < helpers.peak_pages(steps, 8)
    for rid, ids in requests.items():
        want = windowed_reference(w, ids)
        got = torch.stack([results[(rid, p)] for p in range(len(ids))])
        helpers.assert_logits_close(got, want, dtype, f"windowed {rid}")
    if device != "cpu":
        from flexengine_b200 import ops
        ops.check_status(device)
