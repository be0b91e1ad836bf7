"""Makes ``reference_logits.npz``: outputs of the reference's OWN code on tiny models.

Run once, on the CPU, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

Three kinds of record, each computed by code imported from the reference checkout:

* ``<config>/<backend>/...``: last-token logits of ``Qwen2Adapter`` + ``PagedKVCache``
  (src/flexengine/inference/models/qwen2.py:79-136, src/flexengine/engine/kv_cache/allocator.py)
  over the tiny configurations of the tests, with both CPU attention backends, whole prompts and a
  mixed batch (a prefill portion beside a decoded token).  The module tree that the adapter walks
  is built here; its norm and feed-forward modules are restatements (the adapter calls Hugging
  Face modules there), which is why the next two records exist.
* ``parts/rms/*`` and ``parts/mlp/*``: the reference's own ``FakeRMS`` and ``FakeMLP`` modules
  (tests/unit/test_synthetic_qwen.py:19-36) run on fixed inputs (the feed-forward's biases zeroed:
  Qwen2.5 has none).  The plain implementation's ``rms_norm`` and ``swiglu_mlp`` are held to them.
* ``fake/*``: the reference's whole ``FakeQwen`` (tests/unit/test_synthetic_qwen.py:39-61: its own
  norm, feed-forward and layer modules) with fixed weights, the biases that Qwen2.5 lacks zeroed,
  through the adapter: whole, in portions and beside another request.

Weights come from ``fixed_weights``: an integer hash per element, twelve uniforms summed, scaled and
rounded to bfloat16.  Integer and basic IEEE arithmetic only, so every machine makes the same model
and the test never has to skip; the checksum in the file guards it.  ``transformers`` is not imported.
"""
import hashlib
import os
import sys
import types

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))      # helpers imports the package for other tests
sys.path.insert(0, os.path.dirname(HERE))

import helpers  # noqa: E402

SEED = 2024
PROMPTS = {"A": [5, 17, 33], "B": [1, 40, 77], "C": [3, 50], "D": [4, 70]}
FAKE_CONFIG = dict(model_type="qwen2", num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=8, intermediate_size=64, vocab_size=50, rope_theta=1000000.0,
                   rms_norm_eps=1e-6, tie_word_embeddings=False)
FAKE_PROMPTS = [[2, 5, 3, 8, 9, 4, 7, 12, 10], [16, 8, 9, 2]]


# ---- weights that every machine draws alike ----------------------------------------------------------
def _mix(z: np.ndarray) -> np.ndarray:
    """splitmix64's output function on uint64 arrays (wrapping arithmetic)."""
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def fixed_tensor(name: str, shape, seed: int, mean: float, std: float) -> torch.Tensor:
    """About N(mean, std^2): twelve uniforms from an integer hash of (seed, name, element, k), summed, minus six;
    float32, then rounded to bfloat16 and widened again (exactly representable in both)."""
    count = int(np.prod(shape)) if len(shape) else 1
    key = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")
    with np.errstate(over="ignore"):
        base = np.uint64(key) + np.arange(count, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        total = np.zeros(count, dtype=np.float64)
        for k in range(12):
            bits = _mix(base + np.uint64(k + 1) * np.uint64(0xD1B54A32D192ED03))
            total += (bits >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))
    values = ((total - 6.0) * std + mean).astype(np.float32).reshape(shape)
    return torch.from_numpy(values).to(torch.bfloat16).to(torch.float32)


def tensor_shapes(config: dict) -> dict:
    """Names and shapes of a Qwen2.5 checkpoint (the attribute paths of src/flexengine/inference/models/qwen2.py:94-135)."""
    h, i, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    qd = config["num_attention_heads"] * config["head_dim"]
    kd = config["num_key_value_heads"] * config["head_dim"]
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,)}
    if not config.get("tie_word_embeddings"):
        shapes["lm_head.weight"] = (v, h)
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes.update({
            p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
            p + "self_attn.q_proj.weight": (qd, h), p + "self_attn.q_proj.bias": (qd,),
            p + "self_attn.k_proj.weight": (kd, h), p + "self_attn.k_proj.bias": (kd,),
            p + "self_attn.v_proj.weight": (kd, h), p + "self_attn.v_proj.bias": (kd,),
            p + "self_attn.o_proj.weight": (h, qd),
            p + "mlp.gate_proj.weight": (i, h), p + "mlp.up_proj.weight": (i, h), p + "mlp.down_proj.weight": (h, i)})
    return shapes


def fixed_weights(config: dict, seed: int = SEED) -> dict:
    """Matrices and biases about N(0, 0.02), norm weights about 1 + N(0, 0.01)."""
    return {name: fixed_tensor(name, shape, seed, 1.0 if "norm" in name else 0.0, 0.01 if "norm" in name else 0.02)
            for name, shape in tensor_shapes(config).items()}


def weights_checksum(tensors: dict) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].float().contiguous().numpy().tobytes())
    return h.hexdigest()


def prompts_for(name: str) -> list:
    """Token ids from the same integer hash (no library generator)."""
    vocab = helpers.CONFIGS[name]["vocab_size"]
    out = []
    for n in PROMPTS[name]:
        with np.errstate(over="ignore"):
            bits = _mix(np.uint64(1234567 + n) + np.arange(n, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15))
        out.append([int(b % np.uint64(vocab)) for b in bits])
    return out


def part_inputs():
    """Fixed inputs and weights of the two part records."""
    x = fixed_tensor("parts.x", (7, 24), SEED, 0.0, 1.5)
    rms_w = fixed_tensor("parts.rms.weight", (24,), SEED, 1.0, 0.3)
    gate = fixed_tensor("parts.mlp.gate", (48, 24), SEED, 0.0, 0.3)
    up = fixed_tensor("parts.mlp.up", (48, 24), SEED, 0.0, 0.3)
    down = fixed_tensor("parts.mlp.down", (24, 48), SEED, 0.0, 0.3)
    return x, rms_w, gate, up, down


# ---- the module tree the adapter walks, around our tensors ------------------------------------------------
class RMS(nn.Module):
    def __init__(self, weight, eps):
        super().__init__()
        self.weight = nn.Parameter(weight)
        self.variance_epsilon = eps

    def forward(self, x):
        f = x.float()
        return (f * torch.rsqrt(f.square().mean(-1, keepdim=True) + self.variance_epsilon) * self.weight.float()).to(x.dtype)


class MLP(nn.Module):
    def __init__(self, gate, up, down):
        super().__init__()
        self.gate, self.up, self.down = nn.Parameter(gate), nn.Parameter(up), nn.Parameter(down)

    def forward(self, x):
        return (nn.functional.silu(x @ self.gate.T) * (x @ self.up.T)) @ self.down.T


def linear(weight, bias=None):
    m = nn.Linear(weight.shape[1], weight.shape[0], bias=bias is not None)
    m.weight = nn.Parameter(weight)
    if bias is not None:
        m.bias = nn.Parameter(bias)
    return m


def skeleton(config: dict, w: dict) -> nn.Module:
    m = nn.Module()
    m.config = types.SimpleNamespace(
        model_type="qwen2", hidden_size=config["hidden_size"], num_attention_heads=config["num_attention_heads"],
        num_key_value_heads=config["num_key_value_heads"], head_dim=config["head_dim"],
        num_hidden_layers=config["num_hidden_layers"], rope_theta=config["rope_theta"], eos_token_id=None)
    m.model = nn.Module()
    m.model.embed_tokens = nn.Embedding.from_pretrained(w["model.embed_tokens.weight"])
    layers = []
    eps = config["rms_norm_eps"]
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}."
        layer = nn.Module()
        layer.input_layernorm = RMS(w[p + "input_layernorm.weight"], eps)
        layer.post_attention_layernorm = RMS(w[p + "post_attention_layernorm.weight"], eps)
        a = nn.Module()
        a.q_proj = linear(w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"])
        a.k_proj = linear(w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"])
        a.v_proj = linear(w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
        a.o_proj = linear(w[p + "self_attn.o_proj.weight"])
        layer.self_attn = a
        layer.mlp = MLP(w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        layers.append(layer)
    m.model.layers = nn.ModuleList(layers)
    m.model.norm = RMS(w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else w["lm_head.weight"]
    m.lm_head = linear(head)
    return m.eval()


def fill_fake_qwen(model: nn.Module, w: dict) -> None:
    """Put ``w`` into the reference's FakeQwen and zero the biases that Qwen2.5 does not have."""
    def put(param, value):
        with torch.no_grad():
            param.copy_(value)
    put(model.model.embed_tokens.weight, w["model.embed_tokens.weight"])
    put(model.model.norm.weight, w["model.norm.weight"])
    put(model.lm_head.weight, w["lm_head.weight"])
    for l, layer in enumerate(model.model.layers):
        p = f"model.layers.{l}."
        put(layer.input_layernorm.weight, w[p + "input_layernorm.weight"])
        put(layer.post_attention_layernorm.weight, w[p + "post_attention_layernorm.weight"])
        for proj in ("q_proj", "k_proj", "v_proj"):
            put(getattr(layer.self_attn, proj).weight, w[p + f"self_attn.{proj}.weight"])
            put(getattr(layer.self_attn, proj).bias, w[p + f"self_attn.{proj}.bias"])
        put(layer.self_attn.o_proj.weight, w[p + "self_attn.o_proj.weight"])
        layer.self_attn.o_proj.bias.data.zero_()
        for proj in ("gate_proj", "up_proj", "down_proj"):
            put(getattr(layer.mlp, proj).weight, w[p + f"mlp.{proj}.weight"])
            getattr(layer.mlp, proj).bias.data.zero_()


def main(reference_root: str) -> None:
    sys.path.insert(0, os.path.join(reference_root, "src"))
    sys.path.insert(0, os.path.join(reference_root, "tests", "unit"))
    from flexengine.engine.kv_cache.allocator import CacheLayout, PagedKVCache
    from flexengine.engine.scheduler.policies import Chunk
    from flexengine.inference.models.qwen2 import Qwen2Adapter
    import test_synthetic_qwen as reference_test
    out = {}

    # ---- the reference's own norm and feed-forward modules on fixed inputs
    x, rms_w, gate, up, down = part_inputs()
    with torch.no_grad():
        rms = reference_test.FakeRMS(24)
        rms.weight.copy_(rms_w)
        out["parts/rms/out"] = rms(x).numpy()
        mlp = reference_test.FakeMLP(24)
        mlp.gate_proj.weight.copy_(gate), mlp.up_proj.weight.copy_(up), mlp.down_proj.weight.copy_(down)
        mlp.gate_proj.bias.zero_(), mlp.up_proj.bias.zero_(), mlp.down_proj.bias.zero_()
        out["parts/mlp/out"] = mlp(x).numpy()

    # ---- the reference's whole synthetic model, through its adapter
    w = fixed_weights(FAKE_CONFIG)
    out["fake/checksum"] = np.frombuffer(weights_checksum(w).encode(), dtype=np.uint8)
    fake = reference_test.FakeQwen().eval()
    fill_fake_qwen(fake, w)
    a, b = FAKE_PROMPTS
    with torch.no_grad():
        for backend in ("blockwise", "materialized"):
            adapter = Qwen2Adapter(fake, "cpu", attention_backend=backend)
            cache = PagedKVCache(CacheLayout(2, 40, 4, 2, 8))
            cache.reserve("a", len(a)), cache.reserve("b", len(b))
            got = adapter.forward([Chunk("a", a, 0), Chunk("b", b, 0)], cache)
            out[f"fake/{backend}/whole/a"], out[f"fake/{backend}/whole/b"] = got[0].numpy(), got[1].numpy()
            cache.free_request("a")
            cache.reserve("a", len(a))
            adapter.forward([Chunk("a", a[:3], 0)], cache)
            adapter.forward([Chunk("a", a[3:8], 3)], cache)
            out[f"fake/{backend}/portions/a"] = adapter.forward([Chunk("a", a[8:], 8)], cache)[0].numpy()
        out["fake/independent/a"] = reference_test.independent_reference(fake, a).numpy()

    # ---- the adapter over the tests' tiny configurations
    for name, config in helpers.CONFIGS.items():
        w = fixed_weights(config)
        out[f"{name}/checksum"] = np.frombuffer(weights_checksum(w).encode(), dtype=np.uint8)
        model = skeleton(config, w)
        page = helpers.PAGE_SIZE[name]
        prompts = prompts_for(name)
        for backend in ("blockwise", "materialized"):
            adapter = Qwen2Adapter(model, "cpu", attention_backend=backend)
            cache = PagedKVCache(CacheLayout(config["num_hidden_layers"], 64, page, config["num_key_value_heads"],
                                             config["head_dim"]))
            with torch.no_grad():
                for i, ids in enumerate(prompts):
                    cache.reserve(f"w{i}", len(ids))
                    out[f"{name}/{backend}/whole/{i}"] = adapter.forward([Chunk(f"w{i}", ids, 0)], cache)[0].numpy()
                    cache.free_request(f"w{i}")
                # mixed batch: the longest prompt's tail as a portion beside a decoded token of another request
                long_ids, short_ids = prompts[-1], prompts[0]
                cut = len(long_ids) // 2
                cache.reserve("l", len(long_ids)), cache.reserve("s", len(short_ids))
                if len(short_ids) > 1:
                    adapter.forward([Chunk("s", short_ids[:-1], 0)], cache)
                adapter.forward([Chunk("l", long_ids[:cut], 0)], cache)
                got = adapter.forward([Chunk("l", long_ids[cut:], cut), Chunk("s", short_ids[-1:], len(short_ids) - 1)], cache)
                out[f"{name}/{backend}/mixed/long"] = got[0].numpy()
                out[f"{name}/{backend}/mixed/short"] = got[1].numpy()
    assert "transformers" not in sys.modules
    np.savez_compressed(os.path.join(HERE, "reference_logits.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_logits.npz"), len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference/checkout")
    main(sys.argv[1])
