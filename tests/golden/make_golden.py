"""Makes ``reference_logits.npz``: last-token logits computed by the reference's OWN model code.

Run once, on the CPU, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It writes tiny random Qwen2.5 models with ``write_random_model`` (seeded), wraps their tensors
in a module tree of the shape the reference's ``Qwen2Adapter`` walks
(src/flexengine/inference/models/qwen2.py:94-135), runs the adapter with the reference's
``PagedKVCache`` and both of its CPU attention backends, whole and as a mixed batch
(a prefill portion beside a decoded token), and stores the logits together with a checksum
of the weights, so that the test can tell whether it regenerated the same model.  The
RMSNorm and SwiGLU modules of the wrapper are not the reference's code (it calls Hugging
Face modules there); they follow src/flexengine/inference/kernels/rmsnorm.py:24-32 and
tests/unit/test_synthetic_qwen.py:30-36.  ``transformers`` is not imported.
"""
import hashlib
import os
import sys
import tempfile
import types

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import helpers  # noqa: E402
from flexengine_b200.weights import write_random_model  # noqa: E402

SEED = 2024
PROMPTS = {"A": [5, 17, 33], "B": [1, 40, 77], "C": [3, 50]}


def weights_checksum(tensors: dict) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].float().contiguous().numpy().tobytes())
    return h.hexdigest()


def prompts_for(name: str) -> list:
    g = torch.Generator().manual_seed(99)
    vocab = helpers.CONFIGS[name]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in PROMPTS[name]]


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


def main(reference_root: str) -> None:
    sys.path.insert(0, os.path.join(reference_root, "src"))
    from flexengine.engine.kv_cache.allocator import CacheLayout, PagedKVCache
    from flexengine.engine.scheduler.policies import Chunk
    from flexengine.inference.models.qwen2 import Qwen2Adapter
    import plain_model
    out = {}
    for name, config in helpers.CONFIGS.items():
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(config, folder, seed=SEED, dtype="bfloat16")
            _, w = plain_model.read_model_folder(folder)
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
                cache.reserve("l", len(long_ids)); cache.reserve("s", len(short_ids))
                adapter.forward([Chunk("s", short_ids[:-1], 0)], cache) if len(short_ids) > 1 else None
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
