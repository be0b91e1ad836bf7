"""Configuration, registry, weight loading errors and the random-weights mode (CPU)."""
import copy
import json
import os

import pytest
import torch

import helpers
import plain_model
from flexengine_b200.config import (ConfigError, EngineConfig, Qwen2Config, known_architectures,
                                    resolve)
from flexengine_b200.weights import (CheckpointError, CheckpointReader, load_model, random_model, write_random_model,
                                     write_safetensors)


def test_typed_config_reads_its_keys():
    cfg = Qwen2Config.from_dict(helpers.TINY_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 192, 6, 1)
    assert cfg.head_dim == 32 and cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5
    assert cfg.eos_token_ids == (510, 511) and cfg.tie_word_embeddings is False
    again = Qwen2Config.from_dict(cfg.to_dict())
    assert again == cfg


def test_config_defaults_follow_the_reference():
    data = {k: v for k, v in helpers.TINY_A.items() if k not in ("head_dim", "rope_theta")}
    cfg = Qwen2Config.from_dict(data)
    assert cfg.head_dim == 64 // 4 and cfg.rope_theta == 10000.0
    data["rope_scaling"] = {"rope_type": "default", "rope_theta": 1000000.0}
    assert Qwen2Config.from_dict(data).rope_theta == 1000000.0


@pytest.mark.parametrize("change,match", [
    ({"model_type": "llama"}, "model_type=qwen2"),
    ({"use_sliding_window": True}, "Sliding-window"),
    ({"rope_scaling": {"rope_type": "linear", "factor": 2.0}}, "RoPE scaling"),
    ({"num_key_value_heads": 3}, "GQA head ratio"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"vocab_size": "many"}, "vocab_size"),
])
def test_config_rejections(change, match):
    data = dict(helpers.TINY_A)
    data.update(change)
    with pytest.raises(ConfigError, match=match):
        Qwen2Config.from_dict(data)


def test_registry():
    assert "Qwen2ForCausalLM" in known_architectures()
    typed, plan = resolve(helpers.TINY_A)
    assert plan.architecture == "Qwen2ForCausalLM" and len(plan.layers) == 2 and len(plan.run) == 2
    assert [g.kind for g in plan.cache_groups] == ["full", "state"]
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*Qwen2ForCausalLM"):
        resolve({**helpers.TINY_A, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve({k: v for k, v in helpers.TINY_A.items() if k != "architectures"})


def test_engine_config_checks_and_environment(monkeypatch):
    other = EngineConfig(kv_num_blocks=512, kv_block_size=16).with_block_size(8)
    assert (other.kv_num_blocks, other.kv_block_size) == (1024, 8)
    assert EngineConfig(kv_num_blocks=130, kv_block_size=16).with_block_size(32).kv_num_blocks == 65
    with pytest.raises(ValueError, match="KV pool cannot contain"):
        EngineConfig(kv_num_blocks=4, kv_block_size=16, max_model_len=2048)
    with pytest.raises(ValueError, match="scheduler_policy"):
        EngineConfig(scheduler_policy="random")
    monkeypatch.setenv("FLEX_MAX_NUM_BATCHED_TOKENS", "256")
    monkeypatch.setenv("FLEX_KV_BLOCK_SIZE", "8")
    monkeypatch.setenv("FLEX_CUDA_GRAPH", "true")
    monkeypatch.setenv("FLEX_DTYPE", "fp32")
    cfg = EngineConfig.from_env(max_num_seqs=16)
    assert (cfg.max_num_batched_tokens, cfg.kv_block_size, cfg.cuda_graph, cfg.dtype, cfg.max_num_seqs) == \
        (256, 8, True, "float32", 16)


def test_cli_flags_map_to_engine_config(monkeypatch):
    from flexengine_b200.cli.generate import build_parser, engine_config_from_args
    for key in ("FLEX_MAX_NUM_BATCHED_TOKENS", "FLEX_KV_BLOCK_SIZE"):
        monkeypatch.delenv(key, raising=False)
    args = build_parser().parse_args(["--model", "m", "--token-budget", "256", "--block-size", "8", "--num-blocks", "1024",
                                      "--max-model-len", "4096", "--max-num-seqs", "16", "--prefill-chunk-size", "96",
                                      "--policy", "adaptive", "--cuda-graph", "--dtype", "float32"])
    cfg = engine_config_from_args(args)
    assert (cfg.max_num_batched_tokens, cfg.kv_block_size, cfg.kv_num_blocks, cfg.max_model_len, cfg.max_num_seqs,
            cfg.prefill_chunk_size, cfg.scheduler_policy, cfg.cuda_graph, cfg.dtype) == \
        (256, 8, 1024, 4096, 16, 96, "adaptive", True, "float32")


# ---- weights ---------------------------------------------------------------------------------------
@pytest.fixture()
def folder(tmp_path):
    write_random_model(helpers.TINY_A, str(tmp_path), seed=3, dtype="bfloat16")
    return str(tmp_path)


def _rewrite(folder, change):
    """Rewrite model.safetensors with ``change(dict name->tensor)`` applied."""
    reader = CheckpointReader(folder)
    tensors = {n: reader.read(n).clone() for n in reader.names()}
    reader.close()
    change(tensors)
    names = list(tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"), [(n, tuple(tensors[n].shape), tensors[n].dtype) for n in names],
                      lambda n: tensors[n])


def test_random_model_folder_is_seeded_and_readable(folder, tmp_path_factory):
    other = str(tmp_path_factory.mktemp("again"))
    write_random_model(helpers.TINY_A, other, seed=3, dtype="bfloat16")
    a, b = CheckpointReader(folder), CheckpointReader(other)
    assert sorted(a.names()) == sorted(b.names())
    for n in a.names():
        assert torch.equal(a.read(n), b.read(n)) and a.read(n).dtype == torch.bfloat16
    # the framework's reader and the safetensors library agree
    _, lib = plain_model.read_model_folder(folder, keep_dtype=True)
    for n in a.names():
        assert torch.equal(a.read(n), lib[n])
    w = a.read("model.layers.0.input_layernorm.weight").float()
    assert abs(float(w.mean()) - 1.0) < 0.02 and float(w.std()) < 0.03
    m = a.read("model.layers.1.mlp.up_proj.weight").float()
    assert abs(float(m.mean())) < 0.002 and abs(float(m.std()) - 0.02) < 0.002
    assert json.load(open(os.path.join(folder, "config.json")))["hidden_size"] == 64
    third = str(tmp_path_factory.mktemp("other_seed"))
    write_random_model(helpers.TINY_A, third, seed=4, dtype="bfloat16")
    assert not torch.equal(CheckpointReader(third).read("model.norm.weight"), a.read("model.norm.weight"))


def test_load_binds_by_name_and_keeps_precisions(folder):
    cfg, plan, model = load_model(folder, "bfloat16", "cpu")
    mixer = model.blocks[0].mixer
    assert mixer.qkv_weight.dtype == torch.bfloat16 and tuple(mixer.qkv_weight.shape) == (4 * 16 + 2 * 2 * 16, 64)
    assert mixer.qkv_bias.dtype == torch.float32                       # vectors are held in float32
    assert mixer.has_qkv_bias and "qkv.bias" in mixer.parameter_shapes()  # the flag survives the binding of the tensor
    assert model.weight_bytes() > 0
    assert model.head.weight.data_ptr() == model.embedding.weight.data_ptr()        # tied
    reader = CheckpointReader(folder)
    q = reader.read("model.layers.0.self_attn.q_proj.weight")
    v = reader.read("model.layers.0.self_attn.v_proj.weight")
    assert torch.equal(mixer.qkv_weight[:64], q) and torch.equal(mixer.qkv_weight[-32:], v)
    gate = reader.read("model.layers.1.mlp.gate_proj.weight")
    assert torch.equal(model.blocks[1].feed_forward.gate_up_weight[:160], gate)
    _, _, model32 = load_model(folder, "float32", "cpu")
    assert model32.blocks[0].mixer.qkv_weight.dtype == torch.float32
    # a matrix stored in 32-bit stays so in bfloat16 mode
    _rewrite(folder, lambda t: t.update({"model.layers.0.mlp.down_proj.weight": t["model.layers.0.mlp.down_proj.weight"].float()}))
    _, _, mixed = load_model(folder, "bfloat16", "cpu")
    assert mixed.blocks[0].feed_forward.down_weight.dtype == torch.float32
    assert mixed.blocks[1].feed_forward.down_weight.dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_misshapen(folder):
    def change(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16, dtype=torch.bfloat16)
        t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
        t["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(31, dtype=torch.bfloat16)
        t["model.embed_tokens.weight"] = t["model.embed_tokens.weight"].to(torch.float64)
    _rewrite(folder, change)
    with pytest.raises(CheckpointError) as info:
        load_model(folder, "bfloat16", "cpu")
    err = info.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["lm_head.weight", "model.layers.0.self_attn.q_norm.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.bias", (31,), (32,))]
    assert err.wrong_dtype[0][0] == "model.embed_tokens.weight"
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (2)", "wrong shape", "is [31], expected [32]",
                  "tie_word_embeddings is true"):
        assert piece in text


def test_random_model_on_device_matches_plan(tmp_path):
    cfg, plan, model = random_model(helpers.TINY_B, seed=9, dtype="bfloat16", device="cpu")
    assert model.head.weight.data_ptr() != model.embedding.weight.data_ptr()
    assert tuple(model.blocks[2].feed_forward.gate_up_weight.shape) == (768, 192)
    cfg2, _, again = random_model(helpers.TINY_B, seed=9, dtype="bfloat16", device="cpu")
    assert torch.equal(model.blocks[1].mixer.out_weight, again.blocks[1].mixer.out_weight)
    # and it is the model the folder variant describes
    write_random_model(helpers.TINY_B, str(tmp_path), seed=9, dtype="bfloat16")
    _, _, loaded = load_model(str(tmp_path), "bfloat16", "cpu")
    assert torch.equal(loaded.blocks[1].mixer.out_weight, model.blocks[1].mixer.out_weight)
