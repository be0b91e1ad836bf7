"""Randomly drawn tiny configurations (head counts and groups, head sizes in steps of 16, widths,
feed-forward sizes and vocabularies that are no round numbers, tied or not) through the mixed
scenario with page reuse, in float32 and bfloat16, against the plain implementation."""
import random

import pytest

import helpers
from flexengine_b200.weights import write_random_model

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    nkv = rng.choice([1, 2, 3, 4])
    group = rng.choice([1, 2, 3, 5, 7, 8])
    d = rng.choice([16, 32, 48, 64, 80, 96, 128])
    hidden = rng.choice([40, 72, 100, 136, 192, 250])
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=rng.choice([1, 2, 3]),
                hidden_size=hidden, num_attention_heads=nkv * group, num_key_value_heads=nkv, head_dim=d,
                intermediate_size=rng.choice([56, 100, 168, 330]), vocab_size=rng.choice([97, 300, 1000, 2049]),
                rope_theta=rng.choice([1e4, 5e5, 1e6]), rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-4]),
                tie_word_embeddings=rng.random() < 0.5, hidden_act="silu")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_random_configuration(seed, dtype, tmp_path):
    config = draw_config(seed)
    write_random_model(config, str(tmp_path), seed=seed, dtype="bfloat16")
    rng = random.Random(100 + seed)
    page = rng.choice([8, 16, 32])
    requests = {f"r{i}": helpers.random_prompt(rng, n, config["vocab_size"]) for i, n in enumerate([3, 45, 70, 129, 33, 64])}
    steps = helpers.steps_mixed(requests, rng, live=4, decode_tail=5)
    runner = helpers.make_runner(str(tmp_path), dtype, "cuda:0", helpers.peak_pages(steps, page), page, max_requests=4)
    results = helpers.run_steps(runner, steps)
    assert runner.cache.used_pages == 0
    helpers.compare_with_plain(str(tmp_path), results, requests, dtype, f"config {config}", device="cuda:0")
    from flexengine_b200 import ops
    ops.check_status("cuda:0")
