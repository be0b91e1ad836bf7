"""The plain implementation against logits that the reference's own model code produced
(tests/golden/make_golden.py), and against itself."""
import os
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(GOLDEN, "reference_logits.npz"))


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_plain_model_matches_the_reference_adapter(name, golden):
    import make_golden
    config = helpers.CONFIGS[name]
    w = make_golden.fixed_weights(config)          # integer arithmetic: the same on every machine, so no skip
    assert make_golden.weights_checksum(w) == bytes(golden[f"{name}/checksum"]).decode(), \
        "the fixed weights differ from the ones the golden file was made with"
    prompts = make_golden.prompts_for(name)
    for backend in ("blockwise", "materialized"):
        for i, ids in enumerate(prompts):
            want = torch.from_numpy(golden[f"{name}/{backend}/whole/{i}"])
            got = plain_model.forward_logits(config, w, ids)[-1]
            torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)       # the reference's own bar
        long_ids, short_ids = prompts[-1], prompts[0]
        torch.testing.assert_close(plain_model.forward_logits(config, w, long_ids)[-1],
                                   torch.from_numpy(golden[f"{name}/{backend}/mixed/long"]), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(plain_model.forward_logits(config, w, short_ids)[-1],
                                   torch.from_numpy(golden[f"{name}/{backend}/mixed/short"]), atol=1e-5, rtol=1e-5)


def test_norm_and_feed_forward_match_the_reference_modules(golden):
    """``rms_norm`` and ``swiglu_mlp`` against outputs of the reference's own FakeRMS and FakeMLP modules
    (tests/unit/test_synthetic_qwen.py:19-36 of the reference; eps 1e-6 is fixed in FakeRMS)."""
    import make_golden
    x, rms_w, gate, up, down = make_golden.part_inputs()
    torch.testing.assert_close(plain_model.rms_norm(x, rms_w, 1e-6), torch.from_numpy(golden["parts/rms/out"]),
                               atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(plain_model.swiglu_mlp(x, gate, up, down), torch.from_numpy(golden["parts/mlp/out"]),
                               atol=1e-6, rtol=1e-6)


def test_plain_model_matches_the_reference_synthetic_model(golden):
    """The reference's whole FakeQwen (its own norm, feed-forward and layer modules) through its adapter,
    whole, in portions and beside another request, and its own dense check (independent_reference)."""
    import make_golden
    config = make_golden.FAKE_CONFIG
    w = make_golden.fixed_weights(config)
    assert make_golden.weights_checksum(w) == bytes(golden["fake/checksum"]).decode()
    a, b = make_golden.FAKE_PROMPTS
    got_a = plain_model.forward_logits(config, w, a)[-1]
    got_b = plain_model.forward_logits(config, w, b)[-1]
    for backend in ("blockwise", "materialized"):
        torch.testing.assert_close(got_a, torch.from_numpy(golden[f"fake/{backend}/whole/a"]), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(got_b, torch.from_numpy(golden[f"fake/{backend}/whole/b"]), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(got_a, torch.from_numpy(golden[f"fake/{backend}/portions/a"]), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(got_a, torch.from_numpy(golden["fake/independent/a"]), atol=1e-5, rtol=1e-5)


def test_parts_of_the_plain_model():
    torch.manual_seed(0)
    x = torch.randn(5, 24)
    w = torch.rand(24) + 0.5
    y = plain_model.rms_norm(x, w, 1e-6)
    torch.testing.assert_close((y / w).pow(2).mean(-1), torch.ones(5), atol=1e-4, rtol=1e-4)
    # rotation keeps norms and depends only on relative position in the scores
    inv = plain_model.rope_inverse_frequencies(16, 10000.0, "cpu")
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    def score(pq, pk):
        return float((plain_model.apply_rope(q, torch.tensor([pq]), inv) * plain_model.apply_rope(k, torch.tensor([pk]), inv)).sum())
    assert abs(score(7, 3) - score(104, 100)) < 1e-4
    torch.testing.assert_close(plain_model.apply_rope(q, torch.tensor([9]), inv).norm(), q.norm())
    # causal: changing a later token does not change earlier outputs; window hides old keys
    qq, kk, vv = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    base = plain_model.causal_gqa_attention(qq, kk, vv)
    kk2, vv2 = kk.clone(), vv.clone()
    kk2[5] += 1; vv2[5] += 1
    torch.testing.assert_close(plain_model.causal_gqa_attention(qq, kk2, vv2)[:5], base[:5])
    win = plain_model.causal_gqa_attention(qq, kk, vv, window=1)
    torch.testing.assert_close(win, vv.repeat_interleave(2, dim=1))
    # query head h reads key/value head h // ratio
    only = plain_model.causal_gqa_attention(qq[:1], kk[:1], vv[:1])
    torch.testing.assert_close(only[0, 0], vv[0, 0]); torch.testing.assert_close(only[0, 3], vv[0, 1])


def test_sampling_distribution_top_k():
    logits = torch.tensor([0.0, 3.0, 1.0, 2.0])
    p = plain_model.sampling_distribution(logits, 1.0, 2)
    assert p[0] == 0 and p[2] == 0 and abs(float(p.sum()) - 1) < 1e-6 and p[1] > p[3]
    torch.testing.assert_close(plain_model.sampling_distribution(logits, 2.0, 0), torch.softmax(logits / 2, -1))
