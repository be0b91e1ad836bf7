"""Shared by the tests: tiny configurations, model folders in temporary places, scenarios of
steps, and the comparison bars."""
from __future__ import annotations

import random

import torch

import kernel_refs
import plain_model
from flexengine_b200.cache import CacheManager
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.weights import load_model, write_random_model

# Two tiny configurations that differ in every size and option, and a third whose heads do not
# span the hidden size and whose sizes are no powers of two.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=160, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=256, tie_word_embeddings=True,
              use_sliding_window=False, hidden_act="silu", eos_token_id=255)
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3, hidden_size=192,
              num_attention_heads=6, num_key_value_heads=1, head_dim=32, intermediate_size=384, vocab_size=512,
              rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=512, tie_word_embeddings=False,
              use_sliding_window=False, hidden_act="silu", eos_token_id=[510, 511])
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=80,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=112, vocab_size=301,
              rope_theta=50000.0, rms_norm_eps=3e-6, max_position_embeddings=1024, tie_word_embeddings=False,
              use_sliding_window=False, hidden_act="silu")
# head size 64: in bfloat16 its portions take the tcgen05 attention kernel (the others' head sizes take the mma.sync one)
TINY_D = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=96,
              num_attention_heads=8, num_key_value_heads=2, head_dim=64, intermediate_size=176, vocab_size=333,
              rope_theta=200000.0, rms_norm_eps=2e-6, max_position_embeddings=2048, tie_word_embeddings=True,
              use_sliding_window=False, hidden_act="silu")
PAGE_SIZE = {"A": 16, "B": 32, "C": 16, "D": 8}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def make_model_dir(tmp_path_factory, name: str, seed: int = 7, stored: str = "bfloat16") -> str:
    d = tmp_path_factory.mktemp(f"model_{name}")
    write_random_model(CONFIGS[name], str(d), seed=seed, dtype=stored)
    return str(d)


def make_runner(model_dir: str, dtype: str, device: str, num_pages: int, page_size: int, max_requests: int = 4,
                ops=None):
    _cfg, plan, model = load_model(model_dir, dtype, device)
    torch_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    cache = CacheManager(plan.cache_groups, num_pages, page_size, max_requests, torch_dtype, device)
    return ModelRunner(model, cache, ops=ops)


def plain_logits(model_dir: str, ids, device="cpu") -> torch.Tensor:
    config, weights = plain_model.read_model_folder(model_dir, device)
    return plain_model.forward_logits(config, weights, ids).cpu()


# ---- comparison bars ----------------------------------------------------------------------------
# float32: kernels and the plain implementation differ only in the order of float32 sums.
# bfloat16: activations are rounded to 8 bits of mantissa between kernels, so the error scales with the
# spread of the logits.  BF16_SEEN is the worst |difference| that the engine showed over all four scenarios of
# cutting the work, divided by the standard deviation of the plain logits (B200, per tiny configuration; A
# 0.0024, B 0.0065, C 0.0031, D 0.0035 in absolute terms, with the library's products adding in float); the bar
# is three times that, which stays well below the models' typical gap between the best and the second-best logit
# (0.03 to 0.5).
# At the Qwen2.5-7B widths (two layers, 1,100-token prompts, a vocabulary of 152,064) the worst of 230 million
# logits was 0.076 of their spread.
BF16_SEEN = {"A": 0.014, "B": 0.023, "C": 0.018, "D": 0.0175, "7B widths": 0.077}
BF16_SEEN_ELSEWHERE = 0.03
BF16_HEADROOM = 3.0


def bf16_bar(want: torch.Tensor, config: str | None = None) -> float:
    spread = float(want.float().std(dim=-1).mean()) if want.dim() == 2 else float(want.float().std())
    return BF16_HEADROOM * BF16_SEEN.get(config, BF16_SEEN_ELSEWHERE) * spread


def assert_logits_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", config: str | None = None) -> None:
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    bar = 2e-5 * max(1.0, float(want.abs().max())) if dtype == "float32" else bf16_bar(want, config)
    err = (got - want).abs()
    worst = int(err.max(dim=-1).values.argmax()) if err.dim() == 2 else 0
    assert float(err.max()) <= bar, f"{what}: max |diff| {float(err.max()):.3e} > {bar:.3e} (first worst row {worst})"


def assert_near_maximum(row: torch.Tensor, token: int, config: str | None, what: str = "") -> None:
    """A token chosen in bfloat16 is the float32 logits' maximum, or so close to it that bfloat16's error (the
    bar above, on both logits) can have swapped the two."""
    short = float(row.max() - row[token])
    assert short <= bf16_bar(row, config), f"{what}: token {token} is {short:.3e} below the maximum (bar {bf16_bar(row, config):.3e})"


# ---- scenarios: lists of steps; a step is (entries, ended) with entries [(rid, tokens, want)] ----------
def random_prompt(rng: random.Random, length: int, vocab: int) -> list:
    return [rng.randrange(vocab) for _ in range(length)]


def steps_whole(requests: dict) -> list:
    return [([(rid, ids, list(range(len(ids))))], [rid]) for rid, ids in requests.items()]


def steps_last_decoded(requests: dict, tail: int = 32) -> list:
    steps = []
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append(([(rid, ids[:head], list(range(head)))], []))
        for p in range(head, len(ids)):
            steps.append(([(rid, ids[p:p + 1], [0])], [rid] if p == len(ids) - 1 else []))
        if head == len(ids):
            steps[-1] = (steps[-1][0], [rid])
    return steps


def steps_portions(requests: dict, rng: random.Random, sizes=(24, 7, 2, 13, 2, 31, 3, 64, 5)) -> list:
    steps = []
    for rid, ids in requests.items():
        p, i = 0, rng.randrange(len(sizes))
        while p < len(ids):
            n = min(sizes[i % len(sizes)], len(ids) - p)
            if len(ids) - p - n == 1:        # never leave a single token: portions go down to two
                n += 1
            steps.append(([(rid, ids[p:p + n], list(range(n)))], [rid] if p + n == len(ids) else []))
            p, i = p + n, i + 1
    return steps


def steps_mixed(requests: dict, rng: random.Random, live: int = 4, decode_tail: int = 6) -> list:
    """Up to ``live`` requests at a time; each is fed in portions of changing size and its last
    ``decode_tail`` tokens one by one, so that steps hold portions of some requests beside single
    tokens of others; a request is sometimes left out of a step.  Requests start as others end."""
    waiting = list(requests.items())
    active = {}          # rid -> [ids, fed]
    steps = []
    while waiting or active:
        while waiting and len(active) < live:
            rid, ids = waiting.pop(0)
            active[rid] = [ids, 0]
        entries, ended = [], []
        for rid in list(active):
            ids, fed = active[rid]
            if len(active) > 1 and rng.random() < 0.2:
                continue                      # left out of this step
            left = len(ids) - fed
            if left <= decode_tail:
                n = 1
            else:
                n = min(rng.choice((2, 3, 5, 8, 13, 21)), left - decode_tail)
            entries.append((rid, ids[fed:fed + n], list(range(n))))
            active[rid][1] = fed + n
            if fed + n == len(ids):
                ended.append(rid)
                del active[rid]
        if entries:
            steps.append((entries, ended))
    return steps


def run_steps(runner, steps) -> dict:
    """{(rid, position): logits row} for every wanted place."""
    out, fed = {}, {}
    for entries, ended in steps:
        logits = runner.step([StepEntry(rid, toks, want) for rid, toks, want in entries])
        row = 0
        for rid, toks, want in entries:
            base = fed.get(rid, 0)
            for w in want:
                out[(rid, base + w)] = logits[row].float().cpu()
                row += 1
            fed[rid] = base + len(toks)
        for rid in ended:
            runner.finish(rid)
            fed.pop(rid, None)
        runner.cache.assert_invariants()
    return out


def peak_pages(steps, page_size: int) -> int:
    held, fed, peak = {}, {}, 0
    for entries, ended in steps:
        for rid, toks, _ in entries:
            fed[rid] = fed.get(rid, 0) + len(toks)
            held[rid] = -(-fed[rid] // page_size)
        peak = max(peak, sum(held.values()))
        for rid in ended:
            held.pop(rid, None), fed.pop(rid, None)
    return peak


def compare_with_plain(model_dir, results: dict, requests: dict, dtype: str, what: str, device="cpu", config=None) -> None:
    for rid, ids in requests.items():
        want = plain_logits(model_dir, ids, device)
        rows = [p for (r, p) in results if r == rid]
        assert sorted(rows) == list(range(len(ids))), f"{what}: request {rid} misses rows"
        got = torch.stack([results[(rid, p)] for p in range(len(ids))])
        assert_logits_close(got, want, dtype, f"{what} request {rid}", config)
