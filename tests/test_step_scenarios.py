"""The step function against the plain implementation, under every way of cutting the work.

The same scenarios run twice: on the CPU with the PyTorch kernel references handed to the
engine (host logic: metadata, cache, block tables), and, marked ``gpu``, with the CUDA
kernels in float32 and in bfloat16.
"""
import random

import pytest
import torch

import helpers
import kernel_refs

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 40, 77, 130], "C": [3, 50, 64], "D": [300, 70, 150]}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: helpers.make_model_dir(tmp_path_factory, name, seed=11 + i)
            for i, name in enumerate(helpers.CONFIGS)}


def _requests(name: str, seed: int = 3) -> dict:
    rng = random.Random(seed)
    vocab = helpers.CONFIGS[name]["vocab_size"]
    return {f"r{i}": helpers.random_prompt(rng, n, vocab) for i, n in enumerate(LENGTHS[name])}


def _scenario(kind: str, requests: dict, rng: random.Random) -> list:
    if kind == "whole":
        return helpers.steps_whole(requests)
    if kind == "last_decoded":
        return helpers.steps_last_decoded(requests, tail=32)
    if kind == "portions":
        return helpers.steps_portions(requests, rng)
    if kind == "mixed":
        # twice the requests, so that later ones run in pages that earlier ones gave back
        doubled = dict(requests)
        doubled.update({rid + "x": ids[::-1] for rid, ids in requests.items()})
        return helpers.steps_mixed(doubled, rng, live=4)
    raise ValueError(kind)


def _run(model_dir, name, kind, dtype, device, ops):
    rng = random.Random(5)
    requests = _requests(name)
    steps = _scenario(kind, requests, rng)
    page = helpers.PAGE_SIZE[name]
    # just enough pages for the live requests: pages are used again
    pages = helpers.peak_pages(steps, page) + (0 if kind == "mixed" else 1)
    runner = helpers.make_runner(model_dir, dtype, device, pages, page, max_requests=4, ops=ops)
    results = helpers.run_steps(runner, steps)
    assert runner.cache.used_pages == 0
    all_requests = {}
    for entries, _ in steps:
        for rid, toks, _w in entries:
            all_requests.setdefault(rid, []).extend(toks)
    helpers.compare_with_plain(model_dir, results, all_requests, dtype, f"{name}/{kind}/{dtype}", config=name)
    if device != "cpu":
        from flexengine_b200 import ops as cuda_ops
        cuda_ops.check_status(device)


@pytest.mark.parametrize("kind", ["whole", "last_decoded", "portions", "mixed"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_step_on_cpu_with_reference_kernels(model_dirs, name, kind):
    _run(model_dirs[name], name, kind, "float32", "cpu", kernel_refs)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["whole", "last_decoded", "portions", "mixed"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_step_on_gpu(model_dirs, name, kind, dtype):
    _run(model_dirs[name], name, kind, dtype, "cuda:0", None)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_portions_late_in_a_long_context(model_dirs, dtype):
    """A prompt of 1,700 tokens in portions of 2 to 90 while a second request decodes beside it: from 1,024 keys on
    the bfloat16 prefill attention shares the keys of a portion out over several blocks and merges them, with the
    decoded token as a one-row portion in the same launch."""
    rng = random.Random(9)
    vocab = helpers.CONFIGS["D"]["vocab_size"]
    long_ids, side_ids = helpers.random_prompt(rng, 1700, vocab), helpers.random_prompt(rng, 1150, vocab)
    steps = [([("side", side_ids[:1090], [1089])], [])]
    at, side_at = 0, 1090
    while at < len(long_ids):
        n = min(rng.choice((2, 17, 48, 64, 90)), len(long_ids) - at)
        entries = [("long", long_ids[at:at + n], list(range(n)))]
        if side_at < len(side_ids):
            entries.append(("side", side_ids[side_at:side_at + 1], [0]))
            side_at += 1
        steps.append((entries, []))
        at += n
    steps[-1] = (steps[-1][0], ["long", "side"])
    page = helpers.PAGE_SIZE["D"]
    runner = helpers.make_runner(model_dirs["D"], dtype, "cuda:0", helpers.peak_pages(steps, page) + 1, page)
    results = helpers.run_steps(runner, steps)
    assert runner.cache.used_pages == 0
    for rid, ids, first in (("long", long_ids, 0), ("side", side_ids[:side_at], 1089)):
        want = helpers.plain_logits(model_dirs["D"], ids, "cuda:0")
        got = torch.stack([results[(rid, p)] for p in range(first, len(ids))])
        helpers.assert_logits_close(got, want[first:], dtype, f"long context, {rid}, {dtype}", "D")
    from flexengine_b200 import ops as cuda_ops
    cuda_ops.check_status("cuda:0")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_stored_in_32_bit(tmp_path_factory, dtype):
    """A checkpoint stored in float32: in bfloat16 mode its matrices stay 32-bit (their products run
    through the float32 GEMM), activations and cache are bfloat16; both modes match the plain implementation."""
    model_dir = helpers.make_model_dir(tmp_path_factory, "C", seed=77, stored="float32")
    _run(model_dir, "C", "portions", dtype, "cuda:0", None)
    _run(model_dir, "C", "mixed", dtype, "cuda:0", None)


def test_head_sizes_outside_the_kernels_range_are_refused_when_the_model_is_built():
    from flexengine_b200.config import resolve
    from flexengine_b200.parts import DecoderModel
    bad = dict(helpers.TINY_A, head_dim=24)
    _cfg, plan = resolve(bad)
    with pytest.raises(ValueError, match="steps of 16"):
        DecoderModel(plan)
