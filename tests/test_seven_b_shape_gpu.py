"""The layer sizes of the Qwen2.5-7B shape (hidden 3584, 28 heads over 4, head size 128, feed-forward
18944, vocabulary 152064) with two layers and random weights drawn on the device: the kernels at
the sizes they are tuned for (the weight-streaming GEMM's wide and deep variants, the tcgen05
product from 1,024 rows, split-KV decode under CUDA graphs) against the plain implementation."""
import random

import pytest
import torch

import helpers
import plain_model
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import resolve
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.weights import checkpoint_tensors, random_model, random_tensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHAPE = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=3584,
             num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
             rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)


@pytest.fixture(scope="module")
def plain_weights():
    _cfg, plan = resolve(SHAPE)
    return {name: random_tensor(plan, name, shape, 5, torch.bfloat16, DEV) for name, shape in checkpoint_tensors(plan)}


_models = {}


def runner_for(dtype, pages, max_requests=3):
    if dtype not in _models:
        _models[dtype] = random_model(SHAPE, seed=5, dtype=dtype, device=DEV)
    _cfg, plan, model = _models[dtype]
    torch_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    cache = CacheManager(plan.cache_groups, pages, 16, max_requests, torch_dtype, DEV)
    return ModelRunner(model, cache)


def test_bfloat16_prefill_on_tcgen05_then_graph_decode(plain_weights):
    rng = random.Random(1)
    long_ids = helpers.random_prompt(rng, 1100, SHAPE["vocab_size"])
    short = [helpers.random_prompt(rng, n, SHAPE["vocab_size"]) for n in (40, 75)]
    runner = runner_for("bfloat16", 90)
    runner.enable_decode_graphs(3, 1200)
    rows = {0: [], 1: [], 2: []}
    rows[0].append(runner.step([StepEntry("r0", long_ids[:1030], [0, 500, 1023, 1029])]))       # 1,030 rows: tcgen05 product
    for j, ids in enumerate(short, start=1):
        rows[j].append(runner.step([StepEntry(f"r{j}", ids[:-30], [len(ids) - 31])]))
    # a mixed step: a portion of the long request beside decoded tokens of the others
    out = runner.step([StepEntry("r0", long_ids[1030:1070], [39]), StepEntry("r1", short[0][-30:-29], [0]),
                       StepEntry("r2", short[1][-30:-29], [0])])
    rows[0].append(out[0:1]); rows[1].append(out[1:2]); rows[2].append(out[2:3])
    for step in range(29):                                      # decode steps of all three, from CUDA graphs
        out = runner.step([StepEntry("r0", [long_ids[1070 + step]], [0]), StepEntry("r1", [short[0][-29 + step]], [0]),
                           StepEntry("r2", [short[1][-29 + step]], [0])])
        for j in range(3):
            rows[j].append(out[j:j + 1].clone())
    assert runner.graph_replays == 29
    from flexengine_b200 import ops
    ops.check_status(DEV)
    want = plain_model.forward_logits(SHAPE, plain_weights, long_ids[:1099]).cpu()
    picks = [0, 500, 1023, 1029, 1069] + list(range(1070, 1099))
    helpers.assert_logits_close(torch.cat(rows[0]), want[picks], "bfloat16", "7B-shape long request", "7B widths")
    for j, ids in enumerate(short, start=1):
        want = plain_model.forward_logits(SHAPE, plain_weights, ids).cpu()
        helpers.assert_logits_close(torch.cat(rows[j]), want[len(ids) - 31:], "bfloat16", f"7B-shape short request {j}", "7B widths")


def test_a_graph_keeps_its_scratch_when_a_later_bucket_needs_more(plain_weights):
    """The one-request graph is captured first; the eight-request graph then needs a larger scratch buffer for
    the attention splits.  The first graph must still own valid memory when it is replayed afterwards, also
    after the allocator has given every unused block back to the driver."""
    from flexengine_b200 import ops
    ops._scratch.clear()               # as in a fresh process: earlier tests may have left a large buffer behind
    rng = random.Random(3)
    ids = [helpers.random_prompt(rng, 70, SHAPE["vocab_size"]) for _ in range(8)]
    runner = runner_for("bfloat16", 8 * 5 + 2, max_requests=8)
    runner.enable_decode_graphs(8, 8192)        # a limit beyond what one cluster of splits covers: the form with scratch memory
    for j in range(8):
        runner.step([StepEntry(f"r{j}", ids[j][:60], [])])
    first = runner.step([StepEntry("r0", ids[0][60:61], [0])]).clone()                       # captures the graph of one request
    small = ops.scratch(torch.device(DEV), 1)
    all_eight = runner.step([StepEntry(f"r{j}", ids[j][60 + (j == 0):61 + (j == 0)], [0]) for j in range(8)]).clone()
    assert ops.scratch(torch.device(DEV), 1).data_ptr() != small.data_ptr(), "this shape was chosen so that the scratch grows"
    del small
    torch.cuda.empty_cache()
    junk = [torch.full((1 << 20,), 7, dtype=torch.uint8, device=DEV) for _ in range(8)]       # takes freed blocks, if any
    again = runner.step([StepEntry("r0", ids[0][62:63], [0])]).clone()                       # replays the first graph
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert runner.graph_replays == 3 and sorted(runner._graphs) == [1, 8]
    want = plain_model.forward_logits(SHAPE, plain_weights, ids[0][:63]).cpu()
    got = torch.cat([first, all_eight[0:1], again])
    helpers.assert_logits_close(got, want[[60, 61, 62]], "bfloat16", "graph replayed after the scratch grew", "7B widths")
    del junk


def test_float32_path_at_the_seven_b_widths(plain_weights):
    rng = random.Random(2)
    ids = helpers.random_prompt(rng, 150, SHAPE["vocab_size"])
    runner = runner_for("float32", 12, max_requests=1)
    got = [runner.step([StepEntry("a", ids[:100], [0, 50, 99])])]
    got.append(runner.step([StepEntry("a", ids[100:147], [46])]))
    for p in range(147, 150):
        got.append(runner.step([StepEntry("a", ids[p:p + 1], [0])]))
    want = plain_model.forward_logits(SHAPE, plain_weights, ids).cpu()
    helpers.assert_logits_close(torch.cat(got), want[[0, 50, 99, 146, 147, 148, 149]], "float32", "7B-shape float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["whole", "last_decoded", "portions", "mixed"])
def test_every_cut_at_the_seven_b_widths(plain_weights, kind, dtype):
    """The four ways of cutting the work, at the widths where the tuned kernel variants live (two-tile blocks and
    sixteen-warp split-K of the weight-streaming GEMM, the tcgen05 product from 1,024 rows, tcgen05 attention with
    split keys, split-KV decode), with a pool so small that pages are used again; every row of every request
    against the plain implementation, in both precisions."""
    import test_step_scenarios as scenarios
    rng = random.Random(17)
    vocab = SHAPE["vocab_size"]
    requests = {f"s{i}": helpers.random_prompt(rng, n, vocab) for i, n in enumerate((1100, 70, 300, 33))}
    steps = scenarios._scenario(kind, requests, random.Random(5))
    pages = helpers.peak_pages(steps, 16) + (0 if kind == "mixed" else 1)
    runner = runner_for(dtype, pages, max_requests=4)
    results = helpers.run_steps(runner, steps)
    assert runner.cache.used_pages == 0
    fed = {}
    for entries, _ in steps:
        for rid, toks, _w in entries:
            fed.setdefault(rid, []).extend(toks)
    worst = 0.0
    for rid, ids in fed.items():
        want = plain_model.forward_logits(SHAPE, plain_weights, ids).cpu()
        got = torch.stack([results[(rid, p)] for p in range(len(ids))])
        worst = max(worst, float((got - want).abs().max() / want.std(dim=-1).mean()))
        helpers.assert_logits_close(got, want, dtype, f"7B widths, {kind}, {dtype}, {rid}", "7B widths")
    print(f"7B widths {kind} {dtype}: worst |diff| / spread = {worst:.4f}")
    from flexengine_b200 import ops
    ops.check_status(DEV)


def test_a_layer_as_one_call_gives_what_kernel_by_kernel_gives(plain_weights):
    """A step of more than a handful of tokens runs each layer as one call into the kernel library (the same kernels
    and library products in the same order, launched from C); with that switched off the parts launch them one by
    one.  The two agree to the last bit or to a rounding (the library may choose another algorithm for a product)."""
    from flexengine_b200 import ops
    rng = random.Random(23)
    ids = [helpers.random_prompt(rng, n, SHAPE["vocab_size"]) for n in (1100, 40, 150)]
    results = {}
    for native in (True, False):
        ops._native_off = not native
        try:
            runner = runner_for("bfloat16", 90, max_requests=12)
            before = ops.launches
            rows = [runner.step([StepEntry("a", ids[0][:1030], [0, 1029])])]                       # 1,030 rows: the tcgen05 product
            rows.append(runner.step([StepEntry("b", ids[1][:30], [29]), StepEntry("c", ids[2][:100], [99])]))
            rows.append(runner.step([StepEntry("a", ids[0][1030:1070], [39]), StepEntry("b", ids[1][30:31], [0]),
                                     StepEntry("c", ids[2][100:150], [0, 49])]))                   # a mixed step, keys split
            rows.append(runner.step([StepEntry(r, [ids[i][-1]], [0]) for i, r in enumerate("abc")] +
                                    [StepEntry(f"d{j}", [5 + j], [0]) for j in range(9)]))         # twelve decoded tokens
            results[native] = (torch.cat(rows).float().cpu(), ops.launches - before)
        finally:
            ops._native_off = False
    ops.check_status(DEV)
    (fast, fast_launches), (slow, slow_launches) = results[True], results[False]
    assert fast_launches == slow_launches, "the same kernels either way"
    spread = float(slow.std(dim=-1).mean())
    assert float((fast - slow).abs().max()) <= 0.02 * spread
    want = plain_model.forward_logits(SHAPE, plain_weights, ids[0][:1070]).cpu()
    helpers.assert_logits_close(fast[[0, 1, 4]], want[[0, 1029, 1069]], "bfloat16", "a layer as one call", "7B widths")
