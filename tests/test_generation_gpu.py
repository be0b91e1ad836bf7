"""On the GPU: greedy generation through the Python entry point, long decoding, the first tokens
of a sequence, and sampling through the engine, in float32 and bfloat16."""
import random

import pytest
import torch

import helpers
import plain_model
from flexengine_b200.config import EngineConfig
from flexengine_b200.engine import StepEntry
from flexengine_b200.engine.runtime import Engine

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: helpers.make_model_dir(tmp_path_factory, name, seed=41) for name in ("A", "B")}


def engine_for(model_dir, name, dtype, **kw):
    cfg = EngineConfig(model=model_dir, device=DEV, dtype=dtype, max_model_len=kw.pop("max_model_len", 256),
                       max_num_seqs=kw.pop("max_num_seqs", 4), max_num_batched_tokens=kw.pop("budget", 24),
                       kv_block_size=helpers.PAGE_SIZE[name], kv_num_blocks=kw.pop("pages", 32), max_output_tokens=64, **kw)
    return Engine.from_model_dir(model_dir, cfg)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, name):
    config, weights = plain_model.read_model_folder(model_dirs[name], DEV)
    rng = random.Random(1)
    vocab = helpers.CONFIGS[name]["vocab_size"]
    prompts = [helpers.random_prompt(rng, n, vocab) for n in (5, 17, 33, 1, 40)]
    engine = engine_for(model_dirs[name], name, "float32", scheduler_policy="decode_first", prefill_chunk_size=8)
    outputs = engine.generate(prompts, max_tokens=8)
    for prompt, out in zip(prompts, outputs):
        assert out.token_ids == plain_model.greedy_generate(config, weights, prompt, 8)
        assert out.finish_reason in ("length", "stop")
    assert engine.cache.used_pages == 0
    # bfloat16: every chosen token is a maximum of the float32 logits up to bfloat16's observed error
    engine = engine_for(model_dirs[name], name, "bfloat16")
    for prompt, out in zip(prompts, engine.generate(prompts, max_tokens=8)):
        logits = plain_model.forward_logits(config, weights, prompt + out.token_ids[:-1])
        for i, token in enumerate(out.token_ids):
            helpers.assert_near_maximum(logits[len(prompt) - 1 + i].cpu(), token, name, f"{name} token {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, dtype):
    """400 tokens decoded one by one after a short prompt, beside a second request that starts
    later; every logits row against the whole-sequence plain implementation."""
    name = "B"
    rng = random.Random(2)
    ids = helpers.random_prompt(rng, 420, 512)
    other = helpers.random_prompt(rng, 150, 512)
    runner = helpers.make_runner(model_dirs[name], dtype, DEV, 20, 32, max_requests=2)
    rows = {"long": [], "other": []}
    rows["long"].append(runner.step([StepEntry("long", ids[:20], list(range(20)))]))
    for p in range(20, 420):
        entries = [StepEntry("long", ids[p:p + 1], [0])]
        q = p - 200
        if 0 <= q < 150:
            entries.append(StepEntry("other", other[q:q + 1], [0]))
        out = runner.step(entries)
        rows["long"].append(out[:1])
        if len(entries) == 2:
            rows["other"].append(out[1:])
    helpers.assert_logits_close(torch.cat(rows["long"]), helpers.plain_logits(model_dirs[name], ids, DEV), dtype, "long", name)
    helpers.assert_logits_close(torch.cat(rows["other"]), helpers.plain_logits(model_dirs[name], other, DEV), dtype, "other", name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    vocab = helpers.CONFIGS[name]["vocab_size"]
    ids = helpers.random_prompt(random.Random(3), 4, vocab)
    want = helpers.plain_logits(model_dirs[name], ids)
    runner = helpers.make_runner(model_dirs[name], dtype, DEV, 4, helpers.PAGE_SIZE[name], max_requests=4)
    one = torch.cat([runner.step([StepEntry("a", ids[p:p + 1], [0])]) for p in range(4)])
    helpers.assert_logits_close(one, want, dtype, "token by token from position 0", name)
    two = torch.cat([runner.step([StepEntry("b", ids[:1], [0])]), runner.step([StepEntry("b", ids[1:], [0, 1, 2])])])
    helpers.assert_logits_close(two, want, dtype, "1 + 3", name)
    single = runner.step([StepEntry("c", ids[:1], [0])])
    helpers.assert_logits_close(single, want[:1], dtype, "a sequence of one token", name)


def test_temperature_sampling_through_the_engine(model_dirs):
    prompts = [list(range(60, 72)), [7, 200] * 16 + [1], [3, 14, 15, 92, 65], [9]]
    alone = [engine_for(model_dirs["A"], "A", "float32").generate([p], max_tokens=8, temperature=0.8, top_k=20, seed=100 + i)[0].token_ids
             for i, p in enumerate(prompts)]
    together = engine_for(model_dirs["A"], "A", "float32", budget=5, scheduler_policy="decode_first")
    assert [o.token_ids for o in together.generate(prompts, max_tokens=8, temperature=0.8, top_k=20, seed=100)] == alone
    tight = engine_for(model_dirs["A"], "A", "float32", pages=4, budget=48, max_num_seqs=2, max_model_len=64)
    assert [o.token_ids for o in tight.generate(prompts, max_tokens=8, temperature=0.8, top_k=20, seed=100)] == alone
    assert tight.preemption_count >= 1 and tight.cache.used_pages == 0
    # every sampled token lies among the 20 most likely of the plain implementation's distribution
    config, weights = plain_model.read_model_folder(model_dirs["A"], DEV)
    for prompt, tokens in zip(prompts, alone):
        logits = plain_model.forward_logits(config, weights, prompt + tokens[:-1])
        for i, token in enumerate(tokens):
            assert token in torch.topk(logits[len(prompt) - 1 + i], 21).indices.tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_second_tiny_workload_as_it_is_written(model_dirs, dtype):
    """Configuration B with its own workload: four requests with prompts of 1, 40, 77 and 130 tokens, prefill in
    chunks of 24 (the ``adaptive`` policy) mixed with decoding, temperature 0.8, a seed per request, pages of
    32 tokens (the reference's analogue: tests/integration/test_runtime.py:82-118).  In float32 every request draws
    the tokens it draws when it runs alone (a row's arithmetic does not depend on the batch), and each of them lies
    in the support of the plain implementation's distribution at its place.  In bfloat16 a step of a few rows and a
    step of many take different kernels, whose results differ by a rounding: there a draw that falls on the edge
    between two tokens may go either way, so what is checked is the support."""
    rng = random.Random(12)
    prompts = [helpers.random_prompt(rng, n, 512) for n in (1, 40, 77, 130)]
    kw = dict(scheduler_policy="adaptive", prefill_chunk_size=24, budget=32, max_num_seqs=4, pages=12)
    alone = [engine_for(model_dirs["B"], "B", dtype, **kw).generate([p], max_tokens=8, temperature=0.8, seed=300 + i)[0].token_ids
             for i, p in enumerate(prompts)]
    engine = engine_for(model_dirs["B"], "B", dtype, **kw)
    calls = []
    step = engine.runner.step
    engine.runner.step = lambda entries, carried=None: (calls.append([len(e.tokens) for e in entries]), step(entries, carried))[1]
    together = [o.token_ids for o in engine.generate(prompts, max_tokens=8, temperature=0.8, seed=300)]
    if dtype == "float32":
        assert together == alone
    assert max(n for call in calls for n in call) == 24 and any(1 in call and 24 in call for call in calls), \
        "portions of 24 beside decoded tokens"
    assert all(sum(call) <= 32 for call in calls) and engine.cache.used_pages == 0
    assert len({tuple(t) for t in alone}) == 4
    config, weights = plain_model.read_model_folder(model_dirs["B"], DEV)
    for prompt, tokens in zip(prompts + prompts, alone + together):
        assert len(tokens) == 8
        logits = plain_model.forward_logits(config, weights, prompt + tokens[:-1])
        for i, token in enumerate(tokens):
            p = plain_model.sampling_distribution(logits[len(prompt) - 1 + i], 0.8, 0)
            assert float(p[token]) > 1e-5
    from flexengine_b200 import ops
    ops.check_status(DEV)


def test_host_running_ahead_of_the_device(model_dirs):
    """The host enqueues many steps while the device is still busy with earlier work: every step
    must see its own metadata (staging buffers are not reused while a copy is in flight)."""
    name = "A"
    rng = random.Random(5)
    ids = [helpers.random_prompt(rng, 120, 256) for _ in range(3)]
    runner = helpers.make_runner(model_dirs[name], "float32", DEV, 24, 16, max_requests=3)
    big = torch.randn(8192, 8192, device=DEV)
    for _ in range(40):                                  # keeps the device busy for a while
        big = torch.tanh(big @ big * 1e-4)
    outs = [runner.step([StepEntry(f"r{j}", ids[j][:20], list(range(20))) for j in range(3)])]
    for p in range(20, 120):
        outs.append(runner.step([StepEntry(f"r{j}", ids[j][p:p + 1], [0]) for j in range(3)]))
    from flexengine_b200 import ops
    ops.check_status(DEV)
    for j in range(3):
        got = torch.cat([outs[0][20 * j:20 * (j + 1)]] + [o[j:j + 1] for o in outs[1:]])
        helpers.assert_logits_close(got, helpers.plain_logits(model_dirs[name], ids[j], DEV), "float32", f"ahead {j}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_give_the_same_logits(model_dirs, dtype):
    """Decode steps replayed from CUDA graphs (batches padded up to a bucket) against the plain
    implementation, with requests joining and leaving so that several buckets are captured."""
    name = "B"
    rng = random.Random(7)
    ids = [helpers.random_prompt(rng, n, 512) for n in (60, 45, 70, 52, 64)]
    runner = helpers.make_runner(model_dirs[name], dtype, DEV, 20, 32, max_requests=5)
    runner.enable_decode_graphs(5, 128)
    rows = {j: [] for j in range(5)}
    fed = {j: 0 for j in range(5)}
    for j in range(5):                                   # prompts: all but the last 30 tokens
        n = len(ids[j]) - 30
        rows[j].append(runner.step([StepEntry(f"r{j}", ids[j][:n], list(range(n)))]))
        fed[j] = n
    live = [0, 1, 2, 3, 4]
    while live:
        batch = [j for j in live if rng.random() < 0.8] or live[:1]
        out = runner.step([StepEntry(f"r{j}", ids[j][fed[j]:fed[j] + 1], [0]) for j in batch])
        for i, j in enumerate(batch):
            rows[j].append(out[i:i + 1].clone())
            fed[j] += 1
            if fed[j] == len(ids[j]):
                live.remove(j)
                runner.finish(f"r{j}")
    assert runner.graph_replays >= 30 and len(runner._graphs) >= 3
    for j in range(5):
        helpers.assert_logits_close(torch.cat(rows[j]), helpers.plain_logits(model_dirs[name], ids[j], DEV), dtype, f"graph {j}", name)
    from flexengine_b200 import ops
    ops.check_status(DEV)


@pytest.mark.parametrize("overlap", [True, False])
@pytest.mark.parametrize("graphs", [True, False])
def test_engine_with_decode_graphs_and_overlapped_steps_generates_the_same_tokens(model_dirs, graphs, overlap):
    """Tokens sampled by one step go into the next on the device (graphs replayed or not) while the host
    reads them one step late: the same tokens as the plain implementation, greedy and sampled."""
    config, weights = plain_model.read_model_folder(model_dirs["A"], DEV)
    rng = random.Random(8)
    prompts = [helpers.random_prompt(rng, n, 256) for n in (5, 17, 33, 1, 40, 12)]
    engine = engine_for(model_dirs["A"], "A", "float32", cuda_graph=graphs, max_num_seqs=4, overlap_steps=overlap)
    outputs = engine.generate(prompts, max_tokens=10)
    for prompt, out in zip(prompts, outputs):
        assert out.token_ids == plain_model.greedy_generate(config, weights, prompt, 10)
    assert (engine.runner.graph_replays > 0) == graphs and engine.cache.used_pages == 0 and engine._in_flight is None
    sampled = engine.generate(prompts, max_tokens=10, temperature=0.7, top_k=12, seed=5)
    alone = [engine_for(model_dirs["A"], "A", "float32", overlap_steps=False).generate([p], max_tokens=10, temperature=0.7, top_k=12, seed=5 + i)[0].token_ids
             for i, p in enumerate(prompts)]
    assert [o.token_ids for o in sampled] == alone
    from flexengine_b200 import ops
    ops.check_status(DEV)


def test_carry_tokens_kernel():
    from flexengine_b200 import ops
    token_ids = torch.arange(10, dtype=torch.int32, device=DEV)
    previous = torch.tensor([70, 71, 72], dtype=torch.int32, device=DEV)
    rows = torch.tensor([4, -1, 0, 9], dtype=torch.int32, device=DEV)
    sources = torch.tensor([2, 0, 0, 1], dtype=torch.int32, device=DEV)
    ops.carry_tokens(token_ids, rows, sources, previous)
    assert token_ids.tolist() == [70, 1, 2, 3, 72, 5, 6, 7, 8, 71]
    ops.check_status(DEV)


def test_generate_command_line(model_dirs, capsys):
    """``flexengine generate`` on a model folder and with --random-weights, options under the reference's names."""
    import json
    from flexengine_b200.cli import main
    main(["generate", "--model", model_dirs["A"], "--prompt-ids", "3 14 15 92 65", "--prompt-ids", "7,8,9", "--max-tokens", "6",
          "--dtype", "float32", "--token-budget", "16", "--block-size", "16", "--num-blocks", "16", "--max-model-len", "128",
          "--max-num-seqs", "2", "--policy", "decode_first"])
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    config, weights = plain_model.read_model_folder(model_dirs["A"], DEV)
    assert lines[0]["token_ids"] == plain_model.greedy_generate(config, weights, [3, 14, 15, 92, 65], 6)
    assert lines[1]["token_ids"] == plain_model.greedy_generate(config, weights, [7, 8, 9], 6)
    main(["generate", "--model", model_dirs["A"], "--random-weights", "--weights-seed", "2", "--prompt-ids", "1 2 3", "--max-tokens", "4",
          "--temperature", "0.7", "--top-k", "10", "--seed", "5", "--num-blocks", "16", "--max-model-len", "128", "--cuda-graph"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert len(out["token_ids"]) == 4 and out["finish_reason"] in ("length", "stop")


def test_generate_command_line_with_text_prompts(model_dirs, tmp_path, capsys):
    """A folder with ``tokenizer.json``: text in, text out; the words of this tokenizer are ``<id>``."""
    import json
    import shutil
    tokenizers = pytest.importorskip("tokenizers")
    from flexengine_b200.cli import main
    folder = tmp_path / "with_tokenizer"
    shutil.copytree(model_dirs["A"], folder)
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel({f"<{t}>": t for t in range(256)}, unk_token="<0>"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.WhitespaceSplit()
    tok.decoder = tokenizers.decoders.Fuse()
    tok.save(str(folder / "tokenizer.json"))
    main(["generate", "--model", str(folder), "--prompt", "<3> <14> <15> <92> <65>", "--max-tokens", "6", "--dtype", "float32",
          "--num-blocks", "16", "--max-model-len", "128"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    config, weights = plain_model.read_model_folder(model_dirs["A"], DEV)
    want = plain_model.greedy_generate(config, weights, [3, 14, 15, 92, 65], 6)
    assert out["token_ids"] == want and out["prompt_tokens"] == 5
    assert out["text"].replace(" ", "") == "".join(f"<{t}>" for t in want if t != 255)


@pytest.mark.parametrize("policy", ["fcfs", "adaptive", "slo_aware"])
def test_engine_under_churn_matches_the_plain_implementation(model_dirs, policy):
    """Requests arrive while others run, some are cancelled on the way, pages are so few that requests are
    preempted and recomputed, batches shrink and grow across the graph buckets, steps overlap: every request that
    finishes has the plain implementation's greedy tokens, every cancelled one a prefix of them."""
    config, weights = plain_model.read_model_folder(model_dirs["A"], DEV)
    rng = random.Random(21)
    engine = engine_for(model_dirs["A"], "A", "float32", cuda_graph=True, max_num_seqs=6, pages=7, budget=40,
                        max_model_len=96, scheduler_policy=policy, prefill_chunk_size=16)
    todo = [(helpers.random_prompt(rng, rng.choice([1, 3, 9, 17, 30, 44]), 256), rng.randint(1, 12)) for _ in range(30)]
    live, done, cancelled = [], [], []
    while todo or live:
        for _ in range(rng.randint(0, 2)):
            if todo and len(engine.waiting) < 8:
                prompt, n = todo.pop()
                live.append((engine.submit(prompt, max_tokens=n), prompt, n))
        if live and rng.random() < 0.08:
            victim = live.pop(rng.randrange(len(live)))
            engine.cancel(victim[0].request_id)
            cancelled.append(victim)
        progressed = engine.step()
        assert engine.fault is None
        still = []
        for item in live:
            (done if item[0].state.value == "finished" else still).append(item)
        live = still
        assert progressed or todo or not live
    engine.drain()
    assert engine.cache.used_pages == 0 and engine.preemption_count > 0 and len(done) >= 20
    assert len(engine.runner._graphs) >= 3
    for req, prompt, n in done:
        assert req.generated_ids == plain_model.greedy_generate(config, weights, prompt, n)
    for req, prompt, n in cancelled:
        assert -1 not in req.generated_ids
        assert req.generated_ids == plain_model.greedy_generate(config, weights, prompt, n)[:len(req.generated_ids)]
    from flexengine_b200 import ops
    ops.check_status(DEV)
    engine.cache.assert_invariants()
