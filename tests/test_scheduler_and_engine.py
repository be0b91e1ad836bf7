"""The scheduler's decisions and the engine's behaviour, on the CPU.

The engine runs the real model, step function and cache manager with the PyTorch kernel
references as its kernel provider, so generated tokens can be compared with the plain
implementation; decisions that do not need a model use a counting stand-in for the runner."""
from dataclasses import replace

import pytest
import torch

import helpers
import kernel_refs
import plain_model
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import EngineConfig
from flexengine_b200.engine.request import Request, State
from flexengine_b200.engine.runtime import BusyError, Engine
from flexengine_b200.engine.scheduler import Scheduler
from flexengine_b200.parts.spec import CacheGroupSpec
from flexengine_b200.sampling import Sampler


def req(name, prompt, cached=0, generated=None, priority=0):
    r = Request(name, list(prompt), 10, priority=priority)
    r.cached_tokens = cached
    r.generated_ids = list(generated or [])
    r.transition(State.RUNNING)
    return r


# ---- scheduler --------------------------------------------------------------------------------------
def test_token_budget_and_chunked_prefill():
    a, b = req("a", range(30)), req("b", range(20))
    plan = Scheduler("fcfs", 16, 1000, 100).plan([a, b])
    assert sum(len(c.input_ids) for c in plan) <= 16 and len(plan[0].input_ids) == 16
    assert plan[0].wants_logits is False                 # the context is not complete yet
    a.cached_tokens = 16
    plan = Scheduler("fcfs", 16, 1000, 100).plan([a, b])
    assert [(c.request_id, len(c.input_ids), c.start, c.wants_logits) for c in plan] == [("a", 14, 16, True), ("b", 2, 0, False)]


def test_decode_first_order_and_adaptive_cap():
    prefill = req("p", [2, 3, 4, 5, 6])
    decoding = req("d", [1, 2], cached=2, generated=[7])
    plan = Scheduler("decode_first", 4, 1000, 100).plan([prefill, decoding])
    assert [(c.request_id, len(c.input_ids)) for c in plan] == [("d", 1), ("p", 3)]
    assert plan[0].input_ids == [7] and plan[0].start == 2 and plan[0].wants_logits
    long = req("p", range(40))
    decodes = [req(f"d{i}", [1, 2], cached=2, generated=[7]) for i in range(3)]
    plan = Scheduler("adaptive", 8, 1000, 100, prefill_chunk_size=4).plan([long, *decodes])
    assert [c.request_id for c in plan[:3]] == ["d0", "d1", "d2"]
    assert len(next(c for c in plan if c.request_id == "p").input_ids) == 4
    assert sum(len(c.input_ids) for c in plan) == 7


def test_overdue_prefill_goes_first_and_slo_order():
    prefill = req("p", range(40))
    prefill.arrived -= 2.0
    decode = req("d", [1, 2], cached=2, generated=[7])
    plan = Scheduler("adaptive", 5, 1000, 100, prefill_chunk_size=4).plan([decode, prefill])
    assert [c.request_id for c in plan] == ["p", "d"]
    urgent, relaxed = req("u", [1, 2, 3]), req("r", [1, 2, 3])
    urgent.arrived -= 1.5
    plan = Scheduler("slo_aware", 3, 2000, 200).plan([relaxed, urgent])
    assert plan[0].request_id == "u"


def test_replaying_request_wants_no_logits_and_lifecycle():
    r = req("a", [1, 2, 3], cached=0, generated=[9, 8])
    r.replaying = True
    plan = Scheduler("fcfs", 16, 1000, 100).plan([r])
    assert plan[0].input_ids == [1, 2, 3, 9] and plan[0].wants_logits is False
    r.transition(State.FINISHED)
    with pytest.raises(ValueError):
        r.transition(State.RUNNING)
    with pytest.raises(ValueError):
        Scheduler("random", 1, 1, 1)


# ---- engine with a counting stand-in for the model -----------------------------------------------------
class CountingRunner:
    """Stands in for ModelRunner: logits put all mass on (last token + 1) mod vocab."""
    vocab_size = 32

    def __init__(self, pages, page_size, max_requests, fail_at=None):
        groups = [CacheGroupSpec("kv", "full", slots=1, kv_heads=1, head_dim=2), CacheGroupSpec("state", "state", slots=1, state_shape=(0,))]
        self.cache = CacheManager(groups, pages, page_size, max_requests, torch.float32, "cpu")
        self.ops = kernel_refs
        self.device = torch.device("cpu")
        self.calls = []
        self.fail_at = fail_at

    def step(self, entries, carried=None):
        if self.fail_at is not None and len(self.calls) >= self.fail_at:
            raise RuntimeError("injected executor failure")
        self.calls.append([(e.request_id, len(e.tokens), list(e.want)) for e in entries])
        rows = []
        for e in entries:
            start = self.cache.tokens_of(e.request_id)
            assert self.cache.reserved_tokens(e.request_id) >= start + len(e.tokens)
            self.cache.commit(e.request_id, len(e.tokens))
            tokens = e.tokens if e.carry is None else [int(carried[e.carry])]     # a token the host has not read yet
            for w in e.want:
                row = torch.full((32,), -100.0)
                row[(tokens[w] + 1) % 32] = 10.0
                rows.append(row)
        return torch.stack(rows) if rows else None


def counting_engine(**kw):
    cfg = EngineConfig(model="test", device="cpu", dtype="float32", max_model_len=kw.pop("max_model_len", 64),
                       max_num_seqs=kw.pop("max_num_seqs", 4), max_num_batched_tokens=kw.pop("budget", 8),
                       max_waiting=kw.pop("max_waiting", 8), kv_block_size=kw.pop("page", 4),
                       kv_num_blocks=kw.pop("pages", 20), max_output_tokens=16, trace_steps=False, **kw)
    runner = CountingRunner(cfg.kv_num_blocks, cfg.kv_block_size, cfg.max_num_seqs)
    return Engine(cfg, runner, sampler=Sampler(kernel_refs), eos_token_ids=(0,))


def run_until_done(engine, requests, limit=300):
    for _ in range(limit):
        if all(r.state in (State.FINISHED, State.FAILED, State.CANCELLED) for r in requests):
            return
        engine.step()
    raise AssertionError("requests did not finish")


def test_continuous_batching_finishes_and_frees():
    e = counting_engine()
    a, b = e.submit([5, 6, 7, 8], max_tokens=5), e.submit([20], max_tokens=3)
    run_until_done(e, [a, b])
    assert a.generated_ids == [9, 10, 11, 12, 13] and b.generated_ids == [21, 22, 23]
    assert a.finish_reason == b.finish_reason == "length"
    assert e.cache.used_pages == 0 and not e.cache.requests
    e.cache.assert_invariants()
    # logits were asked for only where a token was sampled
    assert all(len(w) <= 1 for call in e.runner.calls for _, _, w in call)
    assert sum(len(w) for call in e.runner.calls for _, _, w in call) == 8


def test_stop_token_cancel_and_backpressure():
    e = counting_engine(max_waiting=1)
    a = e.submit([30], max_tokens=9)                      # 31, then 0 = end of sequence
    with pytest.raises(BusyError):
        e.submit([1], max_tokens=2)
    run_until_done(e, [a])
    assert a.generated_ids == [31, 0] and a.finish_reason == "stop"
    b = e.submit([1, 2, 3], max_tokens=9)
    e.step(); e.step()
    assert e.cancel(b.request_id) and b.state is State.CANCELLED and not e.cancel(b.request_id)
    assert e.cache.used_pages == 0
    with pytest.raises(ValueError, match="max_model_len"):
        e.submit([1] * 59, max_tokens=10)
    with pytest.raises(ValueError, match="token id"):
        e.submit([99], max_tokens=2)
    with pytest.raises(ValueError):
        e.submit([1], max_tokens=2, temperature=9.0)


def test_pages_run_out_preempts_and_recomputes_without_a_second_sample():
    # 3 pages of 4 tokens.  The first step gives the older request one page and the younger two;
    # when the older one needs its second page none is free, and the younger one is preempted
    e = counting_engine(pages=3, page=4, max_model_len=12, max_num_seqs=2, budget=16)
    a, b = e.submit([1, 2, 3], max_tokens=5), e.submit([11, 12, 13, 14, 15, 16], max_tokens=4)
    run_until_done(e, [a, b])
    assert a.generated_ids == [4, 5, 6, 7, 8] and b.generated_ids == [17, 18, 19, 20]
    assert b.preemptions >= 1 and a.preemptions == 0
    assert e.preemption_count >= 1 and (a.preemptions + b.preemptions) == e.preemption_count
    assert e.cache.free_pages == 3
    e.cache.assert_invariants()


def test_forced_preemption_keeps_outputs():
    e = counting_engine()
    a = e.submit([1, 2, 3, 4], max_tokens=7)
    for _ in range(4):
        e.step()
    e.drain()                                   # the last step's token is read before it is compared
    before = list(a.generated_ids)
    assert before
    e.preempt(a)
    assert a.state is State.PREEMPTED and a.cached_tokens == 0 and a.replaying and e.cache.used_pages == 0
    run_until_done(e, [a])
    assert a.generated_ids[:len(before)] == before and a.generated_ids == [5, 6, 7, 8, 9, 10, 11]
    assert e.cache.free_pages == e.cache.total_pages


def test_chunk_that_cannot_get_pages_waits_for_the_next_step():
    # one request holds all pages and is planned first; the other is left out until pages return
    e = counting_engine(pages=2, page=4, max_model_len=8, max_num_seqs=2, budget=8)
    a = e.submit([1, 2, 3, 4, 5], max_tokens=3)
    b = e.submit([9, 10], max_tokens=2)
    run_until_done(e, [a, b])
    assert a.generated_ids == [6, 7, 8] and b.generated_ids == [11, 12]
    assert e.cache.free_pages == 2


def test_executor_failure_faults_the_engine_and_frees_everything():
    e = counting_engine()
    e.runner.fail_at = 2
    a, b = e.submit([1, 2], max_tokens=5), e.submit([3, 4], max_tokens=5)
    for _ in range(5):
        e.step()
    assert e.fault and "injected" in e.fault
    assert a.state is State.FAILED and b.state is State.FAILED and e.cache.used_pages == 0
    with pytest.raises(BusyError):
        e.submit([1], max_tokens=1)


def test_a_fault_recorded_by_a_kernel_fails_the_requests():
    """Kernels record a guarded fault (an index they had to skip, a bounded wait that ran out) in a status word
    on the device; the engine reads it with each step's tokens.  A set bit fails every live request and closes
    the engine: what was sampled from such a step is not handed out as tokens."""
    import types
    word = torch.zeros(1, dtype=torch.int32)
    e = counting_engine()
    e.runner.ops = types.SimpleNamespace(status_word=lambda device: word,
                                         describe_status=lambda v: "a bounded wait ran out" if v & 8 else str(v))
    a, b = e.submit([1, 2], max_tokens=6), e.submit([3, 4], max_tokens=6)
    e.step(); e.step(); e.drain()
    assert a.generated_ids == [3, 4] and e.fault is None
    word[0] = 8
    tokens_before = len(a.generated_ids)
    for _ in range(3):
        e.step()
    assert e.fault and "bounded wait" in e.fault
    assert a.state is State.FAILED and b.state is State.FAILED and e.cache.used_pages == 0
    assert len(a.generated_ids) == tokens_before and -1 not in a.generated_ids       # nothing of the bad step came out
    assert a.events.get_nowait().kind == "token"
    with pytest.raises(BusyError):
        e.submit([1], max_tokens=1)


def test_slo_aware_policy_end_to_end():
    """The policy that orders by slack, through whole generations: same tokens as any other policy, everything freed."""
    e = counting_engine(scheduler_policy="slo_aware", budget=5, ttft_slo_ms=50.0, itl_slo_ms=5.0)
    requests = [e.submit([2 + 3 * i] * (1 + 2 * i), max_tokens=3 + i % 3, priority=i % 3 - 1) for i in range(6)]
    run_until_done(e, requests)
    e.drain()
    for i, r in enumerate(requests):
        first = 2 + 3 * i + 1
        assert r.generated_ids == list(range(first, first + 3 + i % 3)) and r.finish_reason == "length"
    assert e.cache.used_pages == 0 and not e.cache.requests
    assert all(sum(n for _, n, _ in call) <= 5 for call in e.runner.calls)


def test_worker_thread_serves_requests_and_stop_cancels_the_rest():
    """``start()`` runs the step loop on a thread of its own (the reference's serving mode); clients
    read their request's event queue; ``stop()`` cancels what is still alive and frees its pages."""
    import time
    e = counting_engine()
    e.start()
    a = e.submit([5, 6, 7], max_tokens=4)
    events = []
    deadline = time.time() + 10
    while time.time() < deadline:
        ev = a.events.get(timeout=5)
        events.append(ev)
        if ev.kind == "done":
            break
    assert [ev.token_id for ev in events if ev.kind == "token"] == [8, 9, 10, 11] and events[-1].finish_reason == "length"
    b = e.submit([3] * 39, max_tokens=16)
    e.stop()
    assert b.state in (State.CANCELLED, State.FINISHED) and e.cache.used_pages == 0
    snap = e.snapshot()
    assert snap["requests_total"] == 2 and snap["fault"] is None and snap["cache_free_blocks"] == e.cache.total_pages


def test_step_trace_is_written(tmp_path):
    import json
    e = counting_engine(trace_dir=str(tmp_path))
    e.config = replace(e.config, trace_steps=True)
    e.submit([1, 2, 3, 4], max_tokens=2)
    assert e.step()
    record = json.loads((tmp_path / "steps.jsonl").read_text().splitlines()[0])
    assert record["new_tokens"] == 4 and record["scheduler_ms"] >= 0 and record["wall_ms"] >= record["executor_wall_ms"]
    assert (tmp_path / "run_metadata.json").exists()


# ---- the real model on the CPU through the engine ------------------------------------------------------
@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    return helpers.make_model_dir(tmp_path_factory, "A", seed=21)


def real_engine(model_dir, **kw):
    cfg = EngineConfig(model=model_dir, device="cpu", dtype="float32", max_model_len=kw.pop("max_model_len", 128), max_num_seqs=kw.pop("max_num_seqs", 4),
                       max_num_batched_tokens=kw.pop("budget", 24), kv_block_size=16, kv_num_blocks=kw.pop("pages", 16),
                       max_output_tokens=16, **kw)
    return Engine.from_model_dir(model_dir, cfg, ops=kernel_refs)


def test_greedy_generation_matches_the_plain_implementation(model_a):
    config, weights = plain_model.read_model_folder(model_a)
    prompts = [[3, 14, 15, 92, 65], list(range(40, 57)), [7, 200] * 16 + [1]]
    for policy in ("fcfs", "decode_first", "adaptive"):
        engine = real_engine(model_a, scheduler_policy=policy, prefill_chunk_size=6)
        outputs = engine.generate(prompts, max_tokens=8)
        for prompt, out in zip(prompts, outputs):
            assert out.token_ids == plain_model.greedy_generate(config, weights, prompt, 8), policy
        assert engine.cache.used_pages == 0


def test_sampled_tokens_do_not_depend_on_batching_or_preemption(model_a):
    prompts = [list(range(60, 72)), [7, 200] * 16 + [1], [3, 14, 15, 92, 65], [9]]
    alone = []
    for i, p in enumerate(prompts):
        engine = real_engine(model_a)
        alone.append(engine.generate([p], max_tokens=8, temperature=0.8, top_k=20, seed=100 + i)[0].token_ids)
    together = real_engine(model_a, budget=5, scheduler_policy="decode_first")
    outs = together.generate(prompts, max_tokens=8, temperature=0.8, top_k=20, seed=100)
    assert [o.token_ids for o in outs] == alone
    # so few pages that requests are preempted and recomputed
    # 4 pages: the first step gives the older request 1 page and the younger 3; the older one's
    # second page then costs the younger one its place, and it recomputes later
    tight = real_engine(model_a, pages=4, budget=48, max_num_seqs=2, max_model_len=64)
    outs = tight.generate(prompts, max_tokens=8, temperature=0.8, top_k=20, seed=100)
    assert [o.token_ids for o in outs] == alone
    assert tight.preemption_count >= 1 and tight.cache.used_pages == 0
    assert len(set(map(tuple, alone))) > 1


# ---- launching a step before the tokens of the one before have been read ------------------------------------
def test_overlapped_steps_give_the_same_tokens_and_drop_the_token_run_too_far():
    """Counting model, end-of-sequence token 0: a request that starts at 28 stops after 29, 30, 31, 0.  With
    overlap it has been run one step further by the time the host sees the 0; that token is dropped."""
    results = {}
    for overlap in (False, True):
        e = counting_engine(overlap_steps=overlap)
        a, b, c = e.submit([1, 2, 28], max_tokens=9), e.submit([5], max_tokens=6), e.submit([30], max_tokens=9)
        run_until_done(e, [a, b, c])
        e.drain()
        results[overlap] = [(r.generated_ids, r.finish_reason) for r in (a, b, c)]
        assert e.cache.used_pages == 0 and not e.cache.requests and e._in_flight is None
        e.cache.assert_invariants()
        assert all(-1 not in r.generated_ids for r in (a, b, c))
        steps_with_a = sum(1 for call in e.runner.calls if any(rid == a.request_id for rid, _, _ in call))
        assert steps_with_a == (5 if overlap else 4)            # prompt, 29, 30, 31 (, and the 0 when overlapped)
    assert results[True] == results[False]
    assert results[True][0] == ([29, 30, 31, 0], "stop") and results[True][1] == ([6, 7, 8, 9, 10, 11], "length")
    assert results[True][2] == ([31, 0], "stop")


def test_a_request_at_its_last_token_is_not_run_again_and_cancel_meets_a_token_on_its_way():
    e = counting_engine()
    a = e.submit([3], max_tokens=2)
    e.step()                                        # prompt -> first token on its way
    e.step()                                        # first token (carried) -> second token on its way
    assert a.generated_ids[-1] == -1 and a.awaits_last_token
    assert e.scheduler.plan(list(e.running.values())) == []
    assert e.step() is True and a.state is State.FINISHED and a.generated_ids == [4, 5]
    assert e.step() is False and len(e.runner.calls) == 2
    b = e.submit([7], max_tokens=5)
    e.step()
    e.step()
    assert e.cancel(b.request_id) and b.state is State.CANCELLED and -1 not in b.generated_ids
    assert e.step() is True and e.step() is False   # the token on its way finds its request gone
    assert e.cache.used_pages == 0 and b.generated_ids == [8]
    e.cache.assert_invariants()


def test_carried_tokens_in_the_step_function(model_a):
    """A decode step whose tokens come from a tensor (as the step before left them) gives the logits of the
    same step with the tokens in hand; entries with and without a carried token side by side."""
    from flexengine_b200.engine import StepEntry

    def runner():
        return Engine.from_model_dir(model_a, EngineConfig(model=model_a, device="cpu", dtype="float32", max_model_len=64,
                                                           max_num_seqs=4, kv_block_size=16, kv_num_blocks=8),
                                     ops=kernel_refs).runner
    one, two = runner(), runner()
    prompts = {"x": [3, 14, 15, 92], "y": [6, 5], "z": [9, 9, 9]}
    for r in (one, two):
        r.step([StepEntry(rid, ids, []) for rid, ids in prompts.items()])
    want = one.step([StepEntry("x", [41], [0]), StepEntry("y", [7], [0]), StepEntry("z", [200, 11], [1])])
    carried = torch.tensor([7, 99, 41], dtype=torch.int32)
    got = two.step([StepEntry("x", [0], [0], carry=2), StepEntry("y", [0], [0], carry=0), StepEntry("z", [200, 11], [1])], carried)
    torch.testing.assert_close(got, want, atol=0, rtol=0)
    with pytest.raises(ValueError, match="carried"):
        two.step([StepEntry("x", [0], [0], carry=5)], carried)
    with pytest.raises(ValueError, match="carried"):
        two.step([StepEntry("x", [0], [0], carry=0)])


@pytest.mark.parametrize("overlap", [True, False])
def test_end_of_sequence_with_the_real_model_under_tight_pages(model_a, overlap):
    """An end-of-sequence id that greedy generation does produce: every request stops at its first
    occurrence, whatever was launched beyond it, also when pages are so few that requests are preempted."""
    config, weights = plain_model.read_model_folder(model_a)
    prompts = [[3, 14, 15, 92, 65], list(range(40, 57)), [7, 200] * 16 + [1], [9], list(range(100, 130))]
    plain = [plain_model.greedy_generate(config, weights, p, 10) for p in prompts]
    eos = plain[1][4]
    want = [t[:t.index(eos) + 1] if eos in t else t for t in plain]
    assert any(len(w) < 10 for w in want)
    for kw in (dict(), dict(pages=5, budget=48, max_num_seqs=3, max_model_len=64)):
        base = real_engine(model_a, overlap_steps=overlap, **kw)
        engine = Engine(base.config, base.runner, eos_token_ids=(eos,))
        outs = engine.generate(prompts, max_tokens=10)
        assert [o.token_ids for o in outs] == want
        assert [o.finish_reason for o in outs] == ["stop" if w[-1] == eos else "length" for w in want]
        assert engine.cache.used_pages == 0 and engine._in_flight is None
        engine.cache.assert_invariants()


@pytest.mark.parametrize("policy", ["fcfs", "decode_first"])
def test_engine_under_churn_on_the_cpu(model_a, policy):
    """Arrivals, cancellations and so few pages that requests are preempted, with steps overlapped: finished
    requests have the plain implementation's greedy tokens, cancelled ones a prefix of them."""
    import random
    import helpers
    config, weights = plain_model.read_model_folder(model_a)
    rng = random.Random(21)
    engine = real_engine(model_a, max_num_seqs=6, pages=7, budget=40, max_model_len=96, scheduler_policy=policy,
                         prefill_chunk_size=16)
    todo = [(helpers.random_prompt(rng, rng.choice([1, 3, 9, 17, 30, 44]), 256), rng.randint(1, 12)) for _ in range(24)]
    live, done, cancelled = [], [], []
    for _ in range(3000):
        if not (todo or live):
            break
        for _ in range(rng.randint(0, 2)):
            if todo and len(engine.waiting) < 8:
                prompt, n = todo.pop()
                live.append((engine.submit(prompt, max_tokens=n), prompt, n))
        if live and rng.random() < 0.08:
            victim = live.pop(rng.randrange(len(live)))
            engine.cancel(victim[0].request_id)
            cancelled.append(victim)
        engine.step()
        assert engine.fault is None
        done += [item for item in live if item[0].state is State.FINISHED]
        live = [item for item in live if item[0].state is not State.FINISHED]
    engine.drain()
    assert not todo and not live and engine.cache.used_pages == 0 and engine.preemption_count > 0 and cancelled
    engine.cache.assert_invariants()
    for req, prompt, n in done:
        assert req.generated_ids == plain_model.greedy_generate(config, weights, prompt, n)
    for req, prompt, n in cancelled:
        assert -1 not in req.generated_ids
        assert req.generated_ids == plain_model.greedy_generate(config, weights, prompt, n)[:len(req.generated_ids)]


def test_overlapped_steps_plan_the_same_batches_when_requests_end_by_length():
    """A request whose last token is on its way gives up its seat and its pages at once, so that requests which
    wait are admitted in the same step as without overlap: the same batches, step for step."""
    calls = {}
    for overlap in (False, True):
        e = counting_engine(overlap_steps=overlap, max_num_seqs=2)
        requests = [e.submit([1 + i], max_tokens=2 + i % 3) for i in range(7)]       # tokens stay below the end-of-sequence id
        run_until_done(e, requests)
        e.drain()
        calls[overlap] = [[(n, w) for _, n, w in call] for call in e.runner.calls]
        assert e.cache.used_pages == 0 and [r.finish_reason for r in requests] == ["length"] * 7
        e.cache.assert_invariants()
    assert calls[True] == calls[False]
