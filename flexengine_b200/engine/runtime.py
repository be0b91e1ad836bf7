"""The engine: requests come in, take a seat, are run in steps, sampled, and leave.

What happens is what the reference's runtime does (src/flexengine/engine/runtime.py): ``submit`` checks and queues a
request (runtime.py:89-121); a step seats waiting requests while fewer than ``max_num_seqs`` run
(runtime.py:162-179), asks the scheduler for chunks under the token budget (runtime.py:262), and reserves pages
chunk by chunk; when pages run out ONE running request that is not part of this step is preempted (lowest
priority, then the one holding most cached tokens), the reservation is tried once more, and otherwise the chunk
waits for a later step (runtime.py:273-288); a preempted request gives everything back, queues again and later
recomputes its context without sampling from it a second time (runtime.py:242-251,318-324); a token of the
end-of-sequence set ends a request with "stop", its ``max_tokens``-th token with "length" (runtime.py:343-346);
an exception in the executor, or a fault that a kernel recorded, fails every live request and closes the engine
(runtime.py:349-356).  Logits are asked for only where a token will be sampled.

How it happens is this engine's own.  A step is launched before the host has read the tokens of the step before
(``overlap_steps``): sampled tokens stay on the device, the next step takes them from there
(``StepEntry.carry``), and the host reads them, together with the kernels' status word, from pinned memory one
step late, while the device is busy.  Until then ``generated_ids`` holds ``PENDING`` in the token's place.  A
request that turns out to have ended with an end-of-sequence token has been run one token too far; that token
is dropped.  A request whose pending token is its last by ``max_tokens`` leaves its seat at once, so that the
batches are the same, step for step, as without overlap.  Before anyone is preempted the tokens on their way
are read, so that preemption and recomputation see exact state.
"""
from __future__ import annotations

import math
import threading
import time
import uuid
from collections import OrderedDict, deque
from dataclasses import dataclass

import torch

from ..cache.manager import CacheManager
from ..cache.page_pool import CacheExhausted
from ..config.engine_config import EngineConfig
from ..observability.traces import RunTrace, marked
from ..sampling.sampler import Sampler
from .request import PENDING, TERMINAL, Event, Request, State
from .scheduler import Scheduler
from .step import ModelRunner, StepEntry

TEMPERATURE_RANGE = (0.0, 5.0)          # the reference's bounds (runtime.py:95)


class BusyError(RuntimeError):
    """The engine takes no request now: its waiting queue is full, or it has stopped or faulted."""


@dataclass
class GenerationOutput:
    request_id: str
    prompt_ids: list
    token_ids: list
    text: str
    finish_reason: str | None


@dataclass
class _InFlight:
    """A launched step whose sampled tokens the host has not read yet."""
    places: list                         # [(request, index in its generated_ids)] in the order of ``tokens``
    tokens: torch.Tensor | None          # int32 [len(places)] on the device
    where: dict                          # request id -> index in ``tokens`` (for the next step's carry)
    host: torch.Tensor | None = None     # pinned: the tokens, then the kernels' status word
    ready: object = None                 # event after the copy into ``host``


@dataclass
class _Counters:
    steps: int = 0
    submitted: int = 0
    ended: int = 0
    preemptions: int = 0
    output_tokens: int = 0


class Engine:
    def __init__(self, config: EngineConfig, runner: ModelRunner, sampler: Sampler | None = None, tokenizer=None,
                 eos_token_ids=()):
        if runner.cache.capacity_tokens() < config.max_model_len:
            raise ValueError("KV pool cannot contain one max-length request")
        self.config = config
        self.runner = runner
        self.cache: CacheManager = runner.cache
        self.sampler = sampler if sampler is not None else Sampler(runner.ops)
        self.tokenizer = tokenizer
        self.eos_ids = frozenset(int(t) for t in eos_token_ids)
        self.scheduler = Scheduler(config.scheduler_policy, config.max_num_batched_tokens, config.ttft_slo_ms,
                                   config.itl_slo_ms, config.prefill_chunk_size,
                                   granularity=getattr(self.cache, "chunk_granularity", 1))
        self.waiting: deque = deque()              # arrival order; preempted requests rejoin at the back
        self.running: OrderedDict = OrderedDict()  # request id -> request, the seats
        self.all_requests: dict = {}               # every request that has not ended
        self.lock = threading.RLock()
        self.fault: str | None = None
        self.counters = _Counters()
        self._closing = threading.Event()
        self._thread: threading.Thread | None = None
        self._in_flight: _InFlight | None = None
        self._landing: list = []                   # pinned buffers the tokens are copied into, used in turn
        self._landing_at = 0
        self.trace = RunTrace(config.trace_dir)
        self.trace.describe(config)

    # ---- built from a model ------------------------------------------------------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, config: EngineConfig | None = None, tokenizer=None, ops=None) -> "Engine":
        from ..weights.loader import load_model
        config = config or EngineConfig(model=model_dir)
        _typed, _plan, model = load_model(model_dir, config.dtype, config.device)
        return cls.from_model(model, config, tokenizer=tokenizer, ops=ops)

    @classmethod
    def from_model(cls, model, config: EngineConfig, tokenizer=None, ops=None) -> "Engine":
        plan = model.plan
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[config.dtype]
        pages = config.kv_num_blocks or pages_that_fit(plan, config, dtype)
        cache = CacheManager(plan.cache_groups, pages, config.kv_block_size, config.max_num_seqs, dtype, config.device)
        runner = ModelRunner(model, cache, ops=ops)
        if config.cuda_graph:
            runner.enable_decode_graphs(config.max_num_seqs, config.max_model_len)
            runner.capture_decode_graphs()         # when the engine is built, not in the path of the first requests
        return cls(config, runner, tokenizer=tokenizer, eos_token_ids=plan.eos_token_ids)

    # ---- counters under the names callers know -----------------------------------------------------------------
    @property
    def preemption_count(self) -> int:
        return self.counters.preemptions

    @property
    def step_index(self) -> int:
        return self.counters.steps

    @property
    def output_tokens(self) -> int:
        return self.counters.output_tokens

    def snapshot(self) -> dict:
        with self.lock:
            c = self.counters
            return {"waiting": len(self.waiting), "running": len(self.running), "fault": self.fault,
                    "cache_used_blocks": self.cache.used_pages, "cache_free_blocks": self.cache.free_pages,
                    "steps": c.steps, "requests_total": c.submitted, "requests_completed": c.ended,
                    "preemptions": c.preemptions, "output_tokens": c.output_tokens}

    # ---- requests come in ---------------------------------------------------------------------------------------
    def _token_ids(self, prompt) -> list:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; pass token ids instead")
            ids = list(self.tokenizer.encode(prompt, add_special_tokens=False)) if prompt else []
            if not ids:
                start = getattr(self.tokenizer, "bos_token_id", None)
                if not prompt or start is None:
                    raise ValueError("the prompt is empty")
                ids = [start]
            return ids
        ids = [int(t) for t in prompt]
        if not ids:
            raise ValueError("the prompt is empty")
        vocab = self.runner.vocab_size
        if min(ids) < 0 or max(ids) >= vocab:
            raise ValueError(f"token id outside [0, {vocab})")
        return ids

    def submit(self, prompt, max_tokens: int = 128, temperature: float = 0.0, top_k: int = 0, priority: int = 0,
               seed: int | None = None) -> Request:
        """Queue a request.  ``prompt`` is text (needs a tokenizer) or a list of token ids.  Raises ValueError
        for what can never run and BusyError when the engine takes nothing now."""
        ids = self._token_ids(prompt)
        cfg = self.config
        if not 1 <= max_tokens <= cfg.max_output_tokens:
            raise ValueError(f"max_tokens={max_tokens} is outside 1..{cfg.max_output_tokens} (max_output_tokens)")
        low, high = TEMPERATURE_RANGE
        if not low <= temperature <= high:
            raise ValueError(f"temperature={temperature} is outside {low}..{high}")
        if top_k < 0:
            raise ValueError(f"top_k={top_k} is negative")
        if len(ids) + max_tokens > cfg.max_model_len:
            raise ValueError(f"{len(ids)} prompt tokens + max_tokens={max_tokens} exceed max_model_len={cfg.max_model_len}")
        with self.lock:
            if self.fault or self._closing.is_set():
                raise BusyError("the engine has stopped" if not self.fault else f"the engine faulted: {self.fault}")
            if len(self.waiting) >= cfg.max_waiting:
                raise BusyError(f"{len(self.waiting)} requests are waiting already (max_waiting)")
            request = Request(f"cmpl-{uuid.uuid4().hex}", ids, int(max_tokens), float(temperature), int(top_k), int(priority))
            # a default seed that depends only on the order of submission: the same requests in the same order
            # draw the same tokens under every policy and batching (runtime.py:112-116)
            request.seed = cfg.random_seed + self.counters.submitted if seed is None else int(seed)
            self.counters.submitted += 1
            self.all_requests[request.request_id] = request
            self.waiting.append(request)
        return request

    def cancel(self, request_id: str) -> bool:
        with self.lock:
            request = self.all_requests.get(request_id)
            if request is None or request.state in TERMINAL:
                return False
            self._retire(request, State.CANCELLED, "cancelled")
        return True

    # ---- seats ----------------------------------------------------------------------------------------------------
    def _seat_waiting(self) -> None:
        """Waiting requests take free seats in queue order.  A seat is a state slot; pages come later, chunk by chunk."""
        while self.waiting and len(self.running) < self.config.max_num_seqs:
            request = self.waiting.popleft()
            if request.state in TERMINAL:
                continue
            self.cache.admit(request.request_id)
            request.transition(State.RUNNING)
            self.running[request.request_id] = request

    def _retire(self, request: Request, state: State, reason: str, error: str | None = None) -> None:
        """The request ends: its pages and its seat are free, its consumer is told, its report is written."""
        if request.state in TERMINAL:
            return
        request.transition(state)
        request.finish_reason, request.error, request.finished_at = reason, error, time.monotonic()
        generated = request.generated_ids
        while generated and generated[-1] == PENDING:       # launched beyond its end, or cancelled with a token on its way
            generated.pop()
        rid = request.request_id
        self.cache.free(rid)
        self.running.pop(rid, None)
        self.all_requests.pop(rid, None)
        if request in self.waiting:
            self.waiting.remove(request)
        if state is State.FAILED:
            request.events.put(Event("error", error=error or reason, finish_reason=reason))
        else:
            self._emit_text(request, final=True)
            request.events.put(Event("done", finish_reason=reason))
        self.trace.record("requests", request.report())
        self.counters.ended += 1

    def preempt(self, victim: Request) -> None:
        """Take the request's pages and seat; it queues again and recomputes its context when it is seated next."""
        with self.lock:
            self._land()                              # nobody is preempted with a token on its way
            if victim.state in TERMINAL or victim.request_id not in self.running:
                return
            self.cache.free(victim.request_id)
            del self.running[victim.request_id]
            victim.cached_tokens = 0
            victim.replaying = len(victim.generated_ids) > 0     # its context ends in a token it has sampled already
            victim.preemptions += 1
            victim.transition(State.PREEMPTED)
            self.waiting.append(victim)
            self.counters.preemptions += 1

    def _victim_for(self, needy: Request, taken: set) -> Request | None:
        """Who gives way when ``needy`` finds no page: a seated request outside this step that holds pages;
        the lowest priority first, among equals the one with most tokens cached."""
        best = None
        for other in self.running.values():
            if other is needy or other.request_id in taken or not self.cache.holds_pages(other.request_id):
                continue
            if best is None or (other.priority, -other.cached_tokens) < (best.priority, -best.cached_tokens):
                best = other
        return best

    # ---- one step -------------------------------------------------------------------------------------------------
    def _with_pages(self, proposed: list) -> list:
        """The chunks of ``proposed`` that have their pages, in order.  Up to three tries per chunk: as things are;
        after the tokens on their way were read (requests that just ended gave pages back); after one preemption."""
        granted, taken = [], set()
        held = self.cache.requests
        for chunk in proposed:
            request = self.running.get(chunk.request_id)
            if request is None:
                continue
            upto = chunk.start + len(chunk.input_ids)
            record = held.get(chunk.request_id)
            if record is not None and record.room >= upto:      # the usual case in decode: nothing to reserve
                granted.append(chunk)
                taken.add(chunk.request_id)
                continue
            for attempt in ("as is", "after landing", "after preempting"):
                if attempt == "after landing":
                    if self._in_flight is None:
                        continue
                    self._land()
                elif attempt == "after preempting":
                    victim = self._victim_for(request, taken)
                    if victim is None:
                        break
                    self.preempt(victim)
                if request.request_id not in self.running:
                    break                              # reading tokens ended it
                try:
                    self.cache.reserve(request.request_id, upto)
                except CacheExhausted:
                    continue
                granted.append(chunk)
                taken.add(chunk.request_id)
                break
        return [c for c in granted if c.request_id in self.running]

    def step(self) -> bool:
        """One scheduling iteration.  False when there was nothing to do."""
        with self.lock:
            if self.fault:
                return False
            started = time.perf_counter()
            self._seat_waiting()
            with marked("sched/select"):
                proposed = self.scheduler.plan(list(self.running.values()))
            with marked("kv/reserve"):
                chunks = self._with_pages(proposed)
            if not chunks:
                if self._in_flight is None:
                    return False
                self._land()                           # nothing to launch: the tokens on their way are the progress
                return not self.fault
            planned_at = time.perf_counter()
            tracing = self.config.trace_steps and self.trace.enabled
            tokens = sum(len(c.input_ids) for c in chunks)
            prompt_tokens = sum(len(c.input_ids) for c in chunks if self.running[c.request_id].in_prefill) if tracing else 0
            try:
                with marked(f"executor/step batch={len(chunks)} tokens={tokens}"):
                    launched = self._launch(chunks)
                earlier, self._in_flight = self._in_flight, launched
                self._read(earlier)                    # the step before, while the device runs this one
                if not self.config.overlap_steps:
                    self._land()
            except Exception as ex:  # noqa: BLE001 - whatever the executor raises closes the engine
                self._fail_everything(f"{type(ex).__name__}: {ex}")
                return False
            if self.fault:
                return False
            done_at = time.perf_counter()
            self.counters.steps += 1
            if tracing:
                # keys: the reference's step records (runtime.py:358-383), which its analysis reads
                self.trace.record("steps", {
                    "step": self.counters.steps, "policy": self.config.scheduler_policy, "batch_size": len(chunks),
                    "new_tokens": tokens, "prefill_tokens": prompt_tokens, "decode_tokens": tokens - prompt_tokens,
                    "waiting": len(self.waiting), "running": len(self.running),
                    "kv_used_blocks": self.cache.used_pages, "preemptions": self.counters.preemptions,
                    "scheduler_ms": (planned_at - started) * 1e3, "executor_wall_ms": (done_at - planned_at) * 1e3,
                    "wall_ms": (done_at - started) * 1e3})
            return True

    def _fail_everything(self, why: str) -> None:
        self.fault = why
        self._in_flight = None
        for request in list(self.all_requests.values()):
            self._retire(request, State.FAILED, "error", why)

    def _launch(self, chunks: list) -> _InFlight:
        """Run the chunks and sample; nothing here waits for the device."""
        earlier = self._in_flight
        entries, sampled = [], []
        for chunk in chunks:
            request = self.running[chunk.request_id]
            ids, carry = chunk.input_ids, None
            if ids[-1] == PENDING:                     # planned on a token that was on its way
                newest = request.generated_ids[-1]
                if newest == PENDING:
                    ids, carry = [0], earlier.where[chunk.request_id]
                else:
                    ids = [newest]                     # it has landed since
            entries.append(StepEntry(chunk.request_id, ids, [len(ids) - 1] if chunk.wants_logits else [], carry))
            if chunk.wants_logits:
                sampled.append(request)
        logits = self._run_step(entries, earlier.tokens if earlier is not None else None)
        tokens = None
        if sampled:
            tokens = self.sampler.sample_on_device(logits, [r.temperature for r in sampled], [r.top_k for r in sampled],
                                                   [r.seed for r in sampled], [len(r.generated_ids) for r in sampled])
        now = time.monotonic()
        places = []
        for chunk in chunks:
            request = self.running[chunk.request_id]
            if request.first_scheduled_at is None:
                request.first_scheduled_at = now
            request.cached_tokens += len(chunk.input_ids)
            if not chunk.wants_logits:
                request.replaying = request.replaying and request.in_prefill      # a recomputed context gives no second token
                continue
            request.generated_ids.append(PENDING)
            places.append((request, len(request.generated_ids) - 1))
            if len(request.generated_ids) >= request.max_tokens:
                # whatever the token is, it is the last: seat and pages serve others from the next step on (what
                # that step writes there comes after this one on the stream); the request ends when the token lands
                self.cache.free(request.request_id)
                del self.running[request.request_id]
        record = _InFlight(places, tokens, {r.request_id: i for i, (r, _) in enumerate(places)})
        if tokens is not None and tokens.device.type == "cuda":
            self._copy_out(record)
        return record

    def _run_step(self, entries, carried):
        """The runner's step; one that says it can is told that tokens were checked at submit and pages reserved
        chunk by chunk already."""
        trusts = getattr(self, "_runner_trusts", None)
        if trusts is None:
            import inspect
            trusts = self._runner_trusts = "trusted" in inspect.signature(self.runner.step).parameters
        return self.runner.step(entries, carried, trusted=True) if trusts else self.runner.step(entries, carried)

    def _copy_out(self, record: _InFlight) -> None:
        """Start the copy of the sampled tokens and of the kernels' status word into pinned memory."""
        n = record.tokens.numel()
        if not self._landing or self._landing[0].numel() < n + 1:
            # a few buffers kept for good (two records are alive at most): pinning memory at every step would cost
            # a call into the driver each time
            size = max(n, self.config.max_num_seqs) + 1
            self._landing = [torch.empty(size, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._landing_at = (self._landing_at + 1) % len(self._landing)
        record.host = self._landing[self._landing_at][:n + 1]
        record.host[:n].copy_(record.tokens, non_blocking=True)
        word = getattr(self.runner.ops, "status_word", None)
        if word is not None:
            record.host[n:].copy_(word(record.tokens.device), non_blocking=True)
        else:
            record.host[n] = 0
        record.ready = torch.cuda.Event()
        record.ready.record()

    # ---- tokens come back ----------------------------------------------------------------------------------------
    def drain(self) -> None:
        """Wait for the step launched last and take its tokens in: afterwards no request holds ``PENDING``."""
        with self.lock:
            self._land()

    def _land(self) -> None:
        record, self._in_flight = self._in_flight, None
        self._read(record)

    def _read(self, record: _InFlight | None) -> None:
        if record is None or not record.places:
            return
        if record.ready is not None:
            record.ready.synchronize()
            *values, status = record.host.tolist()
        else:
            values = record.tokens.tolist()
            word = getattr(self.runner.ops, "status_word", None)
            status = int(word(record.tokens.device).item()) if word is not None else 0
        if status:
            # a kernel skipped an index it could not use or gave up a bounded wait: what was sampled from such a
            # step is not to be trusted, and neither is anything launched after it
            explain = getattr(self.runner.ops, "describe_status", None)
            self._fail_everything("kernel status: " + (explain(status) if explain else str(status)))
            return
        now = time.monotonic()
        for (request, place), token in zip(record.places, values):
            if request.state not in TERMINAL:          # else it ended or was cancelled meanwhile: one token too far
                self._take_token(request, place, int(token), now)

    def _take_token(self, request: Request, place: int, token: int, now: float) -> None:
        request.generated_ids[place] = token
        if request.first_token_at is None:
            request.first_token_at = now
        request.last_token_at = now
        request.token_times.append(now)
        self.counters.output_tokens += 1
        if self.tokenizer is None:
            request.events.put(Event("token", token_id=token))
        else:
            self._emit_text(request, upto=place + 1, token=token)
        if token in self.eos_ids:
            self._retire(request, State.FINISHED, "stop")
        elif place + 1 >= request.max_tokens:
            self._retire(request, State.FINISHED, "length")

    def _emit_text(self, request: Request, upto: int | None = None, token: int | None = None, final: bool = False) -> None:
        """Decode what is known of the request's tokens and send the text that is new and settled: a trailing
        replacement character may yet be completed by the next token, so it is held back until the end."""
        if self.tokenizer is None:
            return
        if not final:
            request.text = self.tokenizer.decode(request.generated_ids[:upto], skip_special_tokens=True,
                                                 clean_up_tokenization_spaces=False)
        settled = request.text if final else request.text.rstrip("\ufffd")
        if settled.startswith(request.emitted_text) and len(settled) > len(request.emitted_text):
            fresh = settled[len(request.emitted_text):]
            request.emitted_text = settled
            request.events.put(Event("token", text=fresh, token_id=token))

    # ---- entry points -----------------------------------------------------------------------------------------------
    def generate(self, prompts, max_tokens: int = 128, temperature: float = 0.0, top_k: int = 0,
                 seed: int | None = None, max_steps: int | None = None) -> list:
        """Generate for every prompt (text, or lists of token ids) and return the outputs in the order given.
        Steps inline until all have ended; prompts beyond the waiting bound are submitted as room appears.
        ``seed``: prompt i draws with ``seed + i``."""
        if isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int)):
            prompts = [prompts]
        requests: list = []
        steps = 0
        while True:
            while len(requests) < len(prompts) and len(self.waiting) < self.config.max_waiting:
                i = len(requests)
                requests.append(self.submit(prompts[i], max_tokens=max_tokens, temperature=temperature, top_k=top_k,
                                            seed=None if seed is None else seed + i))
            alive = [r for r in requests if r.state not in TERMINAL]
            if not alive and len(requests) == len(prompts):
                break
            moved = self.step()
            steps += 1
            if self.fault:
                raise RuntimeError(f"engine fault: {self.fault}")
            if not moved and len(requests) == len(prompts) and any(r.state not in TERMINAL for r in requests):
                raise RuntimeError("the engine made no progress: the page pool cannot hold any waiting request")
            if max_steps is not None and steps >= max_steps:
                break
        self.drain()
        return [GenerationOutput(r.request_id, r.prompt_ids, list(r.generated_ids), r.text, r.finish_reason)
                for r in requests]

    def start(self) -> None:
        """Serve from a thread of its own: ``submit`` from any thread, read ``Request.events``."""
        if self._thread is not None and self._thread.is_alive():
            return
        self._closing.clear()

        def serve():
            while not (self._closing.is_set() or self.fault):
                if not self.step():
                    time.sleep(self.config.idle_sleep_seconds)

        self._thread = threading.Thread(target=serve, name="flexengine-steps", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        """Stop serving; whatever has not ended is cancelled and gives its pages back."""
        self._closing.set()
        if self._thread is not None:
            self._thread.join(timeout=20)
        with self.lock:
            self._land()
            for request in list(self.all_requests.values()):
                self._retire(request, State.CANCELLED, "cancelled")
        self.trace.close()


def pages_that_fit(plan, config: EngineConfig, dtype) -> int:
    """Pages per paged cache group that fill ``kv_memory_fraction`` of the device memory that is free now."""
    if not str(config.device).startswith("cuda"):
        raise ValueError("kv_num_blocks=0 (size the pool from free memory) needs a CUDA device")
    free, _total = torch.cuda.mem_get_info(torch.device(config.device))
    width = torch.empty((), dtype=dtype).element_size()
    page_bytes = sum(2 * g.slots * g.kv_heads * g.head_dim * (g.page_size or config.kv_block_size) * width
                     for g in plan.cache_groups if g.kind != "state")
    pages = int(free * config.kv_memory_fraction) // max(page_bytes, 1)
    smallest = min((g.page_size or config.kv_block_size for g in plan.cache_groups if g.kind != "state"),
                   default=config.kv_block_size)
    need = math.ceil(config.max_model_len / smallest)
    if pages < need:
        raise ValueError(f"free device memory holds {pages} pages; one request of max_model_len needs {need}")
    return pages
