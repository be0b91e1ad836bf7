"""The engine: queues, admission, one scheduling iteration per ``step()``, sampling,
finishing and freeing, and the Python entry point ``generate()``.

Semantics follow the reference's runtime (src/flexengine/engine/runtime.py): ``submit``
validates and enqueues (runtime.py:89-121); ``step`` admits while fewer than
``max_num_seqs`` run (runtime.py:162-179), plans under the token budget (runtime.py:262),
reserves pages chunk by chunk and, when pages run out, preempts ONE running request that
is not planned in this step (lowest priority, then most cached tokens), retries once and
otherwise leaves the chunk out of the step (runtime.py:273-288); a preempted request gives
its pages back, goes to the back of the waiting queue and later recomputes its context
without sampling a second time from it (runtime.py:242-251,318-324); a token in the end-of-
sequence set finishes with "stop", reaching ``max_tokens`` with "length" (runtime.py:343-346);
an exception in the executor faults the engine and fails every live request
(runtime.py:349-356).  Logits are asked for only where a token will be sampled.

Unlike the reference, a step is launched before the host has read the tokens of the step before
(``overlap_steps``): sampled tokens stay on the device, the next step takes them from there
(``StepEntry.carry``), and the host reads them one step late, while the device is busy.  A request's
``generated_ids`` holds ``PENDING`` in the place of a token that is on its way.  A request that turns
out to have ended with an end-of-sequence token has then been run one token too far; that token is
dropped.  Before anyone is preempted the tokens on their way are read, so that preemption and
recomputation see exact state.
"""
from __future__ import annotations

import threading
import time
import uuid
from collections import OrderedDict, deque
from dataclasses import dataclass

import torch

from ..cache.manager import CacheManager
from ..cache.page_pool import CacheExhausted
from ..config.engine_config import EngineConfig
from ..observability.traces import TraceWriter, nvtx
from ..sampling.sampler import Sampler
from .request import PENDING, TERMINAL, Event, Request, State
from .scheduler import Scheduler
from .step import ModelRunner, StepEntry


class BusyError(RuntimeError):
    pass


@dataclass
class GenerationOutput:
    request_id: str
    prompt_ids: list
    token_ids: list
    text: str
    finish_reason: str | None


@dataclass
class _InFlight:
    """The step whose sampled tokens the host has not read yet."""
    sampled: list                        # [(request, its place in generated_ids)] in the order of ``tokens``
    tokens: torch.Tensor                 # int32 [len(sampled)], where the logits were
    host: torch.Tensor | None = None     # pinned copy, complete once ``event`` has passed
    event: object = None
    index: dict | None = None            # request id -> place in ``tokens``


class Engine:
    def __init__(self, config: EngineConfig, runner: ModelRunner, sampler: Sampler | None = None, tokenizer=None,
                 eos_token_ids=()):
        self.config = config
        self.runner = runner
        self.cache: CacheManager = runner.cache
        self.sampler = sampler if sampler is not None else Sampler(runner.ops)
        self.tokenizer = tokenizer
        self.eos_ids = set(eos_token_ids)
        self.scheduler = Scheduler(config.scheduler_policy, config.max_num_batched_tokens, config.ttft_slo_ms,
                                   config.itl_slo_ms, config.prefill_chunk_size)
        if self.cache.capacity_tokens() < config.max_model_len:
            raise ValueError("KV pool cannot contain one max-length request")
        self.waiting: deque = deque()
        self.running: OrderedDict = OrderedDict()
        self.all_requests: dict = {}
        self.lock = threading.RLock()
        self.shutdown = threading.Event()
        self.worker: threading.Thread | None = None
        self.fault: str | None = None
        self.step_index = 0
        self.request_sequence = 0
        self.completed_count = 0
        self.preemption_count = 0
        self.output_tokens = 0
        self._in_flight: _InFlight | None = None
        self._pinned: list = []
        self._pinned_at = 0
        self.trace = TraceWriter(config.trace_dir)
        self.trace.metadata(config)

    # ---- construction from a model folder ----------------------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, config: EngineConfig | None = None, tokenizer=None, ops=None) -> "Engine":
        from ..weights.loader import load_model
        config = config or EngineConfig(model=model_dir)
        _typed, plan, model = load_model(model_dir, config.dtype, config.device)
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
            runner.capture_decode_graphs()         # at start-up, not in the path of the first requests
        return cls(config, runner, tokenizer=tokenizer, eos_token_ids=plan.eos_token_ids)

    # ---- worker thread (a server would use it; generate() steps inline) --------------------------
    def start(self) -> None:
        if self.worker and self.worker.is_alive():
            return
        self.shutdown.clear()
        self.worker = threading.Thread(target=self._worker, name="flexengine-cuda-worker", daemon=True)
        self.worker.start()

    def stop(self) -> None:
        self.shutdown.set()
        if self.worker:
            self.worker.join(timeout=20)
        with self.lock:
            self._collect()
            for req in list(self.all_requests.values()):
                if req.state not in TERMINAL:
                    self._finish(req, State.CANCELLED, "cancelled")

    def _worker(self) -> None:
        while not self.shutdown.is_set() and not self.fault:
            if not self.step():
                time.sleep(self.config.idle_sleep_seconds)

    # ---- requests ------------------------------------------------------------------------------
    def submit(self, prompt, max_tokens: int = 128, temperature: float = 0.0, top_k: int = 0, priority: int = 0,
               seed: int | None = None) -> Request:
        """``prompt``: a string (needs a tokenizer) or a list of token ids."""
        if isinstance(prompt, str):
            if not prompt:
                raise ValueError("prompt must be a non-empty string")
            if self.tokenizer is None:
                raise ValueError("a string prompt needs a tokenizer; pass token ids instead")
            ids = list(self.tokenizer.encode(prompt, add_special_tokens=False))
            if not ids:
                bos = getattr(self.tokenizer, "bos_token_id", None)
                if bos is None:
                    raise ValueError("empty encoded prompt")
                ids = [bos]
        else:
            ids = [int(t) for t in prompt]
            if not ids:
                raise ValueError("prompt must hold at least one token id")
            if min(ids) < 0 or max(ids) >= self.runner.vocab_size:
                raise ValueError(f"token id outside [0, {self.runner.vocab_size})")
        if not (1 <= max_tokens <= self.config.max_output_tokens):
            raise ValueError(f"max_tokens must be between 1 and {self.config.max_output_tokens}")
        if not (0.0 <= temperature <= 5.0) or top_k < 0:
            raise ValueError("invalid sampling parameters")
        if len(ids) + max_tokens > self.config.max_model_len:
            raise ValueError(f"prompt tokens ({len(ids)}) + max_tokens ({max_tokens}) exceeds max_model_len "
                             f"({self.config.max_model_len})")
        with self.lock:
            if self.shutdown.is_set() or self.fault:
                raise BusyError("engine is not accepting requests")
            if len(self.waiting) >= self.config.max_waiting:
                raise BusyError("bounded waiting queue is full")
            req = Request("cmpl-" + uuid.uuid4().hex, ids, max_tokens, float(temperature), int(top_k), int(priority))
            # the same requests in the same order give the same tokens under every policy
            req.seed = int(seed) if seed is not None else self.config.random_seed + self.request_sequence
            self.request_sequence += 1
            self.waiting.append(req)
            self.all_requests[req.request_id] = req
            return req

    def cancel(self, request_id: str) -> bool:
        with self.lock:
            req = self.all_requests.get(request_id)
            if req is None or req.state in TERMINAL:
                return False
            self._finish(req, State.CANCELLED, "cancelled")
            return True

    def _finish(self, req: Request, state: State, reason: str, error: str | None = None) -> None:
        if req.state in TERMINAL:
            return
        req.transition(state)
        while req.generated_ids and req.generated_ids[-1] == PENDING:      # run one token too far: dropped
            req.generated_ids.pop()
        req.finished_at = time.monotonic()
        req.finish_reason = reason
        req.error = error
        self.cache.free(req.request_id)
        self.running.pop(req.request_id, None)
        if any(r.request_id == req.request_id for r in self.waiting):
            self.waiting = deque(r for r in self.waiting if r.request_id != req.request_id)
        if state is State.FAILED:
            req.events.put(Event("error", error=error or reason, finish_reason=reason))
        else:
            remaining = req.text[len(req.emitted_text):] if req.text.startswith(req.emitted_text) else ""
            if remaining:
                req.emitted_text += remaining
                req.events.put(Event("token", text=remaining))
            req.events.put(Event("done", finish_reason=reason))
        self.trace.write("requests", req.snapshot())
        self.all_requests.pop(req.request_id, None)
        self.completed_count += 1

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.config.max_num_seqs:
            req = self.waiting.popleft()
            if req.state in TERMINAL:
                continue
            self.cache.admit(req.request_id)          # state slot; no page is taken at admission
            req.transition(State.RUNNING)
            self.running[req.request_id] = req

    def _preempt(self, victim: Request) -> None:
        self._collect()                          # nobody is preempted with a token on its way
        if victim.state in TERMINAL:
            return
        self.cache.free(victim.request_id)
        victim.cached_tokens = 0
        victim.replaying = bool(victim.generated_ids)
        victim.preemptions += 1
        victim.transition(State.PREEMPTED)
        self.running.pop(victim.request_id, None)
        self.waiting.append(victim)
        self.preemption_count += 1

    def _reserve_or_preempt(self, proposed: list) -> list:
        planned = []
        for chunk in proposed:
            req = self.running.get(chunk.request_id)
            if req is None:
                continue
            target = chunk.start + len(chunk.input_ids)
            try:
                self.cache.reserve(req.request_id, target)
            except CacheExhausted:
                if self._in_flight is not None:
                    # exact state first: requests that have just ended give their pages back, and nobody is
                    # preempted with a token on its way
                    self._collect()
                    if req.request_id not in self.running:
                        continue
                    try:
                        self.cache.reserve(req.request_id, target)
                        planned.append(chunk)
                        continue
                    except CacheExhausted:
                        pass
                selected = {c.request_id for c in planned}
                victims = [v for v in self.running.values()
                           if v.request_id != req.request_id and v.request_id not in selected
                           and self.cache.holds_pages(v.request_id)]
                if not victims:
                    continue
                self._preempt(min(victims, key=lambda r: (r.priority, -r.cached_tokens)))
                try:
                    self.cache.reserve(req.request_id, target)
                except CacheExhausted:
                    continue
            planned.append(chunk)
        return planned

    # ---- one scheduling iteration -----------------------------------------------------------------
    def step(self) -> bool:
        with self.lock:
            if self.fault:
                return False
            t0 = time.perf_counter()
            self._admit()
            with nvtx("sched/select"):
                proposed = self.scheduler.plan(list(self.running.values()))
            with nvtx("kv/reserve"):
                planned = self._reserve_or_preempt(proposed)
                planned = [c for c in planned if c.request_id in self.running]     # reading tokens may have ended some
            if not planned:
                if self._in_flight is not None:
                    self._collect()          # nothing more to launch: the tokens on their way are the progress
                    return True
                return False
            scheduler_ms = (time.perf_counter() - t0) * 1000.0
            new_tokens = sum(len(c.input_ids) for c in planned)
            prefill_tokens = sum(len(c.input_ids) for c in planned if self.running[c.request_id].in_prefill)
            t1 = time.perf_counter()
            try:
                with nvtx(f"executor/step batch={len(planned)} tokens={new_tokens}"):
                    launched = self._launch(planned)
                previous, self._in_flight = self._in_flight, launched
                self._read_tokens(previous)              # of the step before, while the device runs this one
                if not self.config.overlap_steps:
                    self._collect()
            except Exception as ex:  # noqa: BLE001 - any executor failure faults the engine
                self.fault = f"{type(ex).__name__}: {ex}"
                self._in_flight = None
                for req in list(self.all_requests.values()):
                    if req.state not in TERMINAL:
                        self._finish(req, State.FAILED, "error", self.fault)
                return False
            executor_ms = (time.perf_counter() - t1) * 1000.0
            self.step_index += 1
            if self.config.trace_steps and self.trace.directory:
                self.trace.write("steps", {
                    "step": self.step_index, "batch_size": len(planned), "new_tokens": new_tokens,
                    "prefill_tokens": prefill_tokens, "decode_tokens": new_tokens - prefill_tokens,
                    "kv_used_blocks": self.cache.used_pages, "waiting": len(self.waiting),
                    "running": len(self.running), "wall_ms": (time.perf_counter() - t0) * 1000.0,
                    "scheduler_ms": scheduler_ms, "executor_wall_ms": executor_ms,
                    "policy": self.config.scheduler_policy, "preemptions": self.preemption_count,
                })
            return True

    def _launch(self, planned: list) -> _InFlight:
        """Run the planned chunks and sample; nothing here waits for the device."""
        before = self._in_flight
        entries, sampled = [], []
        for c in planned:
            req = self.running[c.request_id]
            ids, carry = c.input_ids, None
            if ids[-1] == PENDING:                       # a decode step planned on a token that was on its way
                last = req.generated_ids[-1]
                if last == PENDING:
                    ids, carry = [0], before.index[c.request_id]
                else:
                    ids = [last]                         # it has been read since
            entries.append(StepEntry(c.request_id, ids, [len(ids) - 1] if c.wants_logits else [], carry))
            if c.wants_logits:
                sampled.append(req)
        logits = self.runner.step(entries, before.tokens if before is not None else None)
        tokens = None
        if sampled:
            tokens = self.sampler.sample_on_device(logits, [r.temperature for r in sampled], [r.top_k for r in sampled],
                                                   [r.seed for r in sampled], [len(r.generated_ids) for r in sampled])
        now = time.monotonic()
        places = []
        for chunk in planned:
            req = self.running[chunk.request_id]
            if req.first_scheduled_at is None:
                req.first_scheduled_at = now
            req.cached_tokens += len(chunk.input_ids)
            if req.in_prefill:
                continue
            if req.replaying:
                # the recomputed context already gave its token before the preemption
                req.replaying = False
                continue
            req.generated_ids.append(PENDING)
            places.append((req, len(req.generated_ids) - 1))
            if len(req.generated_ids) >= req.max_tokens:
                # the token on its way is its last whatever it is: its seat and its pages serve others from the next
                # step on (what that step writes there comes after this one on the stream); the request itself ends
                # when the token has been read
                self.cache.free(req.request_id)
                self.running.pop(req.request_id, None)
        assert [r.request_id for r, _ in places] == [r.request_id for r in sampled]
        record = _InFlight(places, tokens, index={r.request_id: i for i, (r, _) in enumerate(places)})
        if tokens is not None and tokens.device.type == "cuda":
            # one of a few pinned buffers kept for good (two records are alive at most): allocating pinned memory
            # at every step costs a call into the driver now and then
            if not self._pinned or self._pinned[0].numel() < tokens.numel():
                self._pinned = [torch.empty(max(tokens.numel(), self.config.max_num_seqs), dtype=tokens.dtype, pin_memory=True)
                                for _ in range(4)]
            self._pinned_at = (self._pinned_at + 1) % len(self._pinned)
            record.host = self._pinned[self._pinned_at][:tokens.numel()]
            record.host.copy_(tokens, non_blocking=True)
            record.event = torch.cuda.Event()
            record.event.record()
        return record

    def drain(self) -> None:
        """Wait for the step that was launched last and take its tokens in: afterwards no request
        holds a token that the host has not read."""
        with self.lock:
            self._collect()

    def _collect(self) -> None:
        """Read the tokens that are on their way, if any."""
        record, self._in_flight = self._in_flight, None
        self._read_tokens(record)

    def _read_tokens(self, record: _InFlight | None) -> None:
        if record is None or not record.sampled:
            return
        if record.event is not None:
            record.event.synchronize()
            values = record.host.tolist()
        else:
            values = record.tokens.tolist()
        now = time.monotonic()
        for (req, place), token in zip(record.sampled, values):
            if req.state in TERMINAL:
                continue                                  # ended or cancelled meanwhile: one token too far
            self._accept_token(req, place, int(token), now)

    def _accept_token(self, req: Request, place: int, token: int, now: float) -> None:
        req.generated_ids[place] = token
        known = place + 1                                 # a later place may hold the next token on its way
        if req.first_token_at is None:
            req.first_token_at = now
        req.last_token_at = now
        req.token_times.append(now)
        self.output_tokens += 1
        if self.tokenizer is not None:
            req.text = self.tokenizer.decode(req.generated_ids[:known], skip_special_tokens=True,
                                             clean_up_tokenization_spaces=False)
            # a trailing replacement character may still be completed by the next tokens
            stable = req.text.rstrip("\ufffd")
            delta = stable[len(req.emitted_text):] if stable.startswith(req.emitted_text) else ""
            if delta:
                req.emitted_text += delta
                req.events.put(Event("token", text=delta, token_id=token))
        else:
            req.events.put(Event("token", token_id=token))
        if token in self.eos_ids:
            self._finish(req, State.FINISHED, "stop")
        elif known >= req.max_tokens:
            self._finish(req, State.FINISHED, "length")

    # ---- the Python entry point ----------------------------------------------------------------------
    def generate(self, prompts, max_tokens: int = 128, temperature: float = 0.0, top_k: int = 0,
                 seed: int | None = None, max_steps: int | None = None) -> list:
        """Generate for every prompt (strings or lists of token ids) and return the outputs in
        order.  Runs ``step()`` inline until all are done; prompts beyond the waiting bound are
        submitted as room appears."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        pending = deque(enumerate(prompts))
        requests: dict = {}
        steps = 0
        while pending or any(r.state not in TERMINAL for r in requests.values()):
            while pending and len(self.waiting) < self.config.max_waiting:
                i, p = pending.popleft()
                s = None if seed is None else seed + i
                requests[i] = self.submit(p, max_tokens=max_tokens, temperature=temperature, top_k=top_k, seed=s)
            progressed = self.step()
            steps += 1
            if self.fault:
                raise RuntimeError(f"engine fault: {self.fault}")
            if not progressed and not pending and any(r.state not in TERMINAL for r in requests.values()):
                raise RuntimeError("the engine made no progress: the page pool cannot hold any waiting request")
            if max_steps is not None and steps >= max_steps:
                break
        self.drain()
        return [GenerationOutput(r.request_id, r.prompt_ids, list(r.generated_ids), r.text, r.finish_reason)
                for r in (requests[i] for i in sorted(requests))]

    def snapshot(self) -> dict:
        with self.lock:
            return {"waiting": len(self.waiting), "running": len(self.running),
                    "cache_used_blocks": self.cache.used_pages, "cache_free_blocks": self.cache.free_pages,
                    "steps": self.step_index, "fault": self.fault, "requests_total": self.request_sequence,
                    "requests_completed": self.completed_count, "preemptions": self.preemption_count,
                    "output_tokens": self.output_tokens}


def pages_that_fit(plan, config: EngineConfig, dtype) -> int:
    """Pages per paged group that fill ``kv_memory_fraction`` of the device memory now free."""
    if not str(config.device).startswith("cuda"):
        raise ValueError("kv_num_blocks=0 (size from free memory) needs a CUDA device")
    free, _total = torch.cuda.mem_get_info(torch.device(config.device))
    itemsize = torch.empty((), dtype=dtype).element_size()
    per_page = sum(2 * g.slots * g.kv_heads * g.head_dim * config.kv_block_size * itemsize
                   for g in plan.cache_groups if g.kind != "state")
    pages = int(free * config.kv_memory_fraction) // max(per_page, 1)
    need = -(-config.max_model_len // config.kv_block_size)
    if pages < need:
        raise ValueError(f"free device memory holds {pages} pages; one request of max_model_len needs {need}")
    return pages
