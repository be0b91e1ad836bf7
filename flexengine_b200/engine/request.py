"""A request's life cycle and generation state.

States and legal transitions, ``full_context`` (prompt plus all generated tokens but the
last, which is not yet in the cache), ``in_prefill`` and ``next_inputs`` follow the reference
(src/flexengine/engine/scheduler/state.py:11-26,71-99).  ``replaying`` (set when a
preempted request that already produced tokens is recomputed, so that the logits at the
end of the recomputed context are not sampled again; src/flexengine/engine/runtime.py:242-251,
318-324) is a declared field here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from queue import SimpleQueue
from time import monotonic, time


class State(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    FAILED = "failed"


TERMINAL = {State.FINISHED, State.CANCELLED, State.FAILED}
VALID_TRANSITIONS = {
    State.WAITING: {State.RUNNING, State.CANCELLED, State.FAILED},
    State.RUNNING: {State.PREEMPTED, State.FINISHED, State.CANCELLED, State.FAILED},
    State.PREEMPTED: {State.RUNNING, State.CANCELLED, State.FAILED},
    State.FINISHED: set(), State.CANCELLED: set(), State.FAILED: set(),
}


@dataclass
class Event:
    kind: str                      # "token", "done", "error"
    text: str = ""
    token_id: int | None = None
    finish_reason: str | None = None
    error: str | None = None
    timestamp: float = field(default_factory=monotonic)


PENDING = -1      # in ``generated_ids``: a token that was sampled on the device and that the host has not read yet


@dataclass
class Request:
    request_id: str
    prompt_ids: list
    max_tokens: int
    temperature: float = 0.0
    top_k: int = 0
    priority: int = 0
    seed: int = 0
    created: int = field(default_factory=lambda: int(time()))
    arrived: float = field(default_factory=monotonic)
    state: State = State.WAITING
    cached_tokens: int = 0         # tokens run through the model and held in the cache
    generated_ids: list = field(default_factory=list)
    replaying: bool = False
    text: str = ""
    emitted_text: str = ""
    preemptions: int = 0
    first_token_at: float | None = None
    last_token_at: float | None = None
    finished_at: float | None = None
    first_scheduled_at: float | None = None
    token_times: list = field(default_factory=list)
    error: str | None = None
    finish_reason: str | None = None
    events: SimpleQueue = field(default_factory=SimpleQueue, repr=False)

    def transition(self, new_state: State) -> None:
        if new_state == self.state:
            return
        if new_state not in VALID_TRANSITIONS[self.state]:
            raise ValueError(f"Invalid transition {self.state} -> {new_state}")
        self.state = new_state

    @property
    def full_context(self) -> list:
        return self.prompt_ids + self.generated_ids[:-1] if self.generated_ids else self.prompt_ids

    @property
    def context_length(self) -> int:
        n = len(self.generated_ids)
        return len(self.prompt_ids) + (n - 1 if n else 0)

    @property
    def in_prefill(self) -> bool:
        return self.cached_tokens < self.context_length

    @property
    def awaits_last_token(self) -> bool:
        """The token on its way is the last one ``max_tokens`` allows: nothing more is to be run."""
        return bool(self.generated_ids) and self.generated_ids[-1] == PENDING and len(self.generated_ids) >= self.max_tokens

    def next_inputs(self, count: int) -> list:
        if count <= 0:
            return []
        if self.in_prefill:
            return self.full_context[self.cached_tokens:self.cached_tokens + count]
        if not self.generated_ids:
            return []
        return [self.generated_ids[-1]]

    def snapshot(self) -> dict:
        ttft = None if self.first_token_at is None else (self.first_token_at - self.arrived) * 1000.0
        end = self.finished_at if self.finished_at is not None else monotonic()
        itls = [(b - a) * 1000.0 for a, b in zip(self.token_times, self.token_times[1:])]
        return {
            "request_id": self.request_id, "state": self.state.value,
            "prompt_tokens": len(self.prompt_ids), "output_tokens": len(self.generated_ids),
            "ttft_ms": ttft, "itl_ms": itls,
            "tpot_ms": ((self.token_times[-1] - self.token_times[0]) * 1000.0 / (len(self.token_times) - 1))
            if len(self.token_times) >= 2 else None,
            "e2e_ms": (end - self.arrived) * 1000.0,
            "queue_ms": None if self.first_scheduled_at is None
            else (self.first_scheduled_at - self.arrived) * 1000.0,
            "finish_reason": self.finish_reason, "error": self.error, "preemptions": self.preemptions,
        }
