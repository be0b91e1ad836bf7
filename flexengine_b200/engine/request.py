"""One request: what it asked for, where it stands, and the clock marks its report is made from.

The states and their names are the reference's (src/flexengine/engine/scheduler/state.py:11-26), and so is
the rule that the cache trails the emitted tokens by one: the context a request has to have run through the
model is its prompt plus every generated token but the last (state.py:71-99).  Here that context is never
built as a list: ``context_slice`` reads across the seam between prompt and generated tokens.  ``replaying``
marks a preempted request that recomputes a context it has already sampled from
(src/flexengine/engine/runtime.py:242-251,318-324).  ``PENDING`` stands in ``generated_ids`` for a token that
the device has sampled and the host has not read yet (this engine launches a step before reading the last).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum
from queue import SimpleQueue


class State(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    FAILED = "failed"


TERMINAL = frozenset({State.FINISHED, State.CANCELLED, State.FAILED})
_LIVE = (State.WAITING, State.RUNNING, State.PREEMPTED)
# a request only ever moves along these edges: into a seat, out of it when pages run short and back in, from a seat
# to its regular end, and from anywhere alive to cancellation or failure
_EDGES = frozenset({(State.WAITING, State.RUNNING), (State.RUNNING, State.PREEMPTED), (State.PREEMPTED, State.RUNNING),
                    (State.RUNNING, State.FINISHED)}
                   | {(alive, end) for alive in _LIVE for end in (State.CANCELLED, State.FAILED)})

PENDING = -1


@dataclass
class Event:
    """What a consumer of ``Request.events`` receives: ``kind`` is "token", "done" or "error"."""
    kind: str
    text: str = ""
    token_id: int | None = None
    finish_reason: str | None = None
    error: str | None = None
    timestamp: float = field(default_factory=time.monotonic)


def _ms(later, earlier):
    return None if later is None or earlier is None else (later - earlier) * 1000.0


@dataclass(eq=False)            # a request is itself, not its fields: compared and hashed by identity
class Request:
    request_id: str
    prompt_ids: list
    max_tokens: int
    temperature: float = 0.0
    top_k: int = 0
    priority: int = 0
    seed: int = 0
    created: int = field(default_factory=lambda: int(time.time()))
    arrived: float = field(default_factory=time.monotonic)
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

    # ---- where it stands ---------------------------------------------------------------------------------
    def transition(self, target: State) -> None:
        if target is self.state:
            return
        if (self.state, target) not in _EDGES:
            raise ValueError(f"a {self.state.value} request cannot become {target.value}")
        self.state = target

    @property
    def context_length(self) -> int:
        """Tokens that must be in the cache before the next token can be sampled."""
        return len(self.prompt_ids) + max(0, len(self.generated_ids) - 1)

    @property
    def in_prefill(self) -> bool:
        return self.cached_tokens < self.context_length

    @property
    def awaits_last_token(self) -> bool:
        """The token on its way is the last one ``max_tokens`` allows: nothing more is to be run."""
        g = self.generated_ids
        return bool(g) and g[-1] == PENDING and len(g) >= self.max_tokens

    def context_slice(self, start: int, count: int) -> list:
        """Tokens ``start .. start+count-1`` of the context (prompt, then generated tokens but the last),
        cut at its end."""
        stop = min(start + count, self.context_length)
        if stop <= start:
            return []
        seam = len(self.prompt_ids)
        if stop <= seam:
            return self.prompt_ids[start:stop]
        if start >= seam:
            return self.generated_ids[start - seam:stop - seam]
        return self.prompt_ids[start:] + self.generated_ids[:stop - seam]

    # ---- what is written about it when it ends -----------------------------------------------------------------
    def report(self) -> dict:
        """The request's line of ``requests.jsonl``.  Keys are the reference's trace schema, which its
        analysis reads (state.py:101-123): latencies in milliseconds from the monotonic clock marks."""
        stamps = self.token_times
        gaps = [(b - a) * 1000.0 for a, b in zip(stamps, stamps[1:])]
        per_token = (stamps[-1] - stamps[0]) * 1000.0 / (len(stamps) - 1) if len(stamps) > 1 else None
        ended = self.finished_at if self.finished_at is not None else time.monotonic()
        out = {"request_id": self.request_id, "state": self.state.value,
               "prompt_tokens": len(self.prompt_ids), "output_tokens": len(self.generated_ids)}
        out.update(ttft_ms=_ms(self.first_token_at, self.arrived), itl_ms=gaps, tpot_ms=per_token,
                   e2e_ms=_ms(ended, self.arrived), queue_ms=_ms(self.first_scheduled_at, self.arrived),
                   finish_reason=self.finish_reason, error=self.error, preemptions=self.preemptions)
        return out
