"""Token-budget scheduling: which requests run in a step and with how many tokens.

The decisions are the reference's (src/flexengine/engine/scheduler/policies.py:31-78): requests are put in an
order that depends on the policy, then the step's token budget is dealt out along that order, a request still in
its prompt taking ``min(what is left of the budget, what is left of its context)`` tokens (``adaptive`` caps that at
``prefill_chunk_size``) and a decoding request one token.  Here each policy is one key function in a table, and a
portion may have to be a multiple of ``granularity`` tokens (a mixer whose state advances in blocks asks for that
through its cache group); the last portion of a context is exempt, since it ends where the context ends.

A chunk also says whether its last row's logits are wanted: only when it completes the request's context and
the request is not recomputing after a preemption.
"""
from __future__ import annotations

from dataclasses import dataclass
from time import monotonic

from .request import PENDING, Request


@dataclass
class Chunk:
    request_id: str
    input_ids: list
    start: int
    wants_logits: bool = True


# ---- orders ---------------------------------------------------------------------------------------------------
def _by_arrival(r: Request, now: float, sched: "Scheduler"):
    return (r.arrived, -r.priority)


def _decodes_before_prompts(r: Request, now: float, sched: "Scheduler"):
    """A prompt that has waited past the time-to-first-token target goes first of all; then requests that decode,
    then prompts; inside a class higher priority, then earlier arrival."""
    if not r.in_prefill:
        rank = 1
    elif not r.generated_ids and (now - r.arrived) * 1e3 >= sched.ttft_ms:
        rank = 0
    else:
        rank = 2
    return (rank, -r.priority, r.arrived)


PRIORITY_WORTH_MS = 10.0        # one priority level is worth this much slack
WAIT_WORTH = 0.01               # a millisecond of waiting is worth this many milliseconds of slack ...
WAIT_WORTH_UP_TO_MS = 10000.0   # ... for the first ten seconds


def _least_slack(r: Request, now: float, sched: "Scheduler"):
    """Milliseconds left until the request misses its target (first token: ``ttft_ms`` after arrival; later
    tokens: ``itl_ms`` after the last one), less what its priority and its age are worth."""
    if r.generated_ids:
        due = (r.last_token_at or r.arrived) + sched.itl_ms / 1e3
    else:
        due = r.arrived + sched.ttft_ms / 1e3
    waited_ms = (now - r.arrived) * 1e3
    slack_ms = (due - now) * 1e3 - PRIORITY_WORTH_MS * r.priority - WAIT_WORTH * min(waited_ms, WAIT_WORTH_UP_TO_MS)
    return (slack_ms, r.arrived)


ORDERS = {"fcfs": _by_arrival, "decode_first": _decodes_before_prompts, "adaptive": _decodes_before_prompts,
          "slo_aware": _least_slack}


class Scheduler:
    def __init__(self, policy: str, token_budget: int, ttft_ms: float, itl_ms: float, prefill_chunk_size: int = 128,
                 granularity: int = 1):
        if policy not in ORDERS:
            raise ValueError(f"Unknown policy {policy!r}; known: {sorted(ORDERS)}")
        self.policy = policy
        self.token_budget = int(token_budget)
        self.ttft_ms = float(ttft_ms)
        self.itl_ms = float(itl_ms)
        self.prefill_chunk_size = int(prefill_chunk_size)
        self.granularity = max(1, int(granularity))
        if self.token_budget < self.granularity:
            raise ValueError(f"a token budget of {token_budget} cannot hold one portion of {granularity} tokens")
        self.portion_cap = self.prefill_chunk_size if policy == "adaptive" else None

    def ordered(self, requests: list) -> list:
        now, key = monotonic(), ORDERS[self.policy]
        return sorted(requests, key=lambda r: key(r, now, self))

    def portion_length(self, budget: int, left: int) -> int:
        """How many tokens of a context with ``left`` tokens to go run now under ``budget``."""
        length = min(budget, left)
        if self.portion_cap is not None:
            length = min(length, self.portion_cap)
        if length < left:                                  # not the context's last portion: whole blocks only
            length -= length % self.granularity
        return length

    def plan(self, requests: list) -> list:
        budget = self.token_budget
        chunks = []
        for req in self.ordered(requests):
            if budget <= 0:
                break
            generated = req.generated_ids
            produced = len(generated)
            if produced and generated[-1] == PENDING and produced >= req.max_tokens:
                continue                                   # its last token is on its way
            cached = req.cached_tokens
            context = len(req.prompt_ids) + (produced - 1 if produced else 0)
            if cached < context:                           # still in its prompt, or recomputing
                tokens = req.context_slice(cached, self.portion_length(budget, context - cached))
            elif produced:
                tokens = [generated[-1]]                   # PENDING when the device still holds it
            else:
                continue
            if not tokens:
                continue
            completes = cached + len(tokens) >= context
            chunks.append(Chunk(req.request_id, tokens, cached, completes and not req.replaying))
            budget -= len(tokens)
        return chunks
