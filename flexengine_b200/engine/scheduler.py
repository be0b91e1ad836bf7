"""Token-budget scheduling: which requests run in a step and with how many tokens.

Decisions follow the reference's planner (src/flexengine/engine/scheduler/policies.py:31-78):
requests are ordered by policy, then the step's token budget is filled greedily, a prefill
portion taking ``min(budget, remaining context)`` tokens (``adaptive`` caps it at
``prefill_chunk_size``) and a decode one token.  ``fcfs`` orders by arrival; ``decode_first``
and ``adaptive`` serve overdue prefills, then decodes, then prefills; ``slo_aware`` orders by
slack to the time-to-first-token or inter-token deadline.
A chunk also says whether its last row's logits are wanted: only when it completes the
request's context and the request is not replaying after a preemption.
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


class Scheduler:
    def __init__(self, policy: str, token_budget: int, ttft_ms: float, itl_ms: float, prefill_chunk_size: int = 128):
        if policy not in ("fcfs", "decode_first", "slo_aware", "adaptive"):
            raise ValueError("Unknown policy")
        self.policy = policy
        self.token_budget = int(token_budget)
        self.ttft_ms = float(ttft_ms)
        self.itl_ms = float(itl_ms)
        self.prefill_chunk_size = int(prefill_chunk_size)

    def ordered(self, requests: list) -> list:
        now = monotonic()
        if self.policy == "fcfs":
            return sorted(requests, key=lambda r: (r.arrived, -r.priority))
        if self.policy in ("decode_first", "adaptive"):
            def rank(r: Request):
                overdue = r.in_prefill and not r.generated_ids and (now - r.arrived) * 1000.0 >= self.ttft_ms
                return (not overdue, r.in_prefill, -r.priority, r.arrived)
            return sorted(requests, key=rank)

        def slack(r: Request):
            if not r.generated_ids:
                deadline = r.arrived + self.ttft_ms / 1000.0
            else:
                deadline = (r.last_token_at or r.arrived) + self.itl_ms / 1000.0
            age_bonus = min(now - r.arrived, 10.0) * 0.01
            return (deadline - now) - r.priority * 0.01 - age_bonus
        return sorted(requests, key=lambda r: (slack(r), r.arrived))

    def plan(self, requests: list) -> list:
        budget = self.token_budget
        adaptive = self.policy == "adaptive"
        chunks = []
        for req in self.ordered(requests):
            if budget <= 0:
                break
            # the request's properties, spelled out: this loop runs for every running request at every step
            generated = req.generated_ids
            produced = len(generated)
            if produced and generated[-1] == PENDING and produced >= req.max_tokens:
                continue                                  # its last token is on its way
            cached = req.cached_tokens
            context = len(req.prompt_ids) + (produced - 1 if produced else 0)
            if cached < context:                          # still in its prompt (or recomputing)
                length = min(budget, context - cached)
                if adaptive:
                    length = min(length, self.prefill_chunk_size)
                tokens = req.next_inputs(length)
            elif produced:
                tokens = [generated[-1]]
            else:
                continue
            if not tokens:
                continue
            completes = cached + len(tokens) >= context
            chunks.append(Chunk(req.request_id, tokens, cached, completes and not req.replaying))
            budget -= len(tokens)
        assert sum(len(c.input_ids) for c in chunks) <= self.token_budget
        return chunks
