"""The step function: one batch of (request, its next tokens) through the model.

A batch holds portions of prompts beside single decoded tokens, cut anywhere; only the
given tokens run, against what earlier steps left in the cache, and logits come back
for the wanted places only.  The reference's counterpart is ``Qwen2Adapter.forward``
(src/flexengine/inference/models/qwen2.py:79-136): it flattens ids and positions
(qwen2.py:90-92), loops over requests for attention (qwen2.py:118-126) and projects the
last row of every chunk (qwen2.py:131-136).  Here the per-step metadata (ids,
positions, slot mapping, block tables, row offsets) is built once on the host, copied
in one transfer, and every kernel runs over the whole flattened batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheManager, PagedGroup


@dataclass
class StepEntry:
    request_id: str
    tokens: list
    want: list = field(default_factory=list)     # places among ``tokens`` whose logits are wanted


class GroupView:
    """What a part sees of one cache group during a step."""

    def __init__(self, group, page_size):
        self.spec = group.spec
        self.kind = group.spec.kind
        self.storage = group.storage
        self.page_size = page_size
        self.slot_mapping = None      # int32 [T]: flat slot of every token (paged groups)
        self.block_table = None       # int32 [R, max_pages] (paged groups)
        self.max_pages = 0

    def kv_slot(self, slot: int):
        return self.storage[slot, 0], self.storage[slot, 1]

    def state(self, slot: int):
        """[max_requests, *state_shape] storage of one state slot layer; index with ctx.state_slots."""
        return self.storage[slot]


class StepContext:
    """Everything a part may read during one step.  Device tensors are int32."""

    def __init__(self):
        self.ops = None
        self.dtype = None
        self.device = None
        self.num_tokens = 0
        self.num_requests = 0
        self.num_logit_rows = 0
        self.token_ids = self.positions = self.token_request = None
        self.cu_q = self.q_start = self.ctx_len = self.state_slots = self.logit_rows = None
        self.max_q_len = 0
        self.max_ctx_len = 0
        self.decode_only = False
        self.groups: list[GroupView] = []
        # host copies, for parts that plan on the host
        self.host_starts: list[int] = []
        self.host_lengths: list[int] = []
        self.host_state_slots: list[int] = []
        self.request_ids: list[str] = []


class ModelRunner:
    def __init__(self, model, cache: CacheManager, ops=None):
        if ops is None:
            from .. import ops as cuda_ops      # raises if the CUDA extension cannot be had
            ops = cuda_ops
        self.model = model
        self.cache = cache
        self.ops = ops
        self.device = cache.device
        self.vocab_size = model.plan.vocab_size
        self._ring = []
        self._ring_at = 0
        self.steps_run = 0
        self.h2d_bytes = 0           # bytes of step metadata copied to the device so far

    # ------------------------------------------------------------------------------------------
    def _check(self, entries) -> None:
        if not entries:
            raise ValueError("empty step")
        seen = set()
        for e in entries:
            if len(e.tokens) < 1:
                raise ValueError("empty forward chunks")
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            for w in e.want:
                if not (0 <= w < n):
                    raise ValueError(f"request {e.request_id!r}: wanted place {w} outside its {n} tokens")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab_size:
                raise ValueError(f"request {e.request_id!r}: token id outside [0, {self.vocab_size})")

    def _reserve(self, entries) -> None:
        """Reserve for the whole batch or for none of it."""
        cache = self.cache
        made = []
        try:
            for e in entries:
                target = cache.tokens_of(e.request_id) + len(e.tokens)
                before = cache.reserved_tokens(e.request_id) if e.request_id in cache.requests else None
                cache.reserve(e.request_id, target)
                made.append((e.request_id, before))
        except Exception:
            # undo what this call reserved: pages beyond what each request held before
            for rid, before in made:
                if before is None:
                    cache.free(rid)
                else:
                    rc = cache.requests[rid]
                    keep = before // cache.page_size
                    for gi, g in cache.paged:
                        for page in rc.tables[gi][keep:]:
                            g.pool.release(page)
                        del rc.tables[gi][keep:]
            raise

    def _staging(self, count: int) -> torch.Tensor:
        """A pinned host buffer that no copy still in flight reads from.  The host runs ahead of
        the device, so a buffer is taken again only after the copy that last used it has finished."""
        if not self._ring:
            self._ring = [[torch.empty(1 << 14, dtype=torch.int32, pin_memory=True), torch.cuda.Event()]
                          for _ in range(4)]
            self._ring_at = 0
        self._ring_at = (self._ring_at + 1) % len(self._ring)
        slot = self._ring[self._ring_at]
        slot[1].synchronize()
        if slot[0].numel() < count:
            slot[0] = torch.empty(max(count, 2 * slot[0].numel()), dtype=torch.int32, pin_memory=True)
        return slot[0][:count]

    def _upload(self, arrays: list) -> list:
        """One host buffer, one transfer; returns device views in the order given."""
        sizes = [len(a) for a in arrays]
        # every piece starts on a 16-byte boundary so that kernels may use vector loads
        offsets, total = [], 0
        for s in sizes:
            offsets.append(total)
            total += (s + 3) // 4 * 4
        total = max(total, 4)
        if self.device.type == "cuda":
            host = self._staging(total)
        else:
            host = torch.empty(total, dtype=torch.int32)
        view = host.numpy()
        for a, o, s in zip(arrays, offsets, sizes):
            if s:
                view[o:o + s] = a
        self.h2d_bytes += total * 4
        if self.device.type == "cuda":
            dev = host.to(self.device, non_blocking=True)
            self._ring[self._ring_at][1].record()       # the copy out of this buffer is done after this
        else:
            dev = host.clone()
        return [dev[o:o + s] for o, s in zip(offsets, sizes)]

    # ------------------------------------------------------------------------------------------
    def build_context(self, entries) -> StepContext:
        cache = self.cache
        ctx = StepContext()
        ctx.ops, ctx.dtype, ctx.device = self.ops, self.model.dtype, self.device
        starts = [cache.tokens_of(e.request_id) for e in entries]
        lengths = [len(e.tokens) for e in entries]
        T, R = sum(lengths), len(entries)
        token_ids = [t for e in entries for t in e.tokens]
        positions = [p for s, n in zip(starts, lengths) for p in range(s, s + n)]
        token_request = [r for r, n in enumerate(lengths) for _ in range(n)]
        cu_q = [0]
        for n in lengths:
            cu_q.append(cu_q[-1] + n)
        ctx_len = [s + n for s, n in zip(starts, lengths)]
        state_slots = [cache.requests[e.request_id].state_slot for e in entries]
        logit_rows = [cu_q[r] + w for r, e in enumerate(entries) for w in e.want]
        arrays = [np.asarray(token_ids, dtype=np.int32), np.asarray(positions, dtype=np.int32),
                  np.asarray(token_request, dtype=np.int32), np.asarray(cu_q, dtype=np.int32),
                  np.asarray(starts, dtype=np.int32), np.asarray(ctx_len, dtype=np.int32),
                  np.asarray(state_slots, dtype=np.int32), np.asarray(logit_rows, dtype=np.int32)]
        views = []
        for gi, g in enumerate(cache.groups):
            view = GroupView(g, cache.page_size)
            if isinstance(g, PagedGroup):
                slots = []
                for e, s, n in zip(entries, starts, lengths):
                    slots.extend(cache.slot_mapping(e.request_id, gi, s, n))
                tables = [cache.table(e.request_id, gi) for e in entries]
                view.max_pages = max(1, max(-(-c // cache.page_size) for c in ctx_len))
                bt = np.full((R, view.max_pages), -1, dtype=np.int32)
                for r, t in enumerate(tables):
                    k = min(len(t), view.max_pages)
                    bt[r, :k] = t[:k]
                arrays += [np.asarray(slots, dtype=np.int32), bt.reshape(-1)]
            views.append(view)
        dev = self._upload(arrays)
        (ctx.token_ids, ctx.positions, ctx.token_request, ctx.cu_q, ctx.q_start, ctx.ctx_len,
         ctx.state_slots, ctx.logit_rows) = dev[:8]
        k = 8
        for view, g in zip(views, cache.groups):
            if isinstance(g, PagedGroup):
                view.slot_mapping = dev[k]
                view.block_table = dev[k + 1].view(R, view.max_pages)
                k += 2
        ctx.groups = views
        ctx.num_tokens, ctx.num_requests, ctx.num_logit_rows = T, R, len(logit_rows)
        ctx.max_q_len, ctx.max_ctx_len = max(lengths), max(ctx_len)
        ctx.decode_only = ctx.max_q_len == 1
        ctx.host_starts, ctx.host_lengths, ctx.host_state_slots = starts, lengths, state_slots
        ctx.request_ids = [e.request_id for e in entries]
        return ctx

    @torch.inference_mode()
    def step(self, entries):
        """Run one batch.  Returns float32 logits [number of wanted places, vocab] in the order
        of the entries and of their ``want`` (None when nothing is wanted)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._check(entries)
        self._reserve(entries)
        ctx = self.build_context(entries)
        logits = self.model.forward(ctx)
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        return logits

    def finish(self, request_id: str) -> None:
        """The request is over: what it holds is given back."""
        self.cache.free(request_id)
