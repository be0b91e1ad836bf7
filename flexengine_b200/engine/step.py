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
    carry: int | None = None                     # the one token is element ``carry`` of the tensor given to step()
                                                 # as ``carried`` (on the device); ``tokens`` holds a placeholder


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
        self._graph_buckets = []
        self._graphs = {}
        self.graph_replays = 0

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
        held, paged = cache.requests, cache.paged
        for e in entries:
            rc = held.get(e.request_id)
            if rc is None:
                break
            need = rc.tokens + len(e.tokens)
            if any(len(rc.tables[gi]) * g.page_size < need for gi, g in paged):
                break
        else:
            return                      # the scheduler reserved already
        made = []
        try:
            for e in entries:
                target = cache.tokens_of(e.request_id) + len(e.tokens)
                rc = cache.requests.get(e.request_id)
                before = [len(rc.tables[gi]) for gi, _ in paged] if rc is not None else None
                cache.reserve(e.request_id, target)
                made.append((e.request_id, before))
        except Exception:
            # undo what this call reserved: pages beyond what each request held before
            for rid, before in made:
                if before is None:
                    cache.free(rid)
                    continue
                for (gi, _g), keep in zip(paged, before):
                    cache.truncate(rid, gi, keep)
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

    @staticmethod
    def _layout(sizes: list):
        """Offsets of the pieces in one buffer; every piece starts on a 16-byte boundary."""
        offsets, total = [], 0
        for s in sizes:
            offsets.append(total)
            total += (s + 3) // 4 * 4
        return offsets, max(total, 4)

    def _upload(self, arrays: list, into=None) -> list:
        """One host buffer, one transfer; returns device views in the order given.  ``into``: a
        device buffer of fixed address to copy into (CUDA graphs), else a fresh one."""
        sizes = [len(a) for a in arrays]
        offsets, total = self._layout(sizes)
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
            if into is not None:
                into[:total].copy_(host, non_blocking=True)
                dev = into
            else:
                dev = host.to(self.device, non_blocking=True)
            self._ring[self._ring_at][1].record()       # the copy out of this buffer is done after this
        else:
            dev = host.clone()
        return [dev[o:o + s] for o, s in zip(offsets, sizes)]

    # ------------------------------------------------------------------------------------------
    def _metadata(self, entries, pad_to: int = 0, max_pages=None, carrying: bool = False):
        """The step's index arrays on the host.  ``pad_to`` > len(entries) appends padding requests of
        one token each (token 0 at position 0, no cache write, state slot -1, page 0) so that a
        batch fits a fixed shape; ``entries`` may then be empty (the stand-in batch a graph is captured
        with).  ``max_pages`` fixes the width of each group's block table.  ``carrying``
        appends, for entries whose token is still on the device, the row to fill and where it comes
        from (one pair per request with a fixed shape, row -1 where nothing is carried).

        A padding request must leave no trace: kernels skip cache slot -1, and a part that keeps
        per-request state skips state slot -1 (``parts.base``).

        Everything is array arithmetic over the requests' seats (their state slots): block tables and slot
        mappings are gathered from the cache manager's matrix of table rows, not looped over in Python."""
        cache = self.cache
        held = cache.requests
        real = len(entries)
        caches = [held[e.request_id] for e in entries]
        pad = max(0, pad_to - real)
        R = real + pad
        starts = np.zeros(R, dtype=np.int32)
        lengths = np.ones(R, dtype=np.int32)
        seats = np.full(R, -1, dtype=np.int32)
        if real:
            starts[:real] = [rc.tokens for rc in caches]
            lengths[:real] = [len(e.tokens) for e in entries]
            seats[:real] = [rc.state_slot for rc in caches]
        cu_q = np.zeros(R + 1, dtype=np.int32)
        np.cumsum(lengths, out=cu_q[1:])
        T = int(cu_q[-1])
        ctx_len = starts + lengths
        longest = int(ctx_len.max())
        if int(lengths.max()) == 1:                  # a decode step: one token a request
            token_ids = np.zeros(R, dtype=np.int32)
            if real:
                token_ids[:real] = [e.tokens[0] for e in entries]
            positions = starts
            token_request = np.arange(R, dtype=np.int32)
        else:
            token_ids = np.zeros(T, dtype=np.int32)
            token_ids[:T - pad] = [t for e in entries for t in e.tokens]
            token_request = np.repeat(np.arange(R, dtype=np.int32), lengths)
            positions = np.arange(T, dtype=np.int32) - np.repeat(cu_q[:-1] - starts, lengths)
        if pad_to:
            logit_rows = np.arange(R, dtype=np.int32)          # a fixed shape: every request's one row, padding too
        else:
            logit_rows = np.asarray([cu_q[r] + w for r, e in enumerate(entries) for w in e.want], dtype=np.int32)
        arrays = [token_ids, positions, token_request, cu_q, starts, ctx_len, seats, logit_rows]
        widths = []
        real_tokens = T - pad
        token_seat = seats[token_request[:real_tokens]] if real else None
        for gi, g in enumerate(cache.groups):
            if not isinstance(g, PagedGroup):
                widths.append(0)
                continue
            ps, rows = g.page_size, g.table_rows
            slots = np.full(T, -1, dtype=np.int32)
            if real:
                where = positions[:real_tokens] // ps
                pages = rows[token_seat, where] if int(where.max()) < rows.shape[1] else None
                if pages is None or int(pages.min()) < 0 or g.pool.shared:
                    # something is not as usual (a page not reserved or given back, shared pages in the pool): the
                    # checks and their messages live in the cache manager
                    at = 0
                    for e, n in zip(entries, lengths[:real].tolist()):
                        slots[at:at + n] = cache.slot_mapping(e.request_id, gi, held[e.request_id].tokens, n)
                        at += n
                else:
                    slots[:real_tokens] = pages * ps + positions[:real_tokens] % ps
            width = max_pages[gi] if max_pages else max(1, -(-longest // ps))
            bt = np.full((R, width), -1, dtype=np.int32)
            if real:
                have = min(width, rows.shape[1])
                bt[:real, :have] = rows[seats[:real], :have]
            bt[real:, :] = 0
            arrays += [slots, bt.reshape(-1)]
            widths.append(width)
        if carrying:
            rows_to_fill = np.full(R if pad_to else 0, -1, dtype=np.int32)
            sources = np.zeros(R if pad_to else 0, dtype=np.int32)
            picked = [(r, e.carry) for r, e in enumerate(entries) if e.carry is not None]
            if pad_to:
                for r, c in picked:
                    rows_to_fill[r], sources[r] = cu_q[r], c
            else:
                rows_to_fill = np.asarray([cu_q[r] for r, _ in picked], dtype=np.int32)
                sources = np.asarray([c for _, c in picked], dtype=np.int32)
            arrays += [rows_to_fill, sources]
        info = dict(T=T, R=R, rows=len(logit_rows), starts=starts.tolist(), lengths=lengths.tolist(),
                    state_slots=seats.tolist(), widths=widths, max_q_len=int(lengths.max()), max_ctx_len=longest,
                    request_ids=[e.request_id for e in entries])
        return arrays, info

    def _context(self, dev: list, info: dict) -> StepContext:
        cache = self.cache
        ctx = StepContext()
        ctx.ops, ctx.dtype, ctx.device = self.ops, self.model.dtype, self.device
        (ctx.token_ids, ctx.positions, ctx.token_request, ctx.cu_q, ctx.q_start, ctx.ctx_len,
         ctx.state_slots, ctx.logit_rows) = dev[:8]
        k = 8
        for gi, g in enumerate(cache.groups):
            view = GroupView(g, getattr(g, "page_size", 0))
            if isinstance(g, PagedGroup):
                view.max_pages = info["widths"][gi]
                view.slot_mapping = dev[k]
                view.block_table = dev[k + 1].view(info["R"], view.max_pages)
                k += 2
            ctx.groups.append(view)
        ctx.num_tokens, ctx.num_requests, ctx.num_logit_rows = info["T"], info["R"], info["rows"]
        ctx.max_q_len, ctx.max_ctx_len = info["max_q_len"], info["max_ctx_len"]
        ctx.decode_only = ctx.max_q_len == 1
        ctx.host_starts, ctx.host_lengths = info["starts"], info["lengths"]
        ctx.host_state_slots, ctx.request_ids = info["state_slots"], info["request_ids"]
        return ctx

    def build_context(self, entries, carried=None) -> StepContext:
        arrays, info = self._metadata(entries, carrying=carried is not None)
        dev = self._upload(arrays)
        ctx = self._context(dev, info)
        if carried is not None:
            self.ops.carry_tokens(ctx.token_ids, dev[-2], dev[-1], carried)
        return ctx

    # ---- decode steps as CUDA graphs -----------------------------------------------------------------
    def enable_decode_graphs(self, max_batch: int, max_model_len: int) -> None:
        """Steps in which every request brings one token and wants its logits are replayed from a
        CUDA graph captured per batch-size bucket (the reference captures buckets 1, 2, 4, 8:
        src/flexengine/engine/execution/cuda_graph.py:18-125).  Index arrays live in buffers of
        fixed address and shape: batches are padded up to the bucket, block tables to the longest
        request the engine admits."""
        if self.device.type != "cuda":
            raise ValueError("CUDA graphs need a CUDA device")
        buckets, b = [], 1
        while b < max_batch:
            buckets.append(b)
            b *= 2
        buckets.append(max_batch)
        self._graph_buckets = buckets
        self._graph_max_pages = [-(-max_model_len // g.page_size) if isinstance(g, PagedGroup) else 0
                                 for g in self.cache.groups]
        self._graph_max_len = max_model_len
        self._graphs = {}
        self._graph_pool = torch.cuda.graph_pool_handle()

    def capture_decode_graphs(self) -> int:
        """Capture every bucket now instead of at the first step that needs it (a capture takes tens of
        milliseconds).  Returns how many graphs exist afterwards."""
        for bucket in self._graph_buckets:
            self._graph_for(bucket)
        torch.cuda.synchronize(self.device)
        return len(self._graphs)

    def _graph_for(self, bucket: int):
        """The graph of the forward pass for ``bucket`` requests of one token; captured at first use.

        Warm-up and capture run a stand-in batch of padding requests only: no cache slot is written and no
        state slot touched, so capturing never advances anybody's state, whenever it happens; the real
        requests of the step that asked for the bucket are then run by replaying the graph, once."""
        if bucket in self._graphs:
            return self._graphs[bucket]
        arrays, info = self._metadata([], pad_to=bucket, max_pages=self._graph_max_pages, carrying=True)
        sizes = [len(a) for a in arrays]
        _offsets, total = self._layout(sizes)
        with torch.inference_mode(False):
            static = torch.zeros(total, dtype=torch.int32, device=self.device)
        dev = self._upload(arrays, into=static)
        info = dict(info, max_ctx_len=self._graph_max_len)       # fixes how decode attention splits the keys
        ctx = self._context(dev, info)
        launches_base = getattr(self.ops, "launches", 0)
        # run once outside a graph on a side stream: libraries set themselves up, scratch is allocated
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.model.forward(ctx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        launches_before = getattr(self.ops, "launches", 0)
        # Captured by hand on a stream of its own: the context manager of the library would also collect garbage
        # and hand every cached block back to the driver at each capture (a tenth of a second, and slow allocations
        # afterwards).  All buckets share one memory pool: only one of them runs at a time.
        graph = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph.capture_begin(pool=self._graph_pool, capture_error_mode="thread_local")
            try:
                logits = self.model.forward(ctx)
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)
        launches = getattr(self.ops, "launches", 0) - launches_before
        if hasattr(self.ops, "launches"):
            self.ops.launches = launches_base                    # the stand-in runs are nobody's launches
        record = dict(graph=graph, static=static, logits=logits, total=total, launches=launches)
        self._graphs[bucket] = record
        return record

    def _graph_step(self, entries, carried=None):
        """Replay the graph of the smallest bucket that holds the batch; None if none does."""
        bucket = next((b for b in self._graph_buckets if b >= len(entries)), None)
        if bucket is None:
            return None
        if max(self.cache.tokens_of(e.request_id) for e in entries) + 1 > self._graph_max_len:
            return None
        record = self._graph_for(bucket)
        # the carry arrays are always part of a bucket's buffer, so that its layout does not change
        arrays, _info = self._metadata(entries, pad_to=bucket, max_pages=self._graph_max_pages, carrying=True)
        dev = self._upload(arrays, into=record["static"])
        if carried is not None:
            self.ops.carry_tokens(dev[0], dev[-2], dev[-1], carried)
        record["graph"].replay()
        if hasattr(self.ops, "launches"):
            self.ops.launches += record["launches"]
        self.graph_replays += 1
        return record["logits"][:len(entries)]

    @torch.inference_mode()
    def step(self, entries, carried=None, trusted: bool = False):
        """Run one batch.  Returns float32 logits [number of wanted places, vocab] in the order
        of the entries and of their ``want`` (None when nothing is wanted).  With decode graphs
        on, the returned tensor of a decode step is overwritten by the next such step.
        ``carried``: an int32 tensor on the device from which entries with ``carry`` take their token
        (what the step before sampled, not yet read by the host).  ``trusted``: the caller has checked the
        entries and reserved their pages itself (the engine has: it does not pay for both twice)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not trusted:
            self._check(entries)
        if any(e.carry is not None for e in entries):
            if carried is None:
                raise ValueError("an entry carries its token but no tensor of carried tokens was given")
            for e in entries:
                if e.carry is not None and (len(e.tokens) != 1 or not 0 <= e.carry < carried.numel()):
                    raise ValueError(f"request {e.request_id!r}: a carried token is one token, inside the tensor given")
        else:
            carried = None
        if not trusted:
            self._reserve(entries)
        logits = None
        decode = self._graph_buckets and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        if decode:
            logits = self._graph_step(entries, carried)
        if logits is None:
            ctx = self.build_context(entries, carried)
            logits = self.model.forward(ctx)
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        return logits

    def finish(self, request_id: str) -> None:
        """The request is over: what it holds is given back."""
        self.cache.free(request_id)
