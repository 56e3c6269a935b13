"""The step function: run a batch of (request, its next tokens) from the cache.

``ModelRunner.step(entries)`` takes, per request, the tokens that follow what the cache
already holds for it — a portion of a prompt of any length, or one decoded token — and
the places among them whose logits are wanted.  All entries run as one flat batch; new
keys and values go to the request's pages; logits come back as ``[wanted, vocab]``
32-bit, in the order of the entries and of their ``want`` lists.

The reference's step is either one whole-prompt forward per admitted request or one
rectangular single-token forward over all running requests
(src/minigpt_infer/engine/engine.py:101-118, 210-283); its index tensors are rebuilt
from Python lists and copied every step.  Here the step's integers are packed into one
pinned buffer and cross to the device in one copy.
"""

from __future__ import annotations

from array import array
from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import NO_PAGE, CacheFullError, CacheManager
from ..cache.storage import CacheStorage
from ..parts.base import Part
from ..parts.context import HostBatch, StepContext, StepPlan
from ..parts.model import DecoderModel


class StepError(ValueError):
    """A step that cannot run: bad token ids, positions past the table, empty entry."""


@dataclass
class StepEntry:
    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


@dataclass
class _DecodeGraph:
    """One captured decode step for a fixed number of rows: its static inputs and outputs."""

    rows: int
    offsets: list
    meta: torch.Tensor            # device int32: every integer input of the step
    staging: torch.Tensor         # pinned host copy that is filled each step
    ctx: StepContext
    graph: object = None
    logits: torch.Tensor | None = None
    kernels: int = 0              # kernel launches inside the graph
    # per row: which state of which request's tables the staging buffer holds (None: no pages)
    row_tables: list = field(default_factory=list)


@dataclass
class _Packed:
    """The integers of one step, packed on the host, and what the host itself needs of them."""

    buf: np.ndarray
    offsets: list
    total: int
    q_len: list
    ctx_before: list
    state_slot: list
    wanted: int
    extra: list = field(default_factory=list)      # (name, shape) of what the parts planned
    signature: tuple = ()                          # what else decides the parts' launches


@dataclass
class _ShapeGraph:
    """A captured step of one shape (tokens per request, attention work items, wanted rows)."""

    meta: torch.Tensor
    staging: torch.Tensor
    graph: object
    logits: torch.Tensor | None
    kernels: int


class ModelRunner:
    GRAPH_ROWS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)
    SHAPE_GRAPHS = 16              # most captured prompt-step shapes kept at a time

    def __init__(self, model: DecoderModel, manager: CacheManager, storage: CacheStorage,
                 ops, act_dtype: torch.dtype, device, max_context: int | None = None,
                 use_cuda_graphs: bool = True) -> None:
        self.model = model
        self.manager = manager
        self.storage = storage
        self.ops = ops
        self.act_dtype = act_dtype
        self.device = torch.device(device)
        self.vocab_size = model.spec.vocab_size
        limit = model.max_positions
        self.max_context = limit if max_context is None else (
            max_context if limit is None else min(limit, max_context))
        if self.max_context is None:
            self.max_context = (min(g.num_pages * g.page_tokens for g in manager.groups)
                                if manager.groups else manager.num_pages * manager.page_tokens)
        # width of a block table, per cache group (groups may differ in page size)
        self.max_pages = [manager.max_pages_per_request(self.max_context, g)
                          for g in range(len(manager.groups))]
        # parts that prepare something on the host for every step (Part.plan_step)
        self._planners = [part for part in model.parts()
                          if getattr(type(part), "plan_step", Part.plan_step) is not Part.plan_step]
        self._pinned = None
        self._pinned_size = 0
        self.last_h2d_bytes = 0          # bytes of the last step's one host-to-device copy
        # Steps in which every request brings one token have a fixed shape once the batch is
        # padded to a few sizes: they are captured as CUDA graphs and replayed (the reference
        # shows the gain on its own decode step, src/minigpt_infer/graphs.py:96-116).
        self.use_cuda_graphs = (use_cuda_graphs and self.device.type == "cuda"
                                and all(getattr(p, "graph_safe", False) for p in model.parts()))
        self._graphs: dict[int, _DecodeGraph] = {}
        self._graph_pool = None
        self._copy_done = None
        self.graph_replays = 0
        # Steps with prompt portions: a shape that comes a second time (full portions of a long
        # prompt, a benchmark's repeated prompt) is captured too; the host then issues one launch
        # instead of sixty, which is what bounds such a step on a fast GPU.
        # Ids sampled by a step, where the next step finds its tokens (``token_sources``).  A
        # replayed decode step reads them at its start and leaves the argmax of its own logits
        # there at its end, so steady greedy decoding launches nothing but the graph.
        self.sampled_ids = (torch.zeros(self.GRAPH_ROWS[-1], dtype=torch.int32, device=self.device)
                            if self.use_cuda_graphs else None)
        self.greedy_vocab_limit: int | None = None      # ids at or above it are never chosen
        self._greedy_rows = 0                            # rows of sampled_ids the last step filled
        self._shape_seen: dict[tuple, int] = {}
        self._shape_graphs: dict[tuple, _ShapeGraph] = {}
        self.shape_graph_replays = 0

    # ---- requests ---------------------------------------------------------------------
    def length_of(self, request_id: str) -> int:
        return self.manager.get(request_id).length if self.manager.has(request_id) else 0

    def finish(self, request_id: str) -> None:
        """Give back everything the request holds."""
        if self.manager.has(request_id):
            self.manager.release(request_id)

    # ---- one step -----------------------------------------------------------------------
    @staticmethod
    def _as_int32(tokens) -> np.ndarray:
        """A portion of a prompt as an int32 array (the one conversion of the list in a step)."""
        if isinstance(tokens, np.ndarray):
            if tokens.dtype == np.int32:
                return tokens
            if tokens.dtype.kind not in "iu" or (tokens.size and not (
                    -2**31 <= int(tokens.min()) and int(tokens.max()) < 2**31)):
                raise StepError("token ids must be integers that fit 32 bits")
            return tokens.astype(np.int32)
        try:
            return np.frombuffer(array("i", tokens), dtype=np.int32)
        except (OverflowError, TypeError) as err:
            raise StepError(f"token ids must be integers that fit 32 bits ({err})") from None

    def _validate(self, entries: Sequence[StepEntry]) -> list:
        """Check the entries; returns, per entry, its tokens as an int32 array where the entry is
        a portion of a prompt (None for the few tokens of a decoding request)."""
        seen = set()
        arrays = []
        vocab, max_context, length_of = self.vocab_size, self.max_context, self.length_of
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 1:                                   # a decoding request: the common case, kept short
                t = e.tokens[0]
                want = e.want
                if (0 <= t < vocab and (not want or (len(want) == 1 and want[0] == 0))
                        and length_of(e.request_id) + 1 <= max_context):
                    arrays.append(None)
                    continue                             # (anything else falls through to the messages below)
            if n == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            if n > 16:                                   # a prompt portion: one pass in numpy
                ids = self._as_int32(e.tokens)
                low, high = int(ids.min()), int(ids.max())
                bad = low if low < 0 else high if high >= self.vocab_size else None
                arrays.append(ids)
            else:
                bad = next((t for t in e.tokens if not (0 <= int(t) < self.vocab_size)), None)
                arrays.append(None)
            if bad is not None:
                raise StepError(f"token id {bad} of request {e.request_id!r} is outside "
                                f"the vocabulary (0..{self.vocab_size - 1})")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.request_id!r} wants logits at {w}, "
                                    f"but brings {n} tokens")
            end = self.length_of(e.request_id) + n
            if end > self.max_context:
                raise StepError(
                    f"request {e.request_id!r} would reach {end} tokens; the model's "
                    f"position table ends at {self.max_context}")
        return arrays

    def _reserve(self, entries: Sequence[StepEntry]) -> None:
        m = self.manager
        need = [0] * len(m.groups)
        new_requests = 0
        short = []                       # entries whose pages do not hold the new tokens yet
        for e in entries:
            req = m.requests.get(e.request_id)
            if req is None:
                new_requests += 1
                end = len(e.tokens)
            else:
                end = req.length + len(e.tokens)
                if end <= req.capacity:
                    continue
            short.append(e)
            for g, n in enumerate(m.pages_needed(e.request_id if req is not None else None, end)):
                need[g] += n
        if not short:
            return
        for g, n in enumerate(need):
            if n > m.groups[g].pool.num_free:
                raise CacheFullError(
                    f"step needs {n} new pages in cache group {g}, {m.groups[g].pool.num_free} free")
        if new_requests > m.slots.num_free:
            raise CacheFullError("step admits more requests than there are free state slots")
        for e in short:
            if not m.has(e.request_id):
                m.admit(e.request_id)
            ok = m.reserve(e.request_id, m.get(e.request_id).length + len(e.tokens))
            assert ok, "pages were counted a moment ago"

    def _pack(self, entries: Sequence[StepEntry], arrays=None) -> _Packed:
        """Pack the step's integers into one int32 buffer on the host.  ``arrays``: what
        _validate returned for these entries, if it ran."""
        m = self.manager
        n_groups = len(m.groups)
        R = len(entries)
        N = sum(len(e.tokens) for e in entries)
        W = sum(len(e.want) for e in entries)
        P = self.max_pages
        host_q_len = [len(e.tokens) for e in entries]
        host_ctx = [m.get(e.request_id).length for e in entries]
        host_slot = [m.get(e.request_id).state_slot for e in entries]
        # what the parts plan on the host for this batch (work lists of their kernels and the like)
        plan = StepPlan()
        if self._planners:
            batch = HostBatch(host_q_len, host_ctx, host_slot, self.act_dtype)
            for part in self._planners:
                part.plan_step(batch, plan, self.ops)
        planned = [(name, np.ascontiguousarray(a, dtype=np.int32)) for name, a in plan.arrays.items()]
        # layout of the packed int32 buffer
        sizes = ([N, N, N, R, R, R, R, W] + [R * P[g] for g in range(n_groups)] + [N] * n_groups
                 + [a.size for _, a in planned])
        offsets = [0]
        for size in sizes:
            offsets.append(offsets[-1] + size)
        total = offsets[-1]
        buf = np.empty(max(total, 1), dtype=np.int32)

        def seg(i):
            return buf[offsets[i]: offsets[i + 1]]

        token_ids, positions, token_request = seg(0), seg(1), seg(2)
        q_start, q_len, ctx_before, state_slot, logit_rows = seg(3), seg(4), seg(5), seg(6), seg(7)
        tables = [seg(8 + g).reshape(R, P[g]) for g in range(n_groups)]
        slots = [seg(8 + n_groups + g) for g in range(n_groups)]
        row = 0
        w = 0
        for r, e in enumerate(entries):
            req = m.get(e.request_id)
            n = host_q_len[r]
            q_start[r], q_len[r], ctx_before[r], state_slot[r] = row, n, req.length, req.state_slot
            ids = arrays[r] if arrays is not None else None
            token_ids[row: row + n] = ids if ids is not None else np.asarray(e.tokens, dtype=np.int32)
            token_request[row: row + n] = r
            if n == 1:
                positions[row] = req.length
            else:
                pos = positions[row: row + n]
                pos[:] = np.arange(req.length, req.length + n, dtype=np.int32)
            for g in range(n_groups):
                pt = m.groups[g].page_tokens
                if n == 1:
                    page_index, within = req.length // pt, req.length % pt
                else:
                    page_index = pos // pt
                    within = pos - page_index * pt
                held = req.tables[g]
                tables[g][r, :len(held)] = held
                tables[g][r, len(held):] = NO_PAGE
                if n == 1:
                    pages = held[page_index]
                    bad = pages == NO_PAGE
                else:
                    pages = tables[g][r][page_index]
                    bad = int(pages.min()) == NO_PAGE
                if bad:
                    raise StepError(f"request {e.request_id!r} writes to a page it gave back")
                slots[g][row: row + n] = pages * pt + within
            for k in e.want:
                logit_rows[w] = row + int(k)
                w += 1
            row += n

        for i, (_, a) in enumerate(planned):
            seg(8 + 2 * n_groups + i)[:] = a.reshape(-1)
        return _Packed(buf, offsets, total, host_q_len, host_ctx, host_slot, W,
                       [(name, a.shape) for name, a in planned], tuple(plan.signature))

    def _context(self, dev: torch.Tensor, packed: _Packed) -> StepContext:
        """Describe the batch whose packed integers lie in ``dev``."""
        offsets, n_groups = packed.offsets, len(self.manager.groups)
        R, P = len(packed.q_len), self.max_pages

        def dseg(i):
            return dev[int(offsets[i]): int(offsets[i + 1])]

        return StepContext(
            ops=self.ops, act_dtype=self.act_dtype, num_tokens=sum(packed.q_len), num_requests=R,
            token_ids=dseg(0), positions=dseg(1), token_request=dseg(2),
            req_q_start=dseg(3), req_q_len=dseg(4), req_ctx_before=dseg(5),
            req_state_slot=dseg(6), logit_rows=dseg(7),
            block_tables=[dseg(8 + g).view(R, P[g]) for g in range(n_groups)],
            slot_mapping=[dseg(8 + n_groups + g) for g in range(n_groups)],
            extra={name: dseg(8 + 2 * n_groups + i).view(shape)
                   for i, (name, shape) in enumerate(packed.extra)},
            host_q_len=packed.q_len, host_ctx_before=packed.ctx_before,
            host_state_slot=packed.state_slot,
            max_q_len=max(packed.q_len),
            max_ctx_after=max(a + b for a, b in zip(packed.q_len, packed.ctx_before)),
            decode_only=all(n == 1 for n in packed.q_len), storage=self.storage)

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Pack the step's integers, copy them to the device once, and describe the batch."""
        packed = self._pack(entries)
        return self._context(self._to_device(packed.buf, packed.total), packed)

    def _to_device(self, buf: np.ndarray, total: int) -> torch.Tensor:
        self.last_h2d_bytes = 4 * total
        if self.device.type != "cuda":
            return torch.from_numpy(buf[:total].copy())
        if self._pinned is None or self._pinned_size < total:
            self._pinned_size = max(total, 2 * self._pinned_size, 4096)
            self._pinned = torch.empty(self._pinned_size, dtype=torch.int32, pin_memory=True)
        else:
            # The last step's copy out of the pinned buffer must be over before it is reused.
            torch.cuda.current_stream(self.device).synchronize()
        self._pinned[:total].numpy()[:] = buf[:total]
        return self._pinned[:total].to(self.device, non_blocking=True)

    def _upload(self, meta: torch.Tensor, staging: torch.Tensor) -> None:
        upload = getattr(self.ops, "upload_ints", None)
        if upload is not None and meta.numel() <= 4096:   # larger ones go faster on the copy engine
            upload(meta, staging)
        else:
            meta.copy_(staging, non_blocking=True)

    # ---- decode steps as CUDA graphs ---------------------------------------------------------
    def _graph_layout(self, rows: int):
        g, pages = len(self.manager.groups), self.max_pages
        sizes = [rows] * 8 + [rows * pages[i] for i in range(g)] + [rows] * g + [rows]     # last: token sources
        offsets = [0]
        for n in sizes:
            offsets.append(offsets[-1] + n)
        return offsets

    def _capture(self, rows: int) -> _DecodeGraph:
        g, pages = len(self.manager.groups), self.max_pages
        offsets = self._graph_layout(rows)
        meta = torch.zeros(offsets[-1], dtype=torch.int32, device=self.device)
        staging = torch.zeros(offsets[-1], dtype=torch.int32, pin_memory=True)

        def seg(i):
            return meta[offsets[i]: offsets[i + 1]]

        ctx = StepContext(
            ops=self.ops, act_dtype=self.act_dtype, num_tokens=rows, num_requests=rows,
            token_ids=seg(0), positions=seg(1), token_request=seg(2), req_q_start=seg(3),
            req_q_len=seg(4), req_ctx_before=seg(5), req_state_slot=seg(6), logit_rows=seg(7),
            block_tables=[seg(8 + i).view(rows, pages[i]) for i in range(g)],
            slot_mapping=[seg(8 + g + i) for i in range(g)],
            host_q_len=[1] * rows, host_ctx_before=[0] * rows, host_state_slot=[0] * rows,
            max_q_len=1, max_ctx_after=self.max_context, decode_only=True, storage=self.storage)
        # Tokens that the step before sampled are fetched on the device (source >= 0): by the
        # embedding itself if it can, else by a kernel in front of it.
        sources = meta[offsets[8 + 2 * g]: offsets[9 + 2 * g]]
        fused_fetch = getattr(self.model.embedding, "takes_token_source", False)
        if fused_fetch:
            ctx.token_source, ctx.fed_ids = sources, self.sampled_ids
        state = _DecodeGraph(rows, offsets, meta, staging, ctx)
        self._fill_graph_inputs(state, [])                # all rows are padding: nothing is written
        meta.copy_(staging)
        self._forward(ctx)                           # warm-up outside the capture
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        launches = getattr(self.ops, "launches", 0)
        # Inside the graph every kernel follows a kernel, so the ones that can may start while
        # their predecessor drains (programmatic dependent launch).
        dependent = getattr(self.ops, "set_dependent_launch", None)
        if dependent is not None:
            dependent(True)
        try:
            with torch.cuda.graph(graph, pool=self._graph_pool):
                if not fused_fetch:
                    self.ops.gather_tokens(ctx.token_ids, sources, self.sampled_ids)
                # this step's greedy choice is left where the next step looks for it: by the head
                # on its way if it can, else by the argmax kernels
                ctx.greedy_out, ctx.greedy_vocab_limit = self.sampled_ids[:rows], self.greedy_vocab_limit
                ctx.greedy_taken = False
                state.logits = self._forward(ctx)
                if not ctx.greedy_taken:
                    self.ops.argmax(state.logits, self.greedy_vocab_limit, out=self.sampled_ids[:rows])
        finally:
            if dependent is not None:
                dependent(False)
        state.kernels = getattr(self.ops, "launches", 0) - launches
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        state.graph = graph
        return state

    def capture_decode_graphs(self, max_rows: int) -> int:
        """Capture now, rather than at their first use, the decode graphs of every row bucket that
        batches of up to ``max_rows`` single tokens can meet (a capture runs the model twice on
        padding rows and takes some ten milliseconds: with this the first requests do not pay for
        it).  Returns the number of graphs captured; 0 where decode steps are not replayed."""
        if not self.use_cuda_graphs or max_rows < 1:
            return 0
        made = 0
        for rows in self.GRAPH_ROWS:
            if rows not in self._graphs:
                self._graphs[rows] = self._capture(rows)
                made += 1
            if rows >= max_rows:
                break
        return made

    def _fill_graph_inputs(self, state: _DecodeGraph, entries: Sequence[StepEntry],
                           token_sources=None) -> None:
        """The step's integers into the pinned staging buffer.  The block tables of a row are
        written again only if the row's request or its tables changed since the last step: in
        steady decoding a table changes once per page of tokens."""
        m = self.manager
        rows, off = state.rows, state.offsets
        buf = state.staging.numpy()
        g, pages = len(m.groups), self.max_pages
        n = len(entries)
        if not state.row_tables:                                        # first use: everything is padding
            state.row_tables = [None] * rows
            buf[off[2]: off[3]] = np.arange(rows, dtype=np.int32)       # request of each row
            buf[off[3]: off[4]] = np.arange(rows, dtype=np.int32)
            buf[off[7]: off[8]] = np.arange(rows, dtype=np.int32)       # logits of every row
            for i in range(g):
                buf[off[8 + i]: off[9 + i]] = NO_PAGE
        reqs = [m.get(e.request_id) for e in entries]
        lengths = [req.length for req in reqs]
        buf[off[0]: off[0] + n] = [int(e.tokens[0]) for e in entries]
        buf[off[0] + n: off[1]] = 0
        buf[off[1]: off[1] + n] = lengths
        buf[off[1] + n: off[2]] = -1                                    # position -1 marks padding
        buf[off[4]: off[4] + n] = 1
        buf[off[4] + n: off[5]] = 0
        buf[off[5]: off[5] + n] = lengths
        buf[off[5] + n: off[6]] = 0
        buf[off[6]: off[6] + n] = [req.state_slot for req in reqs]
        buf[off[6] + n: off[7]] = 0
        src = off[8 + 2 * g]
        buf[src: src + rows] = -1                                       # token comes from the host
        if token_sources is not None:
            buf[src: src + n] = token_sources
        row_tables = state.row_tables
        for i in range(g):
            buf[off[8 + g + i] + n: off[9 + g + i]] = -1                # padding rows write nowhere
        for r, req in enumerate(reqs):
            held = (req.serial, req.version)
            fresh = row_tables[r] != held
            length = lengths[r]
            for i in range(g):
                table = req.tables[i]
                pt = m.groups[i].page_tokens
                if fresh:
                    base = off[8 + i] + r * pages[i]
                    buf[base: base + len(table)] = table
                    buf[base + len(table): base + pages[i]] = NO_PAGE
                page = table[length // pt]
                if page == NO_PAGE:
                    raise StepError(f"request {entries[r].request_id!r} writes to a page it gave back")
                buf[off[8 + g + i] + r] = page * pt + length % pt
            row_tables[r] = held
        for r in range(n, rows):                                        # rows that held a request last time
            if row_tables[r] is not None:
                for i in range(g):
                    base = off[8 + i] + r * pages[i]
                    buf[base: base + pages[i]] = NO_PAGE
                row_tables[r] = None

    def _graph_step(self, entries: Sequence[StepEntry], copy: bool, token_sources=None,
                    previous_ids=None):
        rows = next(b for b in self.GRAPH_ROWS if b >= len(entries))
        state = self._graphs.get(rows)
        if state is None:
            state = self._graphs[rows] = self._capture(rows)
        if self._copy_done is not None:
            self._copy_done.synchronize()                 # the staging buffer is free again
        self._fill_graph_inputs(state, entries, token_sources)
        self._upload(state.meta, state.staging)
        if self._copy_done is None:
            self._copy_done = torch.cuda.Event()
        self._copy_done.record()
        self.last_h2d_bytes = 4 * state.offsets[-1]
        if token_sources is not None and previous_ids is not None and (
                previous_ids.data_ptr() != self.sampled_ids.data_ptr()):
            # ids that were sampled into a tensor of the caller's: bring them where the graph looks
            self.sampled_ids[: previous_ids.numel()].copy_(previous_ids)
        state.graph.replay()
        self.graph_replays += 1
        if hasattr(self.ops, "launches"):
            self.ops.launches += state.kernels
        wanted = [r for r, e in enumerate(entries) if len(e.want)]
        self._greedy_rows = len(entries) if len(wanted) == len(entries) else 0
        if not wanted:
            return None
        if len(wanted) == len(entries):
            logits = state.logits[: len(entries)]
        else:
            logits = state.logits[wanted]
            copy = False
        return logits.clone() if copy else logits

    # ---- steps with prompt portions: eager, or replayed once their shape has come twice --------
    def _prompt_step(self, entries: Sequence[StepEntry], copy: bool, arrays=None):
        packed = self._pack(entries, arrays)
        decode_only = all(n == 1 for n in packed.q_len)
        if not self.use_cuda_graphs or decode_only:
            return self._forward(self._context(self._to_device(packed.buf, packed.total), packed))
        # what the launches of a step depend on besides the device-side integers
        key = (tuple(packed.q_len), packed.wanted, tuple(packed.extra), packed.signature)
        state = self._shape_graphs.get(key)
        if state is None:
            seen = self._shape_seen.get(key, 0) + 1
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            self._shape_seen[key] = seen
            if seen < 2:
                return self._forward(self._context(self._to_device(packed.buf, packed.total), packed))
            return self._capture_shape(key, packed)
        self._shape_graphs[key] = self._shape_graphs.pop(key)         # most recently used last
        self._stage(state, packed)
        state.graph.replay()
        self.shape_graph_replays += 1
        if hasattr(self.ops, "launches"):
            self.ops.launches += state.kernels
        if state.logits is None:
            return None
        return state.logits.clone() if copy else state.logits

    def _forward(self, ctx):
        """The model's forward pass over one batch; the kernel set is told that a pass begins (what
        it remembers from launch to launch, such as which matrix followed which, starts anew)."""
        begin = getattr(self.ops, "begin_forward", None)
        if begin is not None:
            begin()
        return self.model.forward(ctx)

    def _stage(self, state: _ShapeGraph, packed: _Packed) -> None:
        if self._copy_done is not None:
            self._copy_done.synchronize()                 # the staging buffer is free again
        state.staging.numpy()[: packed.total] = packed.buf[: packed.total]
        self._upload(state.meta, state.staging)
        if self._copy_done is None:
            self._copy_done = torch.cuda.Event()
        self._copy_done.record()
        self.last_h2d_bytes = 4 * packed.total

    def _capture_shape(self, key: tuple, packed: _Packed):
        """Run the step eagerly from persistent inputs (its result is returned), then capture
        the same launches for the next step of this shape."""
        size = max(packed.total, 1)
        state = _ShapeGraph(torch.zeros(size, dtype=torch.int32, device=self.device),
                            torch.zeros(size, dtype=torch.int32, pin_memory=True), None, None, 0)
        self._stage(state, packed)
        ctx = self._context(state.meta, packed)
        result = self._forward(ctx)
        if result is not None:
            result = result.clone()                        # the capture below reuses the memory
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        launches = getattr(self.ops, "launches", 0)
        dependent = getattr(self.ops, "set_dependent_launch", None)
        if dependent is not None:
            dependent(True)
        try:
            with torch.cuda.graph(graph, pool=self._graph_pool):
                state.logits = self._forward(ctx)
        finally:
            if dependent is not None:
                dependent(False)
        state.kernels = getattr(self.ops, "launches", 0) - launches
        if hasattr(self.ops, "launches"):
            self.ops.launches = launches                   # captured, not run
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        state.graph = graph
        while len(self._shape_graphs) >= self.SHAPE_GRAPHS:
            self._shape_graphs.pop(next(iter(self._shape_graphs)))     # least recently used
        self._shape_graphs[key] = state
        return result

    def greedy_ids(self, rows: int):
        """The argmax of each of the last step's ``rows`` logit rows, if that step took it on its
        way (a replayed decode step whose every entry wanted its logits); else None."""
        if rows and self._greedy_rows == rows:
            return self.sampled_ids[:rows]
        return None

    def can_feed_tokens_on_device(self, n_entries: int) -> bool:
        """Whether a step of ``n_entries`` single tokens may take its tokens from the ids that the
        previous step sampled, without the host seeing them first (``token_sources``)."""
        return self.use_cuda_graphs and 0 < n_entries <= self.GRAPH_ROWS[-1]

    def step(self, entries: Sequence[StepEntry], copy: bool = True, token_sources=None,
             previous_ids=None) -> torch.Tensor | None:
        """Run the entries as one batch.  Returns ``[wanted, vocab]`` float32 logits on the
        device (None if nothing was wanted).  With ``copy=False`` the result may be a view of
        a buffer that the next step overwrites.

        ``token_sources`` (one int per entry, only for steps of single tokens): where it is
        >= 0 the entry's token is taken on the device from ``previous_ids[token_sources[i]]``
        (int32 ids sampled by the step before) and the entry's own token is a placeholder."""
        entries = list(entries)
        self._greedy_rows = 0
        if not entries:
            return None
        arrays = self._validate(entries)
        self._reserve(entries)
        if token_sources is not None and not (
                self.can_feed_tokens_on_device(len(entries)) and all(len(e.tokens) == 1 for e in entries)):
            raise StepError("tokens can be fed on the device only to steps of single tokens")
        if (self.use_cuda_graphs and len(entries) <= self.GRAPH_ROWS[-1]
                and all(len(e.tokens) == 1 for e in entries)):
            logits = self._graph_step(entries, copy, token_sources, previous_ids)
        else:
            logits = self._prompt_step(entries, copy, arrays)
        for e in entries:
            self.manager.advance(e.request_id, self.manager.get(e.request_id).length + len(e.tokens))
        return logits
