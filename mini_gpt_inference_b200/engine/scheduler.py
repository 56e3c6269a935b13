"""The scheduler: who runs in the next step, with how many tokens, and who gives way.

Kept from the reference (src/minigpt_infer/engine/scheduler.py:23-117): a FIFO ``waiting``
queue and a ``running`` list in admission order; at most ``max_batch_size`` running;
admission stops at the first waiting request that does not fit (no skipping ahead);
prompts take precedence over decoding; when pages run out the newest running request other
than the one in need is preempted — its pages are given back, it returns to the FRONT of
the waiting queue and is recomputed from its tokens (prompt plus what it generated) when
readmitted; if no other is left, the one in need is preempted itself.  Finishing and
cancelling give pages back at once.

Added here, because the reference runs whole prompts alone and decodes separately
(src/minigpt_infer/engine/scheduler.py:9-12): a token budget per step, prompts cut into
portions (``prefill_chunk``), and steps that mix portions with single decoded tokens.  Pages
are taken portion by portion, so a request can be preempted half-way through its prompt.

Order of claims in one step: (1) running requests, oldest first, claim pages for their
share — under ``prefill_priority`` the ones still working through a prompt get the budget
first, then the decoding ones; (2) waiting requests are admitted with what budget and pages
are left.  Only a decoding request preempts; a portion of a prompt shrinks to the free pages
or waits.  If nobody can move, the newest running request gives way.  A request whose prompt plus ``max_tokens`` could never fit the pool or the
position table is refused when it is added, so the queue cannot live-lock on it.
"""

from __future__ import annotations

from collections import deque

from ..cache.manager import CacheManager
from .request import ScheduledChunk, SequenceState, SequenceStatus


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_size: int, max_num_batched_tokens: int,
                 prefill_chunk: int | None = None, policy: str = "prefill_priority") -> None:
        if policy not in ("prefill_priority", "decode_priority"):
            raise ValueError(f"unknown scheduling policy {policy!r}")
        self.cache = cache
        self.max_batch_size = max_batch_size
        self.max_num_batched_tokens = max_num_batched_tokens
        self.prefill_chunk = min(prefill_chunk or max_num_batched_tokens, max_num_batched_tokens)
        self.policy = policy
        self.waiting: deque[SequenceState] = deque()
        self.running: list[SequenceState] = []
        self.num_preemptions = 0
        self._arrivals = 0

    # ---- queue -----------------------------------------------------------------------------
    def add_request(self, seq: SequenceState) -> None:
        # The last sampled token is never fed back, so the cache holds one token less.
        total = seq.prompt_len + seq.request.sampling_params.max_tokens - 1
        if not self.cache.can_ever_hold(total):
            raise ValueError(
                f"request {seq.request_id!r} can never fit: its {total} tokens need more pages "
                f"than a pool has ({', '.join(f'{g.pages_for(total)} of {g.num_pages}' for g in self.cache.groups)})")
        seq.arrival = self._arrivals
        self._arrivals += 1
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    # ---- one step --------------------------------------------------------------------------
    def schedule(self) -> list[ScheduledChunk]:
        """The chunks of the next step.  If every running request is stuck for pages (each
        holds some, none can grow), the newest gives way until someone can move."""
        admit = True
        while True:
            chunks = self._schedule_once(admit)
            if chunks or not self.running:
                return chunks
            self._preempt(self.running[-1])
            admit = False

    def _schedule_once(self, admit: bool) -> list[ScheduledChunk]:
        budget = self.max_num_batched_tokens
        chunks: list[ScheduledChunk] = []
        preemptions_before = self.num_preemptions

        def in_prompt(s: SequenceState) -> bool:
            return s.num_pending_tokens > 1

        first, second = ([s for s in self.running if in_prompt(s)],
                         [s for s in self.running if not in_prompt(s)])
        if self.policy == "decode_priority":
            first, second = second, first
        for seq in first + second:
            if budget == 0:
                break
            if seq.status != SequenceStatus.RUNNING:
                continue                          # preempted a moment ago, in this same pass
            count = min(seq.num_pending_tokens, self.prefill_chunk, budget)
            if in_prompt(seq):
                # A portion of a prompt never pushes anyone out: it shrinks to the pages that
                # are free, and waits a step if there are none.
                count = min(count, self.cache.tokens_that_fit(seq.request_id,
                                                            seq.num_computed_tokens))
                if count == 0:
                    continue
                ok = self.cache.reserve(seq.request_id, seq.num_computed_tokens + count)
                assert ok
            elif not self._claim_pages(seq, count, chunks):
                continue                          # it was preempted itself
            chunks.append(self._chunk(seq, count))
            budget -= count

        # No admission in a step that had to preempt: the pool is short, and the request at
        # the front of the queue is the one that just gave way.
        preempted_now = not admit or self.num_preemptions != preemptions_before
        while (self.waiting and budget > 0 and len(self.running) < self.max_batch_size
               and not preempted_now):
            seq = self.waiting[0]
            count = min(seq.num_pending_tokens, self.prefill_chunk, budget)
            if self.cache.slots.num_free == 0 or not self.cache.can_reserve(None, count):
                break                             # head of the line does not fit: stop admitting
            self.waiting.popleft()
            self.cache.admit(seq.request_id)
            self.cache.reserve(seq.request_id, count)
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            chunks.append(self._chunk(seq, count))
            budget -= count
        return chunks

    def schedule_steady_decode(self) -> list[SequenceState] | None:
        """If the next step is plain decoding — nobody waits, every running request has exactly
        its last token pending (or already has all the tokens it may generate) and the pages for
        one more token each are free — reserve those pages and return the requests to run.
        Otherwise change nothing and return None: the caller takes the general path.  It looks
        at token counts only, never at token values, so it can run before the host has seen the
        tokens of the step before."""
        if self.waiting or not self.running or len(self.running) > self.max_num_batched_tokens:
            return None
        rows = []
        for seq in self.running:
            if seq.num_generated >= seq.request.sampling_params.max_tokens:
                continue                          # complete by length: finishes when its ids arrive
            if seq.num_pending_tokens != 1:
                return None
            rows.append(seq)
        need = [0] * len(self.cache.groups)
        short = []
        for seq in rows:
            pages = self.cache.pages_needed(seq.request_id, seq.num_computed_tokens + 1)
            if not any(pages):
                continue
            short.append(seq)
            for g, n in enumerate(pages):
                need[g] += n
        if any(n > group.pool.num_free for n, group in zip(need, self.cache.groups)):
            return None
        for seq in short:
            ok = self.cache.reserve(seq.request_id, seq.num_computed_tokens + 1)
            assert ok
        return rows

    @staticmethod
    def _chunk(seq: SequenceState, count: int) -> ScheduledChunk:
        start = seq.num_computed_tokens
        return ScheduledChunk(seq, start, count, samples=start + count == seq.num_tokens)

    def _claim_pages(self, seq: SequenceState, count: int, chunks: list[ScheduledChunk]) -> bool:
        """Reserve pages for ``count`` more tokens of a running request, preempting the newest
        other running request while the pool is short.  False if ``seq`` itself had to go."""
        target = seq.num_computed_tokens + count
        while not self.cache.reserve(seq.request_id, target):
            victim = self._newest_running_other_than(seq)
            if victim is None:
                self._preempt(seq)
                return False
            self._preempt(victim)
            chunks[:] = [c for c in chunks if c.seq is not victim]
        return True

    def _newest_running_other_than(self, seq: SequenceState) -> SequenceState | None:
        for cand in reversed(self.running):
            if cand is not seq and cand.status == SequenceStatus.RUNNING:
                return cand
        return None

    def _preempt(self, seq: SequenceState) -> None:
        self.cache.release(seq.request_id)
        seq.num_computed_tokens = 0
        seq.status = SequenceStatus.WAITING
        self.running.remove(seq)
        self.waiting.appendleft(seq)
        self.num_preemptions += 1

    # ---- end of a request --------------------------------------------------------------------
    def finish(self, seq: SequenceState, reason: str) -> None:
        seq.status = SequenceStatus.FINISHED
        seq.finish_reason = reason
        if self.cache.has(seq.request_id):
            self.cache.release(seq.request_id)
        if seq in self.running:
            self.running.remove(seq)

    def cancel_by_id(self, request_id: str) -> bool:
        for seq in self.running:
            if seq.request_id == request_id:
                self.finish(seq, "cancelled")
                return True
        for seq in list(self.waiting):
            if seq.request_id == request_id:
                self.waiting.remove(seq)
                seq.status = SequenceStatus.FINISHED
                seq.finish_reason = "cancelled"
                return True
        return False
