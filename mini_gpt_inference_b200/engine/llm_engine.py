"""The Python entry point: ``LLMEngine`` with ``add_request`` / ``step`` / ``generate``.

Names and meanings follow the reference's engine (src/minigpt_infer/engine/engine.py:42-118):
``add_request(Request)``, ``step() -> list[RequestOutput]``, ``has_unfinished_requests()``,
``cancel_request(id)``; finish reasons ``"eot" | "length" | "stop" | "cancelled"`` checked in
the reference's order, end-of-text before length (src/minigpt_infer/engine/engine.py:186-194).
A request is refused when it is added if its prompt plus ``max_tokens`` would run past the
position table (src/minigpt_infer/engine/engine.py:69-88).  ``generate`` is a convenience the
reference's engine lacks (its ``generation.py`` has one for the static cache only).

The engine works on token ids (the reference's tokenizer needs files from the network).  Stop
conditions are token ids (``stop_token_ids``); with a ``token_bytes`` function from the caller's
tokenizer the engine also streams text (``RequestOutput.text_delta``) and honours stop strings
(``SamplingParams.stop``), see ``text.py``.  Without it a request that sets ``stop`` is refused.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Sequence

import torch

from ..config.engine_config import EngineConfig, SamplingParams
from ..sampling.sampler import Sampler
from .build import LoadedModel, load_model, make_runner
from .request import Request, RequestOutput, SequenceState
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler
from .text import IncrementalText, cut_at_stop


@dataclass
class _InFlight:
    """A decoding step whose sampled ids are still on their way to the host."""

    seqs: list                 # the requests of the step, in row order
    ids_device: Any            # int32 ids on the device (input of the next step)
    ids_host: Any              # pinned copy in progress
    ready: Any                 # event recorded after the copy
    status_host: Any = None    # pinned copy of the kernels' status word, taken with the ids


class LLMEngine:
    def __init__(self, loaded: LoadedModel, engine_cfg: EngineConfig | None = None, ops=None,
                 vocab_limit: int | None = None, seed: int = 0, token_bytes=None) -> None:
        self.engine_cfg = engine_cfg or EngineConfig()
        self.token_bytes = token_bytes                  # token id -> bytes, or None (ids only)
        self._texts: dict[str, IncrementalText] = {}
        if ops is None:
            from ..kernels.ops import default_ops

            ops = default_ops(loaded.device)
        self.loaded = loaded
        self.config = loaded.config
        self.runner: ModelRunner = make_runner(
            loaded, ops, self.engine_cfg.block_size, self.engine_cfg.num_blocks,
            self.engine_cfg.max_batch_size, self.engine_cfg.use_cuda_graphs,
            max_step_tokens=self.engine_cfg.prefill_chunk)
        self.scheduler = Scheduler(self.runner.manager, self.engine_cfg.max_batch_size,
                                   self.engine_cfg.max_num_batched_tokens,
                                   self.engine_cfg.prefill_chunk)
        self.sampler = Sampler(ops, loaded.device, vocab_limit, seed)
        self.runner.greedy_vocab_limit = vocab_limit     # before the first decode step is captured
        self.max_context = self.runner.max_context
        self._sequences: dict[str, SequenceState] = {}
        # Steady decoding overlaps the host with the device: a step is launched with the tokens
        # of the step before still on the device, and that step's ids are read while this one
        # runs.  What step() returns then lags one step behind what the device has computed.
        self._overlap = (self.engine_cfg.overlap_decode and loaded.device.type == "cuda"
                         and self.runner.use_cuda_graphs)
        self._inflight: _InFlight | None = None
        self._held_outputs: list[RequestOutput] = []
        self._pinned_ids = [None, None]
        # The kernels' status word (non-zero after a bounded wait ran out) travels to the host with
        # every step's ids and is checked where the ids are read.
        self._watch_status = hasattr(ops, "status_to_host")
        self._pinned_status = [None, None]
        self.num_overlapped_steps = 0
        self.num_steps = 0
        self.num_tokens_run = 0
        self.num_tokens_generated = 0

    @classmethod
    def from_pretrained(cls, model_dir: str | Path, engine_cfg: EngineConfig | None = None,
                        **kwargs) -> "LLMEngine":
        engine_cfg = engine_cfg or EngineConfig()
        loaded = load_model(model_dir, dtype=engine_cfg.dtype, device=engine_cfg.device)
        return cls(loaded, engine_cfg, **kwargs)

    # ---- requests ---------------------------------------------------------------------------
    def warm_up(self) -> dict:
        """Optional, before the first request: capture the CUDA graphs of decode batches of every
        size up to ``max_batch_size`` now instead of when such a batch first forms.  Nothing else
        changes; an engine that is never warmed up captures each graph at its first use."""
        made = self.runner.capture_decode_graphs(self.engine_cfg.max_batch_size)
        return {"decode_graphs_captured": made}

    def add_request(self, request: Request) -> None:
        prompt_len = len(request.prompt_token_ids)
        if prompt_len == 0:
            raise ValueError(f"request {request.request_id!r} has an empty prompt")
        if request.request_id in self._sequences:
            raise ValueError(f"request id {request.request_id!r} is already in use")
        vocab = self.runner.vocab_size
        bad = [t for t in request.prompt_token_ids if not (0 <= t < vocab)]
        if bad:
            raise ValueError(f"request {request.request_id!r}: token id {bad[0]} is outside the "
                             f"vocabulary (0..{vocab - 1})")
        longest = prompt_len + request.sampling_params.max_tokens
        if longest > self.max_context:
            raise ValueError(
                f"prompt_len ({prompt_len}) + max_tokens ({request.sampling_params.max_tokens}) "
                f"= {longest} > {self.max_context}; this request can never finish without "
                "running past the position table")
        if request.sampling_params.stop and self.token_bytes is None:
            raise ValueError(
                f"request {request.request_id!r} sets stop strings, but the engine was given no "
                "token_bytes function to turn ids into text; use stop_token_ids, or construct "
                "the engine with token_bytes=")
        if self.token_bytes is not None:
            self._texts[request.request_id] = IncrementalText(self.token_bytes)
        seed = request.sampling_params.seed
        seq = SequenceState(request=request,
                            seed=self.sampler.fresh_seed() if seed is None else int(seed))
        self.scheduler.add_request(seq)
        self._sequences[request.request_id] = seq

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None or bool(self._held_outputs)

    def cancel_request(self, request_id: str) -> bool:
        # What is still on its way from the device is read first; the next step() returns it
        # (the cancelled request's own last token included, as it was generated before the call).
        self._held_outputs.extend(self._drain())
        self._sequences.pop(request_id, None)
        self._texts.pop(request_id, None)
        return self.scheduler.cancel_by_id(request_id)

    # ---- one step ---------------------------------------------------------------------------
    def step(self) -> list[RequestOutput]:
        """Advance by one step and return what became known: one RequestOutput per request whose
        next token the host has read.  In steady decoding these are the tokens of the step before
        the one just launched."""
        held, self._held_outputs = self._held_outputs, []
        return held + self._step()

    def _step(self) -> list[RequestOutput]:
        if self._overlap:
            rows = self.scheduler.schedule_steady_decode()
            if rows is not None and self.runner.can_feed_tokens_on_device(len(rows)):
                return self._step_overlapped(rows)
            # (pages that the attempt reserved stay with their requests; the general path
            # reserves the same ones again, which changes nothing)
        outputs = self._drain()
        return outputs + self._step_general()

    def _step_overlapped(self, rows: list[SequenceState]) -> list[RequestOutput]:
        previous = self._inflight
        if not rows:                                    # everybody is complete by length
            return self._drain()
        source_row = {id(s): i for i, s in enumerate(previous.seqs)} if previous else {}
        entries, sources = [], []
        for seq in rows:
            if seq.num_inflight:
                entries.append(StepEntry(seq.request_id, [0], [0]))     # the token is on the device
                sources.append(source_row[id(seq)])
            else:
                entries.append(StepEntry(seq.request_id, [seq.token_at(seq.num_computed_tokens)], [0]))
                sources.append(-1)
        logits = self.runner.step(entries, copy=False, token_sources=sources,
                                  previous_ids=previous.ids_device if previous else None)
        self.num_steps += 1
        self.num_overlapped_steps += 1
        self.num_tokens_run += len(rows)
        # ids go where the next step's graph looks for its tokens; greedy rows are there already
        ids = self.sampler.sample(
            logits, [s.request.sampling_params for s in rows], [s.seed for s in rows],
            [s.num_generated for s in rows], greedy_ids=self.runner.greedy_ids(len(rows)),
            out=self.runner.sampled_ids[: len(rows)])
        slot = self.num_steps % 2
        if self._pinned_ids[slot] is None or self._pinned_ids[slot].numel() < len(rows):
            self._pinned_ids[slot] = torch.empty(max(len(rows), self.engine_cfg.max_batch_size),
                                                 dtype=torch.int32, pin_memory=True)
        host = self._pinned_ids[slot][: len(rows)]
        host.copy_(ids, non_blocking=True)
        status_host = None
        if self._watch_status:
            status_host = self._pinned_status[slot] = self.runner.ops.status_to_host(self._pinned_status[slot])
        ready = torch.cuda.Event()
        ready.record()
        for seq in rows:
            seq.num_computed_tokens += 1
            seq.num_inflight += 1
        self._inflight = _InFlight(rows, ids, host, ready, status_host)
        # while the device runs this step, read the ids of the step before
        return self._process(previous) if previous else []

    def _process(self, flight: _InFlight) -> list[RequestOutput]:
        """The ids of an earlier step have arrived (or are waited for): record them."""
        flight.ready.synchronize()
        if flight.status_host is not None:
            self.runner.ops.raise_on_status(flight.status_host)
        outputs = []
        for seq, token in zip(flight.seqs, flight.ids_host.tolist()):
            if seq.is_finished():
                continue                                # it ended a step earlier; this token is dropped
            seq.num_inflight -= 1
            outputs.append(self._record(seq, int(token)))
        return outputs

    def _drain(self) -> list[RequestOutput]:
        """Read the ids that are still on their way, so that the host knows every token."""
        if self._inflight is None:
            return []
        flight, self._inflight = self._inflight, None
        return self._process(flight)

    def _step_general(self) -> list[RequestOutput]:
        chunks = self.scheduler.schedule()
        if not chunks:
            return []
        entries = [StepEntry(c.seq.request_id, c.seq.tokens(c.start, c.count),
                             [c.count - 1] if c.samples else []) for c in chunks]
        logits = self.runner.step(entries, copy=False)      # sampled before the next step
        self.num_steps += 1
        self.num_tokens_run += sum(c.count for c in chunks)
        for c in chunks:
            c.seq.num_computed_tokens += c.count
        sampled = [c.seq for c in chunks if c.samples]
        if not sampled:
            return []
        ids = self.sampler.sample(
            logits, [s.request.sampling_params for s in sampled], [s.seed for s in sampled],
            [len(s.output_token_ids) for s in sampled])
        status_host = None
        if self._watch_status:
            status_host = self._pinned_status[0] = self.runner.ops.status_to_host(self._pinned_status[0])
        ids = ids.tolist()                                   # waits for the step, the status copy included
        if status_host is not None:
            self.runner.ops.raise_on_status(status_host)
        outputs = []
        for seq, token in zip(sampled, ids):
            outputs.append(self._record(seq, int(token)))
        return outputs

    def _record(self, seq: SequenceState, token: int) -> RequestOutput:
        """A request's next token has reached the host: append it, extend its text, and end the
        request if a finish condition holds."""
        seq.output_token_ids.append(token)
        self.num_tokens_generated += 1
        text = self._texts.get(seq.request_id)
        delta = text.add_token(token) if text is not None else ""
        reason = self._check_finish(seq, token, text.text if text is not None else "")
        whole = None
        if reason is not None:
            if text is not None:
                delta += text.finalize()
                whole = text.text
                delta, stop = cut_at_stop(whole, delta, seq.request.sampling_params.stop)
                if stop is not None:
                    reason, whole = "stop", whole[: whole.find(stop)]
            self.scheduler.finish(seq, reason)
            self._sequences.pop(seq.request_id, None)
            self._texts.pop(seq.request_id, None)
        return RequestOutput(seq.request_id, [token], delta, seq.is_finished(), seq.finish_reason, whole)

    @staticmethod
    def _check_finish(seq: SequenceState, token: int, text: str = "") -> str | None:
        request = seq.request
        params = request.sampling_params
        if request.eot_token_id is not None and token == request.eot_token_id:
            return "eot"
        if len(seq.output_token_ids) >= params.max_tokens:
            return "length"
        if params.stop_token_ids and token in params.stop_token_ids:
            return "stop"
        if params.stop and text:
            for stop in params.stop:
                if stop and stop in text:
                    return "stop"
        return None

    # ---- convenience ------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
                 eot_token_id: int | None = None) -> list[dict]:
        """Run the prompts to completion.  Returns, in the order of the prompts, dicts with
        ``token_ids`` (generated only), ``finish_reason`` and ``text`` (empty without a
        ``token_bytes`` function)."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = []
        for i, (prompt, params) in enumerate(zip(prompts, sampling_params)):
            rid = f"gen-{self.num_steps}-{i}-{len(self._sequences)}"
            self.add_request(Request(rid, list(prompt), params, eot_token_id))
            ids.append(rid)
        results = {rid: {"token_ids": [], "finish_reason": None, "text": ""} for rid in ids}
        while self.has_unfinished_requests():
            for out in self.step():
                if out.request_id in results:
                    results[out.request_id]["token_ids"].extend(out.new_token_ids)
                    results[out.request_id]["text"] += out.text_delta
                    if out.text is not None:
                        results[out.request_id]["text"] = out.text
                    if out.finished:
                        results[out.request_id]["finish_reason"] = out.finish_reason
        return [results[rid] for rid in ids]

    def stats(self) -> dict:
        out = dict(self.runner.manager.stats())
        out.update(steps=self.num_steps, overlapped_steps=self.num_overlapped_steps,
                   tokens_run=self.num_tokens_run,
                   tokens_generated=self.num_tokens_generated,
                   preemptions=self.scheduler.num_preemptions,
                   running=len(self.scheduler.running), waiting=len(self.scheduler.waiting))
        return out
