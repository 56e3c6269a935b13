"""The Python entry point: ``LLMEngine`` with ``add_request`` / ``step`` / ``generate``.

Names and meanings follow the reference's engine (src/minigpt_infer/engine/engine.py:42-118):
``add_request(Request)``, ``step() -> list[RequestOutput]``, ``has_unfinished_requests()``,
``cancel_request(id)``; finish reasons ``"eot" | "length" | "stop" | "cancelled"`` checked in
the reference's order, end-of-text before length (src/minigpt_infer/engine/engine.py:186-194).
A request is refused when it is added if its prompt plus ``max_tokens`` would run past the
position table (src/minigpt_infer/engine/engine.py:69-88).  ``generate`` is a convenience the
reference's engine lacks (its ``generation.py`` has one for the static cache only).

The engine works on token ids; text is the caller's business (the reference's tokenizer needs
files from the network).  Stop conditions are therefore token ids (``stop_token_ids``).
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from ..config.engine_config import EngineConfig, SamplingParams
from ..sampling.sampler import Sampler
from .build import LoadedModel, load_model, make_runner
from .request import Request, RequestOutput, SequenceState
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler


class LLMEngine:
    def __init__(self, loaded: LoadedModel, engine_cfg: EngineConfig | None = None, ops=None,
                 vocab_limit: int | None = None, seed: int = 0) -> None:
        self.engine_cfg = engine_cfg or EngineConfig()
        if ops is None:
            from ..kernels.ops import default_ops

            ops = default_ops(loaded.device)
        self.loaded = loaded
        self.config = loaded.config
        self.runner: ModelRunner = make_runner(
            loaded, ops, self.engine_cfg.block_size, self.engine_cfg.num_blocks,
            self.engine_cfg.max_batch_size, self.engine_cfg.use_cuda_graphs)
        self.scheduler = Scheduler(self.runner.manager, self.engine_cfg.max_batch_size,
                                   self.engine_cfg.max_num_batched_tokens,
                                   self.engine_cfg.prefill_chunk)
        self.sampler = Sampler(ops, loaded.device, vocab_limit, seed)
        self.max_context = self.runner.max_context
        self._sequences: dict[str, SequenceState] = {}
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
        seed = request.sampling_params.seed
        seq = SequenceState(request=request,
                            seed=self.sampler.fresh_seed() if seed is None else int(seed))
        self.scheduler.add_request(seq)
        self._sequences[request.request_id] = seq

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_work()

    def cancel_request(self, request_id: str) -> bool:
        self._sequences.pop(request_id, None)
        return self.scheduler.cancel_by_id(request_id)

    # ---- one step ---------------------------------------------------------------------------
    def step(self) -> list[RequestOutput]:
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
            [len(s.output_token_ids) for s in sampled]).tolist()
        outputs = []
        for seq, token in zip(sampled, ids):
            seq.output_token_ids.append(int(token))
            self.num_tokens_generated += 1
            reason = self._check_finish(seq, int(token))
            if reason is not None:
                self.scheduler.finish(seq, reason)
                self._sequences.pop(seq.request_id, None)
            outputs.append(RequestOutput(seq.request_id, [int(token)], "", seq.is_finished(),
                                         seq.finish_reason))
        return outputs

    @staticmethod
    def _check_finish(seq: SequenceState, token: int) -> str | None:
        params = seq.request.sampling_params
        if seq.request.eot_token_id is not None and token == seq.request.eot_token_id:
            return "eot"
        if len(seq.output_token_ids) >= params.max_tokens:
            return "length"
        if token in params.stop_token_ids:
            return "stop"
        return None

    # ---- convenience ------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
                 eot_token_id: int | None = None) -> list[dict]:
        """Run the prompts to completion.  Returns, in the order of the prompts, dicts with
        ``token_ids`` (generated only) and ``finish_reason``."""
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
        results = {rid: {"token_ids": [], "finish_reason": None} for rid in ids}
        while self.has_unfinished_requests():
            for out in self.step():
                if out.request_id in results:
                    results[out.request_id]["token_ids"].extend(out.new_token_ids)
                    if out.finished:
                        results[out.request_id]["finish_reason"] = out.finish_reason
        return [results[rid] for rid in ids]

    def stats(self) -> dict:
        out = dict(self.runner.manager.stats())
        out.update(steps=self.num_steps, tokens_run=self.num_tokens_run,
                   tokens_generated=self.num_tokens_generated,
                   preemptions=self.scheduler.num_preemptions,
                   running=len(self.scheduler.running), waiting=len(self.scheduler.waiting))
        return out
