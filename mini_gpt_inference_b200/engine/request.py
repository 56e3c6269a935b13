"""What a caller asks for and what the engine keeps about it.

As in the reference (src/minigpt_infer/engine/request.py:20-75): an immutable ``Request``,
a mutable ``SequenceState`` whose ``num_computed_tokens`` counts the tokens that are in the
cache, and a ``RequestOutput`` per step.  No torch in this module.
"""

from __future__ import annotations

from array import array
from dataclasses import dataclass, field
from enum import Enum, auto

import numpy as np

from ..config.engine_config import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    eot_token_id: int | None = None


@dataclass
class SequenceState:
    request: Request
    output_token_ids: list[int] = field(default_factory=list)
    status: SequenceStatus = SequenceStatus.WAITING
    # Tokens whose keys and values are in the cache.  The next token to run is always the one
    # at this position (src/minigpt_infer/engine/request.py:40-45).
    num_computed_tokens: int = 0
    finish_reason: str | None = None
    seed: int = 0
    arrival: int = 0
    # Tokens sampled on the device whose ids the host has not read yet (0 or 1): they count as
    # generated for scheduling, their values arrive one step later.
    num_inflight: int = 0
    # The prompt as an int32 array, made when a portion of it is first asked for: portions are
    # then views, and a long prompt is converted once instead of once per portion.
    _prompt_array: np.ndarray | None = field(default=None, repr=False, compare=False)

    @property
    def request_id(self) -> str:
        return self.request.request_id

    @property
    def prompt_len(self) -> int:
        return len(self.request.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        """Prompt plus everything generated so far (tokens still on their way from the device
        included)."""
        return self.prompt_len + len(self.output_token_ids) + self.num_inflight

    @property
    def num_generated(self) -> int:
        return len(self.output_token_ids) + self.num_inflight

    @property
    def num_pending_tokens(self) -> int:
        """Tokens not yet in the cache: one in steady decoding, more while a prompt (or a
        recomputation after preemption) is under way."""
        return self.num_tokens - self.num_computed_tokens

    def token_at(self, i: int) -> int:
        p = self.prompt_len
        return self.request.prompt_token_ids[i] if i < p else self.output_token_ids[i - p]

    def tokens(self, start: int, count: int):
        """``count`` tokens from position ``start`` of prompt + generated, without building
        the whole list (a decoding step asks for one token of a long sequence)."""
        p = self.prompt_len
        end = start + count
        if end <= p:
            if count > 16:
                if self._prompt_array is None:
                    try:
                        self._prompt_array = np.frombuffer(array("i", self.request.prompt_token_ids), dtype=np.int32)
                    except (OverflowError, TypeError):       # the step function names the bad id
                        return self.request.prompt_token_ids[start:end]
                return self._prompt_array[start:end]
            return self.request.prompt_token_ids[start:end]
        if start >= p:
            return self.output_token_ids[start - p: end - p]
        return self.request.prompt_token_ids[start:] + self.output_token_ids[: end - p]

    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED


@dataclass
class RequestOutput:
    request_id: str
    new_token_ids: list[int]
    text_delta: str = ""
    finished: bool = False
    finish_reason: str | None = None
    # On the output that finishes a request of an engine that makes text: the request's whole text,
    # ending where a stop string begins.  (The deltas are handed out as they come; the beginning of
    # a stop string that was spread over several tokens may already have gone out with them.)
    text: str | None = None


@dataclass
class ScheduledChunk:
    """A request's share of one step: ``count`` tokens from position ``start``; ``samples`` if
    the chunk ends at the request's last token, so that its logits give the next token."""

    seq: SequenceState
    start: int
    count: int
    samples: bool
