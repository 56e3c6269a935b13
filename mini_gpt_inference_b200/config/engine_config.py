"""Engine and sampling parameters.

``EngineConfig`` keeps the reference's names and meanings
(src/minigpt_infer/config.py:21-29: ``block_size`` = tokens per KV page,
``num_blocks`` = pages in the fixed pool, ``max_batch_size`` = most running
requests) and adds what the reference has no notion of: a token budget per step,
a largest prompt portion, and the compute dtype.

``SamplingParams`` is the reference's (src/minigpt_infer/config.py:32-41);
unlike the reference, ``seed`` is honoured (per-request counter-based RNG).
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class EngineConfig:
    block_size: int = 16                 # tokens per KV page
    num_blocks: int = 2048               # pages in the pool (per cache group)
    max_batch_size: int = 256            # most running requests
    max_num_batched_tokens: int = 2048   # token budget of one step
    max_prefill_chunk: int | None = None # largest prompt portion; None = the budget
    dtype: str = "bfloat16"              # "bfloat16" | "float32"
    device: str = "cuda:0"
    use_cuda_graphs: bool = True         # replay decode-only steps from CUDA graphs
    overlap_decode: bool = True          # in steady decoding, feed sampled tokens back on the device
                                         # and read their ids one step late (outputs lag by a step)

    def __post_init__(self) -> None:
        if self.block_size <= 0 or self.num_blocks <= 0:
            raise ValueError("block_size and num_blocks must be positive")
        if self.max_batch_size <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_batch_size and max_num_batched_tokens must be positive")
        if self.max_prefill_chunk is not None and self.max_prefill_chunk <= 0:
            raise ValueError("max_prefill_chunk must be positive when given")
        self.dtype = canonical_dtype(self.dtype)

    @property
    def prefill_chunk(self) -> int:
        if self.max_prefill_chunk is None:
            return self.max_num_batched_tokens
        return min(self.max_prefill_chunk, self.max_num_batched_tokens)


def canonical_dtype(name: str) -> str:
    table = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32",
             "float32": "float32", "float": "float32"}
    key = str(name).replace("torch.", "").lower()
    if key not in table:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")
    return table[key]


@dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 1.0             # 0.0 => greedy
    top_k: int | None = None
    top_p: float | None = None
    repetition_penalty: float = 1.0      # accepted; not applied (as in the reference engine)
    stop: list[str] = field(default_factory=list)   # stop strings: honoured by an engine that was given
                                                    # token_bytes=, refused by an ids-only engine
    seed: int | None = None
    n: int = 1
    stop_token_ids: list[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if self.n != 1:
            # src/minigpt_infer/engine/engine.py:70 asserts the same.
            raise ValueError("n > 1 completions per request are not supported")
        if self.top_k is not None and self.top_k <= 0:
            raise ValueError("top_k must be positive when given")
        if self.top_p is not None and not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1] when given")
