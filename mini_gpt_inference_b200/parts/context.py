"""The batch one step runs on, as the parts see it.

Tokens of all requests lie flat, request after request (``N`` rows).  A request brings
``q_len`` new tokens that follow ``ctx_before`` tokens already in the cache; a single
decoded token and a portion of a prompt differ in nothing but ``q_len``.  The reference
has rectangular ``(B, T)`` batches that are either all prompts or all single tokens
(src/minigpt_infer/batch.py:19-64); this flat form is what lets one step mix them.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass
class HostBatch:
    """The batch of a step as the host knows it before anything is on the device: what a part's
    ``plan_step`` sees."""

    q_len: list                            # per request: tokens it brings
    ctx_before: list                       # per request: tokens already in the cache
    state_slot: list                       # per request: its slot of the state pool
    act_dtype: Any = None

    @property
    def num_tokens(self) -> int:
        return sum(self.q_len)

    @property
    def decode_only(self) -> bool:
        return all(n == 1 for n in self.q_len)

    @property
    def max_ctx_after(self) -> int:
        return max(a + b for a, b in zip(self.q_len, self.ctx_before))


@dataclass
class StepPlan:
    """What parts prepare on the host for one step.  ``arrays``: int32 numpy arrays by name; the
    step function packs them into the step's one upload and hands them to the parts as
    ``ctx.extra[name]`` (same shape, on the device).  Parts that would plan the same thing share
    a name, and the second one finds it there.  ``signature``: anything else that decides which
    kernels a part launches with which sizes (a step is replayed from a captured graph only if
    the token counts, the shapes of the arrays and the signature all repeat)."""

    arrays: dict = field(default_factory=dict)
    signature: list = field(default_factory=list)


@dataclass
class StepContext:
    ops: Any                              # the kernel set the parts call
    act_dtype: torch.dtype                # compute dtype between norm and projection
    num_tokens: int
    num_requests: int
    # device, int32
    token_ids: torch.Tensor               # [N]
    positions: torch.Tensor               # [N] absolute position of each token
    token_request: torch.Tensor           # [N] index of the token's request in this batch
    req_q_start: torch.Tensor             # [R] first row of the request
    req_q_len: torch.Tensor               # [R] new tokens of the request
    req_ctx_before: torch.Tensor          # [R] tokens in the cache before this step
    req_state_slot: torch.Tensor          # [R] slot of the state pool
    block_tables: list[torch.Tensor]      # per cache group [R, max_pages], -1 = no page
    slot_mapping: list[torch.Tensor]      # per cache group [N] flat row of each new token
    logit_rows: torch.Tensor              # [W] rows whose logits are wanted
    # What parts planned for this step on the host (``Part.plan_step``): int32 tensors by name.
    extra: dict = field(default_factory=dict)
    # Optional: where token_source[i] >= 0, token i is fed_ids[token_source[i]] (a token the step
    # before sampled, still on the device) instead of token_ids[i].
    token_source: torch.Tensor | None = None
    fed_ids: torch.Tensor | None = None
    # Optional: where the head may leave the argmax of every logits row (ids at or above
    # greedy_vocab_limit excluded); it sets greedy_taken if it did.
    greedy_out: torch.Tensor | None = None
    greedy_vocab_limit: int | None = None
    greedy_taken: bool = False
    # host mirrors for parts that plan on the host
    host_q_len: list[int] = field(default_factory=list)
    host_ctx_before: list[int] = field(default_factory=list)
    host_state_slot: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_after: int = 0                # longest context once this step's tokens are in
    decode_only: bool = False             # every request brings exactly one token
    storage: Any = None                   # cache.storage.CacheStorage

    def cache_view(self, cache_layer: int, writes: bool = True):
        return self.storage.layer_view(cache_layer, writes) if self.storage is not None else None
