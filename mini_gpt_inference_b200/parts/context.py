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
    # work list of kernels that take tiles of queries: see query_tiles(); None if not built
    attn_work: torch.Tensor | None = None
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


QUERY_TILE = 128       # most consecutive tokens of one request in a tile
KEY_CHUNK = 512        # most key positions one work item walks over


def query_tiles(q_lens, ctx_befores, slots=None):
    """Cut a ragged batch into work items ``(request, first row, rows, chunk, chunks)``.

    The tokens of each request are cut into runs of at most QUERY_TILE rows.  The keys a run
    may see (positions 0 .. its last token) are cut into ``chunks`` parts of at most KEY_CHUNK
    positions, one work item each, so that a long context is spread over several CTAs; their
    partial results are merged afterwards.  Items of one run are consecutive, chunk 0 first; the
    runs come longest item first, so that when the grid does not fit the GPU at once, the CTAs
    that start last are the short ones.

    ``slots``: how many work items the GPU runs at once (per head).  If the items exceed it by
    less than half, longer parts (up to twice KEY_CHUNK) are tried, so that a second round of a
    few CTAs is not added to the first."""

    runs = []                                     # (request, first row, rows, keys it may see)
    row = 0
    for r, (n, before) in enumerate(zip(q_lens, ctx_befores)):
        for b in range(0, n, QUERY_TILE):
            rows = min(QUERY_TILE, n - b)
            runs.append((r, row + b, rows, before + b + rows))
        row += n

    def count(limit):
        return sum(max(1, -(-keys // limit)) for _, _, _, keys in runs)

    limit = KEY_CHUNK
    items = count(limit)
    if slots and slots < items <= slots + slots // 2:
        for longer in range(KEY_CHUNK + QUERY_TILE, 2 * KEY_CHUNK + 1, QUERY_TILE):
            if count(longer) <= slots:
                limit = longer
                break
    cut = []
    for i, (r, row0, rows, keys) in enumerate(runs):
        chunks = max(1, -(-keys // limit))
        cut.append((-(keys / chunks), i, r, row0, rows, chunks))
    cut.sort()
    return [(r, row0, rows, c, chunks) for _, _, r, row0, rows, chunks in cut for c in range(chunks)]
