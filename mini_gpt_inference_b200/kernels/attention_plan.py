"""The work list of the tiled prompt-attention kernel: which CTA takes which queries and keys.

It belongs to the kernel (its tile sizes and how many of its CTAs the GPU runs at once decide
the cut); the attention mixer asks for it through ``CudaOps.plan_prompt_attention`` from its
``plan_step`` hook, and the step function carries it to the device with the step's other integers.
"""

from __future__ import annotations

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
