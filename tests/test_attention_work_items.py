"""The work list of the tiled prompt attention (host logic, no GPU): every token row lies in
exactly one run of one request, a run's items are its key chunks in order, and the longest items
come first."""

from __future__ import annotations

import random

import pytest

from mini_gpt_inference_b200.kernels.attention_plan import KEY_CHUNK, QUERY_TILE, query_tiles


def _check(q_lens, ctx_befores, slots=None):
    items = query_tiles(q_lens, ctx_befores, slots)
    starts = [sum(q_lens[:r]) for r in range(len(q_lens))]
    covered = [0] * sum(q_lens)
    runs = {}
    for r, row0, rows, chunk, chunks in items:
        assert 0 <= r < len(q_lens) and 1 <= rows <= QUERY_TILE and 0 <= chunk < chunks
        assert starts[r] <= row0 and row0 + rows <= starts[r] + q_lens[r], "a run stays inside its request"
        runs.setdefault((r, row0, rows, chunks), []).append(chunk)
    for (r, row0, rows, chunks), seen in runs.items():
        assert seen == list(range(chunks)), "the chunks of a run are consecutive items, chunk 0 first"
        for i in range(row0, row0 + rows):
            covered[i] += 1
        keys = ctx_befores[r] + (row0 - starts[r]) + rows          # positions 0 .. the run's last token
        assert chunks == 1 or -(-keys // chunks) <= 2 * KEY_CHUNK, "no item walks over more than twice KEY_CHUNK keys"
        if slots is None:
            assert chunks == max(1, -(-keys // KEY_CHUNK))
    assert covered == [1] * sum(q_lens), "every token row belongs to exactly one run"
    # items of one run are adjacent in the list
    order = [(r, row0) for r, row0, _, _, _ in items]
    firsts = [i for i, key in enumerate(order) if i == 0 or order[i - 1] != key]
    assert len(firsts) == len(runs)
    return items


def test_single_tokens_and_short_prompts():
    assert query_tiles([1], [0]) == [(0, 0, 1, 0, 1)]
    items = _check([1, 1, 1], [5, 700, 0])
    assert sorted(i[:3] for i in items if i[3] == 0) == [(0, 0, 1), (1, 1, 1), (2, 2, 1)]
    assert [i for i in items if i[0] == 1] == [(1, 1, 1, 0, 2), (1, 1, 1, 1, 2)]      # 701 keys: two chunks
    assert _check([], []) == []


def test_a_long_prompt_is_cut_into_tiles_and_key_chunks():
    items = _check([2048], [0])
    assert len({(row0, rows) for _, row0, rows, _, _ in items}) == 2048 // QUERY_TILE
    last = [i for i in items if i[1] == 2048 - QUERY_TILE]
    assert len(last) == 2048 // KEY_CHUNK                            # the last tile sees all 2048 keys


def test_longest_items_first():
    items = _check([300, 1, 40], [0, 1500, 200])
    starts = [0, 300, 301]

    def per_item(it):
        r, row0, rows, _, chunks = it
        keys = [0, 1500, 200][r] + (row0 - starts[r]) + rows
        return keys / chunks
    sizes = [per_item(it) for it in items]
    assert all(a >= b - 1e-9 for a, b in zip(sizes, sizes[1:]))


@pytest.mark.parametrize("seed", range(20))
def test_random_batches(seed):
    rng = random.Random(seed)
    n = rng.randint(1, 6)
    q_lens = [rng.choice([1, 1, 2, 7, 64, 128, 129, 300, 1000]) for _ in range(n)]
    ctx = [rng.choice([0, 0, 1, 63, 511, 512, 513, 1500, 4000]) for _ in range(n)]
    _check(q_lens, ctx)
    _check(q_lens, ctx, slots=rng.choice([1, 8, 37, 296]))
