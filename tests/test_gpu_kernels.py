"""Each kernel alone against a plain 32-bit torch reference of the same operation, at sizes
other than the engine's tiny configurations: odd widths, tails of tiles, head sizes in steps
of 16, grouped heads, windows, page edges."""

from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

import plain_gpt

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from mini_gpt_inference_b200.kernels.ops import default_ops

    return default_ops("cuda:0")


def _tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def randn(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,vocab", [(96, 509), (520, 1000), (33, 77)])
def test_embed(ops, dtype, width, vocab):
    tok, pos = randn(vocab, width, dtype=dtype, seed=1), randn(300, width, dtype=dtype, seed=2)
    ids = torch.randint(0, vocab, (45,), dtype=torch.int32).cuda()
    positions = torch.randint(0, 300, (45,), dtype=torch.int32).cuda()
    got = ops.embed(ids, positions, tok, pos)
    want = tok.float()[ids.long()] + pos.float()[positions.long()]
    assert got.dtype == torch.float32 and torch.equal(got, want)
    assert torch.equal(ops.embed(ids, positions, tok, None), tok.float()[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps,bias", [(7, 96, 3e-4, False), (130, 520, 1e-5, True),
                                                 (1, 33, 1e-2, True), (64, 2048, 1e-5, True)])
def test_layernorm(ops, dtype, rows, width, eps, bias):
    x = randn(rows, width, seed=3, scale=3.0) + 1.5          # a mean far from zero
    gain = randn(width, seed=4) + 1.0
    shift = randn(width, seed=5) if bias else None
    got = ops.layernorm(x, gain, shift, eps, dtype)
    want = F.layer_norm(x.double(), (width,), gain.double(), None if shift is None else shift.double(), eps)
    assert got.dtype == dtype
    assert (got.double() - want).abs().max() <= _tol(dtype, 4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 509, 96), (45, 200, 96), (130, 96, 200), (64, 1536, 512),
                                   (3, 77, 33), (257, 65, 129), (8, 50304, 512), (300, 2048, 512),
                                   (2048, 512, 2048), (17, 1536, 512), (33, 512, 2048),
                                   (65, 1536, 512), (128, 128, 64), (129, 130, 72), (16, 16, 8)])
def test_linear_and_epilogues(ops, dtype, m, n, k):
    x = randn(m, k, dtype=dtype, seed=6)
    w = randn(n, k, dtype=dtype, seed=7, scale=1 / math.sqrt(k))
    b = randn(n, seed=8)
    ref = x.double() @ w.double().T
    assert (ops.linear(x, w, None, "none", dtype).double() - ref).abs().max() <= _tol(dtype, 3)
    assert (ops.linear(x, w, b, "none", dtype).double() - (ref + b.double())).abs().max() <= _tol(dtype, 3)
    gelu = plain_gpt.gelu_tanh(ref + b.double())
    assert (ops.linear(x, w, b, "gelu_tanh", dtype).double() - gelu).abs().max() <= _tol(dtype, 3)
    logits = ops.logits(x, w)
    assert logits.dtype == torch.float32
    assert (logits.double() - ref).abs().max() <= 2e-5        # inputs exact, 32-bit sums and output
    res = randn(m, n, seed=9)
    before = res.clone()
    ops.linear_residual(x, w, b, res)
    assert (res.double() - (before.double() + ref + b.double())).abs().max() <= 3e-5
    ops.check_status()


def test_tensor_core_and_cuda_core_products_agree(ops):
    """The tcgen05 path and the plain FMA path compute the same sums from the same bfloat16
    inputs; with 32-bit output they differ only by the order of the additions."""
    # (the last shape has enough tiles for the 128 x 256 variant of the tensor-core kernel)
    for m, n, k in [(5, 300, 512), (200, 136, 200), (64, 50304, 512), (1000, 1536, 512), (4200, 4800, 328)]:
        x = randn(m, k, dtype=torch.bfloat16, seed=11)
        w = randn(n, k, dtype=torch.bfloat16, seed=12, scale=1 / math.sqrt(k))
        ops.use_tensor_cores = True
        before = ops.launches
        fast = ops.logits(x, w)
        ops.use_tensor_cores = False
        slow = ops.logits(x, w)
        ops.use_tensor_cores = True
        assert ops.launches == before + 2
        assert (fast - slow).abs().max() <= 1e-5, (m, n, k)
    ops.check_status()


def test_tensor_core_tiles_of_256_columns_with_every_epilogue(ops):
    """Steps of thousands of tokens on a large matrix take tiles of 128 x 256: bias, GELU with a
    bfloat16 store, the residual add and the QKV projection's page write must come out as from the
    plain FMA kernel (the same bfloat16 inputs, sums in another order)."""
    m, k = 4300, 200
    n_head, n_kv, d, pt = 40, 20, 64, 16                    # 5120 columns: 34 x 20 tiles of 256
    n = (n_head + 2 * n_kv) * d
    x = randn(m, k, dtype=torch.bfloat16, seed=41)
    w = randn(n, k, dtype=torch.bfloat16, seed=42, scale=1 / math.sqrt(k))
    b = randn(n, seed=43)
    res = randn(m, n, seed=44)
    pages = -(-m // pt) + 2
    slots = torch.randperm(pages * pt)[:m].to(torch.int32)
    slots[7] = -1
    slots = slots.cuda()

    def run():
        cache = SimpleNamespace(k_pages=torch.zeros(pages, n_kv, pt, d, dtype=torch.bfloat16).cuda(),
                                v_pages=torch.zeros(pages, n_kv, pt, d, dtype=torch.bfloat16).cuda(),
                                page_tokens=pt, writes=True)
        r = res.clone()
        ops.linear_residual(x, w, b, r)
        return (ops.linear(x, w, b, "gelu_tanh", torch.bfloat16).float(), r,
                ops.linear_qkv(x, w, b, n_head, n_kv, d, cache, slots, torch.bfloat16).float(), cache)

    before = ops.launches
    fast = run()
    assert ops.launches == before + 3, "each call was expected to be one tensor-core launch"
    ops.use_tensor_cores = False
    try:
        slow = run()
    finally:
        ops.use_tensor_cores = True
    def one_bf16_step(a, c):
        # results rounded to bfloat16 may land on neighbouring values where a sum lies at a rounding
        # edge (a step is 2^-7 of the value's power of two), never further apart
        return bool(((a - c).abs() <= 2.0 ** -7 * c.abs().clamp(min=2.0 ** -6)).all())

    assert one_bf16_step(fast[0], slow[0])
    assert (fast[1] - slow[1]).abs().max() <= 1e-5          # 32-bit sums in another order
    assert one_bf16_step(fast[2], slow[2])
    for a, c in ((fast[3].k_pages, slow[3].k_pages), (fast[3].v_pages, slow[3].v_pages)):
        assert one_bf16_step(a.float(), c.float())
    # keys of token i lie where its slot says, bit for bit what the projection returned
    qkv = ops.linear_qkv(x, w, b, n_head, n_kv, d, fast[3], slots, torch.bfloat16)
    tok = 100
    s_ = int(slots[tok])
    assert torch.equal(fast[3].k_pages[s_ // pt, :, s_ % pt].reshape(-1), qkv[tok, n_head * d: (n_head + n_kv) * d])
    ops.check_status()


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 11, 16])
@pytest.mark.parametrize("n,k", [(1536, 512), (512, 2048), (509, 96), (50304, 512), (200, 200), (77, 40)])
def test_small_batch_projection_with_fused_norm(ops, m, n, k):
    """Up to 16 tokens take the weight-streaming kernel; with a deferred LayerNorm (and a row
    gather) fused into its prologue it must agree with the separate kernels."""
    x32 = randn(m + 3, k, seed=21, scale=2.0) + 0.5
    rows = torch.tensor([(3 * i + 1) % (m + 3) for i in range(m)], dtype=torch.int32).cuda()
    gain, shift = randn(k, seed=22) + 1.0, randn(k, seed=23)
    w = randn(n, k, dtype=torch.bfloat16, seed=24, scale=1 / math.sqrt(k))
    b = randn(n, seed=25)
    want = torch.nn.functional.layer_norm(x32[rows.long()].double(), (k,), gain.double(), shift.double(), 1e-5)
    want = want.to(torch.bfloat16).double() @ w.double().T + b.double()
    before = ops.launches
    fused = ops.linear(ops.defer_layernorm(x32, gain, shift, 1e-5, torch.bfloat16, rows), w, b, "none",
                       torch.float32)
    assert ops.launches == before + 1, "norm, gather and projection were expected in one kernel"
    assert (fused.double() - want).abs().max() <= 2e-2       # bf16 rounding of the normalised rows
    ops.use_skinny = False
    try:
        apart = ops.linear(ops.defer_layernorm(x32, gain, shift, 1e-5, torch.bfloat16, rows), w, b, "none",
                           torch.float32)
    finally:
        ops.use_skinny = True
    assert (fused - apart).abs().max() <= 2e-5               # same bf16 inputs, 32-bit sums
    res = randn(m, n, seed=26)
    keep = res.clone()
    y = ops.layernorm(ops.gather_rows(x32, rows), gain, shift, 1e-5, torch.bfloat16)
    ops.linear_residual(y, w, b, res)
    assert (res.double() - (keep.double() + want)).abs().max() <= 2e-2
    g = ops.linear(y, w, b, "gelu_tanh", torch.bfloat16)
    assert (g.double() - plain_gpt.gelu_tanh(want)).abs().max() <= 5e-2
    ops.check_status()


@pytest.mark.parametrize("m,c,f,bias", [(1, 512, 2048, True), (8, 512, 2048, True), (16, 512, 2048, True),
                                        (9, 512, 2048, False), (5, 96, 200, False), (3, 64, 256, True),
                                        (11, 768, 3072, True), (8, 1600, 6400, True), (2, 192, 520, True),
                                        (7, 40, 24, True), (16, 1024, 72, False)])
def test_whole_feed_forward_in_one_kernel(ops, m, c, f, bias):
    """LayerNorm, fc, tanh-GELU and proj of up to 16 tokens as one kernel that adds partial products
    of slices of the inner dimension into a zeroed buffer: against the formula (with the same
    roundings to bfloat16 as the two-kernel path) and against that path; three times in a row, so
    that the three buffers have taken every role."""
    x = randn(m, c, seed=41, scale=2.0) + 0.3
    gain, shift = randn(c, seed=42) + 1.0, (randn(c, seed=43) if bias else None)
    w1 = randn(f, c, dtype=torch.bfloat16, seed=44, scale=1 / math.sqrt(c))
    w2 = randn(c, f, dtype=torch.bfloat16, seed=45, scale=1 / math.sqrt(f))
    b1, b2 = (randn(f, seed=46), randn(c, seed=47)) if bias else (None, None)

    def formula(xin):
        y = F.layer_norm(xin.double(), (c,), gain.double(), None if shift is None else shift.double(), 1e-5)
        h = y.to(torch.bfloat16).double() @ w1.double().T + (b1.double() if bias else 0)
        h = plain_gpt.gelu_tanh(h).to(torch.bfloat16).double()
        return xin.double() + h @ w2.double().T + (b2.double() if bias else 0)

    before = ops.launches
    if c > 512:
        # wider than the fused kernel takes: the two projections run, in place
        keep = x.clone()
        same = ops.mlp_residual(ops.defer_layernorm(x, gain, shift, 1e-5, torch.bfloat16), w1, b1, w2, b2,
                                "gelu_tanh", x, torch.bfloat16)
        assert same is x and ops.launches == before + 2
        want = formula(keep)
        assert (same.double() - want).abs().max() <= 2e-2 * max(1.0, float(want.abs().max()))
        return
    first = ops.mlp_residual(ops.defer_layernorm(x, gain, shift, 1e-5, torch.bfloat16), w1, b1, w2, b2,
                             "gelu_tanh", x, torch.bfloat16)
    assert first is not x, "the fused kernel was expected to run and hand back another buffer"
    assert ops.launches == before + 2                      # the zero fill of the first call, and the kernel
    want = formula(x)
    scale = max(1.0, float(want.abs().max()))
    assert (first.double() - want).abs().max() <= 2e-2 * scale   # a hidden value at a bfloat16 rounding edge
    second = ops.mlp_residual(ops.defer_layernorm(first, gain, shift, 1e-5, torch.bfloat16), w1, b1, w2, b2,
                              "gelu_tanh", first, torch.bfloat16)
    assert ops.launches == before + 3 and second is not first and second is not x
    assert (second.double() - formula(first)).abs().max() <= 2e-2 * scale
    third = ops.mlp_residual(ops.defer_layernorm(second, gain, shift, 1e-5, torch.bfloat16), w1, b1, w2, b2,
                             "gelu_tanh", second, torch.bfloat16)
    assert third is x and ops.launches == before + 4         # the first buffer's turn again
    assert (third.double() - formula(second)).abs().max() <= 2e-2 * scale
    # the two-kernel path from the same input
    x2 = second.clone()
    ops.use_fused_mlp = False
    try:
        apart = ops.mlp_residual(ops.defer_layernorm(x2, gain, shift, 1e-5, torch.bfloat16), w1, b1, w2, b2,
                                 "gelu_tanh", x2, torch.bfloat16)
    finally:
        ops.use_fused_mlp = True
    assert apart is x2
    assert (apart - third).abs().max() <= 1e-2 * scale
    ops.check_status()


@pytest.mark.parametrize("m", [17, 24, 32, 33, 50, 64, 65, 96, 100, 128])
@pytest.mark.parametrize("n,k", [(1536, 512), (512, 2048), (509, 96), (200, 200), (77, 40), (2048, 4096),
                                 (6400, 1600), (4800, 1600), (5003, 520)])
def test_mid_batch_projection_over_a_cluster(ops, m, n, k):
    """17 to 128 tokens: K cut over the CTAs of a cluster, partial sums met through distributed
    shared memory; every epilogue, against the formula and against the tensor-core kernel.  The
    matrices of 4800 rows and more make a warp take two tiles (up to 64 tokens); beyond 64 tokens
    the kernel holds six or eight groups of 16 tokens and serves matrices of up to 3 MB (the larger
    ones here then go to the tensor-core kernel, and the comparison holds all the same)."""
    x = randn(m, k, dtype=torch.bfloat16, seed=31)
    w = randn(n, k, dtype=torch.bfloat16, seed=32, scale=1 / math.sqrt(k))
    b = randn(n, seed=33)
    want = x.double() @ w.double().T + b.double()
    before = ops.launches
    got = ops.linear(x, w, b, "none", torch.float32)
    assert ops.launches == before + 1
    assert (got.double() - want).abs().max() <= 2e-4
    ops.use_cluster = False
    try:
        other = ops.linear(x, w, b, "none", torch.float32)
    finally:
        ops.use_cluster = True
    assert (got - other).abs().max() <= 1e-4                  # same bf16 inputs, 32-bit sums
    res = randn(m, n, seed=34)
    keep = res.clone()
    ops.linear_residual(x, w, b, res)
    assert (res.double() - (keep.double() + want)).abs().max() <= 2e-4
    gl = ops.linear(x, w, None, "gelu_tanh", torch.bfloat16)
    assert (gl.double() - plain_gpt.gelu_tanh(want - b.double())).abs().max() <= 3e-2
    ops.check_status()


@pytest.mark.parametrize("m", [1, 5, 8, 16, 24, 33, 64])
@pytest.mark.parametrize("vocab,k,limit", [(50304, 512, None), (50304, 512, 50257), (509, 96, 300), (77, 40, None),
                                           (9001, 200, 9000)])
def test_greedy_choice_on_the_way_of_the_head_projection(ops, m, vocab, k, limit):
    """The head's projection may leave the argmax of every row while it writes the logits: it
    must be the argmax of exactly those logits (lowest index among equals, ids at or above the
    limit never), whichever kernel runs."""
    x32 = randn(m + 2, k, seed=61, scale=1.5)
    rows = torch.tensor([(3 * i + 1) % (m + 2) for i in range(m)], dtype=torch.int32).cuda()
    gain, shift = randn(k, seed=62) + 1.0, randn(k, seed=63)
    w = randn(vocab, k, dtype=torch.bfloat16, seed=64, scale=1 / math.sqrt(k))
    w[vocab // 2] = w[3]                                        # equal logits: the lower index must win
    w[vocab - 1] = w[3]
    ids = torch.full((m,), -1, dtype=torch.int32, device="cuda")
    y = ops.defer_layernorm(x32, gain, shift, 1e-5, torch.bfloat16, rows)
    logits, taken = ops.logits(y, w, ids, limit)
    if not taken:
        ids = ops.argmax(logits, limit)
    assert taken == (m <= 16), "up to 16 rows the projection takes the choice on its way"
    masked = logits.clone()
    if limit is not None:
        masked[:, limit:] = -float("inf")
    want = masked.argmax(-1)
    best = masked.max(-1).values
    first = (masked == best[:, None]).float().argmax(-1)      # lowest index among equal maxima
    assert torch.equal(ids.long(), first), (ids, want)
    plain = ops.logits(y, w)
    assert torch.equal(plain, logits), "the logits themselves must not change"
    ops.check_status()


@pytest.mark.parametrize("m", [3, 16, 24, 64])
def test_streaming_projection_of_a_wide_matrix_takes_up_to_64_rows(ops, m):
    """The kernel that streams a wide matrix through shared memory is used for up to 16 rows; it
    takes 64, checked here by raising the limit."""
    from mini_gpt_inference_b200.kernels import ops as ops_module

    n, k = 9001, 200
    x = randn(m, k, dtype=torch.bfloat16, seed=71)
    w = randn(n, k, dtype=torch.bfloat16, seed=72, scale=1 / math.sqrt(k))
    b = randn(n, seed=73)
    want = x.double() @ w.double().T + b.double()
    was = ops_module.STREAM_ROWS
    ops_module.STREAM_ROWS = 64
    ops.use_wide = False                                     # (the kernel of tiled copies takes 16 rows; this one is meant)
    try:
        ids = torch.full((m,), -1, dtype=torch.int32, device="cuda")
        got = ops.linear(x, w, b, "none", torch.float32)
        logits, taken = ops.logits(x, w, ids, 9000)
    finally:
        ops_module.STREAM_ROWS = was
        ops.use_wide = True
    assert taken
    assert (got.double() - want).abs().max() <= 2e-4
    masked = logits.clone()
    masked[:, 9000:] = -float("inf")
    assert torch.equal(ids.long(), masked.argmax(-1))
    ops.check_status()


@pytest.mark.parametrize("wide", [True, False], ids=["tiles", "rows"])
@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(640, 1600), (203, 6400), (9001, 1608), (77, 3080), (4800, 1600), (1600, 6400)])
def test_streamed_projection_of_long_rows(ops, m, n, k, wide):
    """Large matrices are streamed: as boxes of whole rows by TMA through a ring (rows of a multiple
    of 64 and up to 2048 values; longer ones only for the residual epilogue, K cut over CTAs whose
    partial sums are added in L2), or, where that kernel refuses, row by row in K chunks (a tile's
    sums stay in registers from chunk to chunk); with the LayerNorm prologue: one launch, and the
    same numbers as the separate kernels."""
    x32 = randn(m + 3, k, seed=81, scale=2.0) + 0.5
    rows = torch.tensor([(3 * i + 1) % (m + 3) for i in range(m)], dtype=torch.int32).cuda()
    gain, shift = randn(k, seed=82) + 1.0, randn(k, seed=83)
    w = randn(n, k, dtype=torch.bfloat16, seed=84, scale=1 / math.sqrt(k))
    b = randn(n, seed=85)
    want = torch.nn.functional.layer_norm(x32[rows.long()].double(), (k,), gain.double(), shift.double(), 1e-5)
    want = want.to(torch.bfloat16).double() @ w.double().T + b.double()
    flags = (ops.stream_min_bytes, ops.stream_max_chunks, ops.use_skinny, ops.use_cluster, ops.use_wide)
    ops.stream_min_bytes, ops.stream_max_chunks, ops.use_skinny, ops.use_cluster = 0, 1 << 20, False, False
    ops.use_wide = wide
    # 16 rows of 6400 values leave no room for stages beside them: refused, other kernels take it
    fits = (8 if m <= 8 else 16) * (2 * k + 64) + 8 * k + 8 * 4 * 8 * (2 * 64 + 64) <= 226 * 1024
    if wide:
        fits = fits or k <= 2048                              # the tiled kernel stages rows of up to 2048 values
    try:
        before = ops.launches
        fused = ops.linear(ops.defer_layernorm(x32, gain, shift, 1e-5, torch.bfloat16, rows), w, b, "none",
                           torch.float32)
        assert (ops.launches == before + 1) == fits, "norm, gather and projection in one streaming kernel"
        y = ops.layernorm(ops.gather_rows(x32, rows), gain, shift, 1e-5, torch.bfloat16)
        streamed = ops.linear(y, w, b, "none", torch.float32)
        g = ops.linear(y, w, b, "gelu_tanh", torch.bfloat16)
        res = randn(m, n, seed=86)
        keep = res.clone()
        ops.linear_residual(y, w, b, res)
        ops.use_stream = ops.use_wide = False
        apart = ops.linear(y, w, b, "none", torch.float32)
    finally:
        ops.stream_min_bytes, ops.stream_max_chunks, ops.use_skinny, ops.use_cluster, ops.use_wide = flags
        ops.use_stream = True
    assert (fused.double() - want).abs().max() <= 2e-2       # bf16 rounding of the normalised rows
    assert (fused - streamed).abs().max() <= 2e-5             # the fused norm rounds as the stand-alone kernel
    assert (streamed - apart).abs().max() <= 2e-5             # same bf16 inputs, 32-bit sums
    assert (res.double() - (keep.double() + want)).abs().max() <= 2e-2
    assert (g.double() - plain_gpt.gelu_tanh(want)).abs().max() <= 5e-2
    ops.check_status()


@pytest.mark.parametrize("m,vocab,k,limit", [(1, 50304, 512, None), (8, 50257, 1600, 50000), (16, 9001, 192, 9000),
                                             (3, 777, 64, None), (13, 50257, 1024, None)])
def test_large_matrix_kernel_takes_the_greedy_choice_on_its_way(ops, m, vocab, k, limit):
    """The head through the kernel of tiled copies: 32-bit logits, and the first stage of the greedy
    argmax in its epilogue (lowest index among equal maxima, ids at or above the limit excluded)."""
    x = randn(m, k, dtype=torch.bfloat16, seed=75)
    w = randn(vocab, k, dtype=torch.bfloat16, seed=76, scale=1 / math.sqrt(k))
    w[vocab // 2] = w[7]                                     # a tie between two rows
    flags = (ops.stream_min_bytes, ops.use_stream, ops.use_skinny)
    ops.stream_min_bytes, ops.use_stream, ops.use_skinny = 0, False, False
    try:
        ids = torch.full((m,), -1, dtype=torch.int32, device="cuda")
        before = ops.launches
        logits, taken = ops.logits(x, w, ids, limit)
        assert taken and ops.launches == before + 2          # the projection and the merge of its candidates
    finally:
        ops.stream_min_bytes, ops.use_stream, ops.use_skinny = flags
    want = x.double() @ w.double().T
    assert (logits.double() - want).abs().max() <= 2e-5
    masked = logits.clone()
    if limit is not None:
        masked[:, limit:] = -float("inf")
    best = masked.max(-1).values
    first = (masked == best[:, None]).float().argmax(-1)     # lowest index among equal maxima
    assert torch.equal(ids.long(), first)
    ops.check_status()


def test_large_matrix_kernel_at_random_shapes(ops):
    """Shapes drawn at random (1 to 16 tokens, rows in multiples of 64 up to 4096, any number of
    weight rows, each epilogue, with and without bias and LayerNorm prologue): the cuts of the
    kernel of tiled copies (rows per box, slices of K, warps that own or share a box, bias kept in
    shared memory or not) against a 64-bit product."""
    import random

    rng = random.Random(5)
    flags = (ops.stream_min_bytes, ops.use_stream, ops.use_skinny, ops.use_cluster)
    ops.stream_min_bytes, ops.use_stream, ops.use_skinny, ops.use_cluster = 0, False, False, False
    taken = 0
    try:
        for case in range(40):
            m = rng.choice([1, 2, 3, 5, 8, 9, 13, 16])
            k = 64 * rng.choice([1, 2, 3, 5, 8, 12, 16, 17, 25, 32, 40, 64])
            n = rng.choice([8, 17, 64, 100, 333, 1024, 1601, 4099, 20011, 70001])
            epilogue = rng.choice(["none", "gelu_tanh", "residual"])
            prologue = rng.random() < 0.5 and k <= 2048
            with_bias = rng.random() < 0.7
            x32 = randn(m, k, seed=200 + case, scale=1.5) + 0.25
            gain, shift = randn(k, seed=300 + case) + 1.0, randn(k, seed=400 + case)
            w = randn(n, k, dtype=torch.bfloat16, seed=500 + case, scale=1 / math.sqrt(k))
            b = randn(n, seed=600 + case) if with_bias else None
            if prologue:
                xin = ops.defer_layernorm(x32, gain, shift, 1e-5, torch.bfloat16)
                xr = torch.nn.functional.layer_norm(x32.double(), (k,), gain.double(), shift.double(), 1e-5)
                xr = xr.to(torch.bfloat16).double()
            else:
                xin = x32.to(torch.bfloat16)
                xr = xin.double()
            want = xr @ w.double().T + (b.double() if with_bias else 0.0)
            before = ops.launches
            if epilogue == "residual":
                res = randn(m, n, seed=700 + case)
                keep = res.clone()
                if prologue:
                    xin = xin.materialize()
                ops.linear_residual(xin, w, b, res)
                got, want = res.double(), keep.double() + want
                tol = 2e-2 if prologue else 2e-4
            else:
                got = ops.linear(xin, w, b, epilogue, torch.float32).double()
                if epilogue == "gelu_tanh":
                    want = plain_gpt.gelu_tanh(want)
                tol = 2e-2 if prologue else 2e-4
            taken += int(ops.launches == before + 1)
            assert (got - want).abs().max() <= tol, (case, m, n, k, epilogue, prologue, with_bias)
    finally:
        ops.stream_min_bytes, ops.use_stream, ops.use_skinny, ops.use_cluster = flags
    assert taken >= 25, "most of these shapes are the kernel's own (the others it refuses: other kernels run)"
    ops.check_status()


def test_large_matrix_kernel_asks_for_the_matrix_that_followed_it_last_time(ops):
    """The kernel for large matrices asks the weights of the projection that came next the last
    time into L2 (a hint learned from the order of the calls): results do not change with it, and
    a matrix that is gone is not asked for."""
    import gc

    m, n, k = 8, 4800, 1600
    x = randn(m, k, dtype=torch.bfloat16, seed=95)
    w1 = randn(n, k, dtype=torch.bfloat16, seed=96, scale=1 / math.sqrt(k))
    w2 = randn(n, k, dtype=torch.bfloat16, seed=97, scale=1 / math.sqrt(k))
    want1 = x.double() @ w1.double().T
    first = ops.linear(x, w1, None, "none", torch.float32)                # nothing is known to follow w1 yet
    ops.linear(x, w2, None, "none", torch.float32)
    assert ops._next_weight[w1.data_ptr()]() is w2
    again = ops.linear(x, w1, None, "none", torch.float32)                # asks for w2 on its way
    assert torch.equal(first, again) and (first.double() - want1).abs().max() <= 2e-5
    del w2
    gc.collect()
    assert ops._next_weight[w1.data_ptr()]() is None
    once_more = ops.linear(x, w1, None, "none", torch.float32)            # the follower is gone: no hint
    assert torch.equal(first, once_more)
    ops.check_status()


@pytest.mark.parametrize("wide", [True, False], ids=["tiles", "rows"])
@pytest.mark.parametrize("m", [1, 8, 16])
def test_streamed_qkv_projection_writes_keys_and_values(ops, m, wide):
    """A QKV matrix of many megabytes is streamed as well; the epilogue of the streaming kernel
    copies key and value features to their cache rows like the other projection kernels."""
    n_head, n_kv, d, pt, k = 5, 5, 64, 16, 1600
    width = (n_head + 2 * n_kv) * d
    x = randn(m, k, dtype=torch.bfloat16, seed=91)
    w = randn(width, k, dtype=torch.bfloat16, seed=92, scale=1 / math.sqrt(k))
    b = randn(width, seed=93)
    pages = 6
    slots = torch.randperm(pages * pt)[:m].to(torch.int32)
    if m > 1:
        slots[0] = -1                                        # a padding row writes nothing
    slots = slots.cuda()
    cache = SimpleNamespace(k_pages=torch.zeros(pages, n_kv, pt, d, dtype=torch.bfloat16).cuda(),
                            v_pages=torch.zeros(pages, n_kv, pt, d, dtype=torch.bfloat16).cuda(),
                            page_tokens=pt, writes=True)
    flags = (ops.stream_min_bytes, ops.stream_max_chunks, ops.use_skinny, ops.use_cluster, ops.use_wide)
    ops.stream_min_bytes, ops.stream_max_chunks, ops.use_skinny, ops.use_cluster, ops.use_wide = 0, 1 << 20, False, False, wide
    try:
        before = ops.launches
        qkv = ops.linear_qkv(x, w, b, n_head, n_kv, d, cache, slots, torch.bfloat16)
        assert ops.launches == before + 1, "projection and page write were expected in one streaming kernel"
    finally:
        ops.stream_min_bytes, ops.stream_max_chunks, ops.use_skinny, ops.use_cluster, ops.use_wide = flags
    kk = qkv[:, n_head * d: (n_head + n_kv) * d].reshape(m, n_kv, d)
    vv = qkv[:, (n_head + n_kv) * d:].reshape(m, n_kv, d)
    want_k, want_v = torch.zeros_like(cache.k_pages), torch.zeros_like(cache.v_pages)
    for i, s_ in enumerate(slots.tolist()):
        if s_ >= 0:
            want_k[s_ // pt, :, s_ % pt] = kk[i]
            want_v[s_ // pt, :, s_ % pt] = vv[i]
    assert torch.equal(cache.k_pages, want_k) and torch.equal(cache.v_pages, want_v)
    ref = x.double() @ w.double().T + b.double()
    assert (qkv.double() - ref).abs().max() <= 5e-2
    ops.check_status()


@pytest.mark.parametrize("heads", [(6, 2, 32), (3, 1, 48)])
@pytest.mark.parametrize("m", [1, 4, 8, 9, 40, 70, 200, 333])
def test_qkv_projection_writes_keys_and_values_to_their_pages(ops, m, heads):
    # every projection kernel (small batch, mid batch, tensor cores) has the copy in its epilogue
    n_head, n_kv, d = heads
    pt, k = 8, 96
    pages = max(12, m // pt + 3)
    width = (n_head + 2 * n_kv) * d
    x = randn(m, k, dtype=torch.bfloat16, seed=31)
    w = randn(width, k, dtype=torch.bfloat16, seed=32, scale=0.1)
    b = randn(width, seed=33)
    slots = torch.randperm(pages * pt)[:m].to(torch.int32)
    slots[0] = -1                                            # a padding row writes nothing
    slots = slots.cuda()
    cache = SimpleNamespace(k_pages=torch.zeros(pages, n_kv, pt, d, dtype=torch.bfloat16).cuda(),
                            v_pages=torch.zeros(pages, n_kv, pt, d, dtype=torch.bfloat16).cuda(),
                            page_tokens=pt, writes=True)
    qkv = ops.linear_qkv(x, w, b, n_head, n_kv, d, cache, slots, torch.bfloat16)
    kk = qkv[:, n_head * d: (n_head + n_kv) * d].reshape(m, n_kv, d)
    vv = qkv[:, (n_head + n_kv) * d:].reshape(m, n_kv, d)
    want_k, want_v = torch.zeros_like(cache.k_pages), torch.zeros_like(cache.v_pages)
    for i, s_ in enumerate(slots.tolist()):
        if s_ >= 0:
            want_k[s_ // pt, :, s_ % pt] = kk[i]
            want_v[s_ // pt, :, s_ % pt] = vv[i]
    assert torch.equal(cache.k_pages, want_k) and torch.equal(cache.v_pages, want_v)
    ref = x.double() @ w.double().T + b.double()
    assert (qkv.double() - ref).abs().max() <= 5e-2


def _attention_case(ops, dtype, n_head, n_kv_head, head_dim, page_tokens, window, lengths, q_lens,
                    seed=0, spike=None):
    """Requests with `lengths[i]` tokens in total, of which the last `q_lens[i]` are new.
    spike = (request, key position, gain): that key is `gain` in every feature and the request's
    queries of head 0 are all ones, so that its score stands far above every other."""
    g = torch.Generator().manual_seed(seed)
    R = len(lengths)
    max_pages = max(-(-n // page_tokens) for n in lengths) + 1
    num_pages = sum(-(-n // page_tokens) for n in lengths) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()       # pages in scattered order
    tables = torch.full((R, max_pages), -1, dtype=torch.int32)
    k_all, v_all = [], []
    k_pages = torch.full((num_pages, n_kv_head, page_tokens, head_dim), float("nan"))
    v_pages = torch.full((num_pages, n_kv_head, page_tokens, head_dim), float("nan"))
    for r, n in enumerate(lengths):
        k = torch.randn(n, n_kv_head, head_dim, generator=g).to(dtype).float()
        v = torch.randn(n, n_kv_head, head_dim, generator=g).to(dtype).float()
        if spike is not None and spike[0] == r:
            k[spike[1]] = spike[2]
        k_all.append(k)
        v_all.append(v)
        for i in range(-(-n // page_tokens)):
            page = perm.pop()
            tables[r, i] = page
            chunk = slice(i * page_tokens, min(n, (i + 1) * page_tokens))
            k_pages[page, :, : chunk.stop - chunk.start] = k[chunk].transpose(0, 1)
            v_pages[page, :, : chunk.stop - chunk.start] = v[chunk].transpose(0, 1)
    # unused rows of pages hold NaN: reading past a request's length would poison the output
    qkv_rows, token_request, positions, want = [], [], [], []
    scale = 1.0 / math.sqrt(head_dim)
    for r, (n, ql) in enumerate(zip(lengths, q_lens)):
        q = torch.randn(ql, n_head, head_dim, generator=g).to(dtype).float() * 2.0
        if spike is not None and spike[0] == r:
            q[:, 0] = 1.0
        for i in range(ql):
            p = n - ql + i
            lo = 0 if not window else max(0, p - window + 1)
            row = torch.zeros(n_head, head_dim, dtype=torch.float64)
            for h in range(n_head):
                kh = h // (n_head // n_kv_head)
                s = (k_all[r][lo: p + 1, kh].double() @ q[i, h].double()) * scale
                row[h] = torch.softmax(s, 0) @ v_all[r][lo: p + 1, kh].double()
            want.append(row.reshape(-1))
            filler = torch.zeros(2 * n_kv_head * head_dim)
            qkv_rows.append(torch.cat([q[i].reshape(-1), filler]))
            token_request.append(r)
            positions.append(p)
    cache = SimpleNamespace(k_pages=k_pages.to(dtype).cuda(), v_pages=v_pages.to(dtype).cuda(),
                            group=0, page_tokens=page_tokens, window=window or None, writes=False)
    from mini_gpt_inference_b200.parts.context import HostBatch, StepPlan

    # the host half of the tiled prompt attention, as the attention mixer asks for it
    plan = StepPlan()
    ops.plan_prompt_attention(HostBatch(q_lens, [n - ql for n, ql in zip(lengths, q_lens)], [0] * len(q_lens),
                                        dtype), plan, n_head, n_kv_head, head_dim)
    ctx = SimpleNamespace(block_tables=[tables.cuda()],
                          token_request=torch.tensor(token_request, dtype=torch.int32).cuda(),
                          positions=torch.tensor(positions, dtype=torch.int32).cuda(),
                          decode_only=all(q == 1 for q in q_lens), max_ctx_after=max(lengths),
                          extra={k: torch.from_numpy(v).cuda() for k, v in plan.arrays.items()})
    qkv = torch.stack(qkv_rows).to(dtype).cuda()
    before = ops.launches
    got = ops.paged_attention(qkv, n_head, n_kv_head, head_dim, scale, cache, ctx)
    _attention_case.kernels = ops.launches - before
    return got.double().cpu(), torch.stack(want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_tokens,window", [
    (8, 8, 64, 16, 0), (3, 3, 32, 8, 0), (5, 1, 48, 4, 0), (6, 2, 16, 16, 0), (4, 4, 80, 32, 0),
    (2, 2, 128, 16, 0), (4, 2, 256, 64, 0), (4, 4, 32, 8, 5), (6, 3, 64, 16, 33)])
def test_paged_attention_general(ops, dtype, n_head, n_kv_head, head_dim, page_tokens, window):
    pt = page_tokens
    lengths = [1, 2, pt - 1, pt, pt + 1, 2 * pt, 3 * pt + 1, 150]
    q_lens = [1, 2, 1, pt, 3, 1, 2 * pt + 1, 31]
    got, want = _attention_case(ops, dtype, n_head, n_kv_head, head_dim, pt, window, lengths, q_lens)
    assert not torch.isnan(got).any(), "attention read a cache row beyond a request's length"
    assert (got - want).abs().max() <= _tol(dtype, 1.0)


@pytest.mark.parametrize("gain", [4.0, 9.0, 24.0])
def test_prompt_attention_with_a_key_far_above_the_others(ops, gain):
    """One key, hundreds of positions into the prompt, scores 8 * gain above the rest (head 0; other
    heads see it at random heights, above and below).  The tensor-core kernel takes each row's
    reference exponent from the first block and must move it when this key comes: at 9 the
    weights leave the range it allows, at 24 they leave the range of 32-bit floats.  Queries
    before the key must not see it; the tile is cut along the keys, so parts with references far
    apart are merged."""
    lengths, q_lens = [1000, 300], [700, 300]
    got, want = _attention_case(ops, torch.bfloat16, 4, 2, 64, 16, 0, lengths, q_lens, seed=5,
                                spike=(0, 611, gain))
    ops.check_status()
    assert not torch.isnan(got).any()
    # rows that see the key return its value row, not an average of many: the results are as
    # large as single values are (up to 4), and a bfloat16 result is that much coarser
    assert (got - want).abs().max() <= _tol(torch.bfloat16, max(1.0, float(want.abs().max())))
    assert float(want.abs().max()) > 2.0


@pytest.mark.parametrize("n_head,n_kv_head,page_tokens,window", [
    (8, 8, 16, 0), (2, 2, 8, 0), (4, 1, 64, 0), (2, 2, 128, 0), (2, 1, 256, 0), (3, 3, 32, 0),
    (4, 2, 16, 33), (2, 2, 64, 200)])
def test_prompt_portions_on_the_tensor_cores(ops, n_head, n_kv_head, page_tokens, window):
    """Portions of prompts with head size 64 in bfloat16 take the tcgen05 kernel: query tiles of
    128 rows over key blocks of 64 from the pages; tiles that start anywhere in a request,
    tiles of one row, contexts that end at any place inside a block or a page."""
    lengths = [300, 129, 128, 1000, 1, 77, 513, 1300, 2048]
    q_lens = [300, 129, 5, 700, 1, 2, 257, 3, 130]
    got, want = _attention_case(ops, torch.bfloat16, n_head, n_kv_head, 64, page_tokens, window,
                                lengths, q_lens, seed=3)
    ops.check_status()
    assert not torch.isnan(got).any()
    assert (got - want).abs().max() <= _tol(torch.bfloat16, 1.0)
    ops.use_prefill_tc = False
    try:
        general, _ = _attention_case(ops, torch.bfloat16, n_head, n_kv_head, 64, page_tokens, window,
                                     lengths, q_lens, seed=3)
    finally:
        ops.use_prefill_tc = True
    assert (general - got).abs().max() <= _tol(torch.bfloat16, 1.0)
    assert not torch.equal(general, got), "the two kernels were expected to differ in rounding"


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_tokens,window", [
    (8, 8, 64, 16, 0), (8, 8, 64, 64, 0), (3, 3, 32, 8, 0), (6, 2, 16, 16, 0), (2, 2, 128, 16, 0),
    (4, 2, 256, 64, 0), (4, 4, 32, 8, 5), (6, 3, 64, 16, 300)])
def test_paged_attention_split_over_keys(ops, n_head, n_kv_head, head_dim, page_tokens, window):
    """Single query tokens in bfloat16 take the kernel that splits the keys into blocks of 256
    and merges: lengths around the block edges (blocks of 32 to 256 keys by head size), one token, long contexts."""
    lengths = [1, 2, 63, 64, 65, 127, 129, 255, 256, 257, 511, 513, 700, 1025, page_tokens, page_tokens + 1]
    got, want = _attention_case(ops, torch.bfloat16, n_head, n_kv_head, head_dim, page_tokens, window,
                                lengths, [1] * len(lengths))
    assert _attention_case.kernels == 1, "the split kernel (with its own merge) was expected to run"
    ops.check_status()
    assert not torch.isnan(got).any()
    assert (got - want).abs().max() <= _tol(torch.bfloat16, 1.0)
    # the general kernel gives the same within rounding
    ops.use_split_attention = False
    try:
        general, _ = _attention_case(ops, torch.bfloat16, n_head, n_kv_head, head_dim, page_tokens, window,
                                     lengths, [1] * len(lengths))
    finally:
        ops.use_split_attention = True
    assert (general - got).abs().max() <= _tol(torch.bfloat16, 1.0)


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_tokens,rows", [
    (8, 8, 64, 64, 64),        # the 50M model's batch of 64: 64 x 8 x 9 blocks
    (24, 2, 64, 16, 170),      # 12 query heads per kv head: two tiles of eight heads per CTA
    (40, 2, 32, 8, 200),       # 20 heads per kv head: two CTAs per kv head, the second not full
    (4, 4, 128, 32, 70)])
def test_split_attention_of_many_rows_merges_in_a_second_kernel(ops, n_head, n_kv_head, head_dim,
                                                                  page_tokens, rows):
    """A grid of several waves leaves its partial rows in scratch and a second kernel merges them.
    Every row's context is long enough for three or more key blocks that all hold keys, and the
    lengths differ from row to row, so that a block merged twice, dropped, or taken from the
    neighbour's scratch shows."""
    block = ops.lib.mg_attention_split_keys(head_dim)
    lengths = [2 * block + 37 + (11 * i) % (2 * block + 150) for i in range(rows)]
    assert min(lengths) > 2 * block
    got, want = _attention_case(ops, torch.bfloat16, n_head, n_kv_head, head_dim, page_tokens, 0,
                                lengths, [1] * rows, seed=11)
    assert _attention_case.kernels == 2, "the merge was expected to run as a kernel of its own"
    ops.check_status()
    assert not torch.isnan(got).any()
    assert (got - want).abs().max() <= _tol(torch.bfloat16, 1.0)
    # the counters stay zero for the next launch, whichever kernel merged
    assert int(ops._counters(1).abs().sum()) == 0


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_tokens,lengths,launches", [
    (2, 2, 64, 64, [2049, 2200, 4097, 6000, 8191, 2176], 1),     # 17 to 64 blocks of 128 keys, merged by the last CTA
    (4, 1, 64, 16, [9000, 3333], 1),                             # grouped heads, 71 and 27 blocks
    (2, 2, 32, 64, [4400, 5000, 7000], 1),                       # blocks of 256 keys: 18 to 28
    (2, 2, 128, 32, [1100, 1500, 2300], 1),                      # blocks of 64 keys: 18 to 36
    (8, 8, 64, 64, [2100 + 37 * i for i in range(12)], 2)])      # 12 x 8 x 20 blocks: the second kernel merges
def test_split_attention_with_many_key_blocks(ops, n_head, n_kv_head, head_dim, page_tokens, lengths, launches):
    """Contexts of more than sixteen key blocks: the merge then shares a row's blocks among the four
    warps of a CTA (quarters, added in warp order), inside the attention kernel or in the second one.
    A spike far back in the longest request must still decide its row."""
    block = ops.lib.mg_attention_split_keys(head_dim)
    assert min(lengths) > 16 * block
    longest = max(range(len(lengths)), key=lambda i: lengths[i])
    for spike in (None, (longest, 5, 3.0)):
        got, want = _attention_case(ops, torch.bfloat16, n_head, n_kv_head, head_dim, page_tokens, 0,
                                    lengths, [1] * len(lengths), seed=21, spike=spike)
        assert _attention_case.kernels == launches
        ops.check_status()
        assert not torch.isnan(got).any()
        assert (got - want).abs().max() <= _tol(torch.bfloat16, 1.0)
    assert int(ops._counters(1).abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_key_among_hundreds_decides(ops, dtype):
    """One key far back gets a score that dominates: the output must be that key's value."""
    n_head, head_dim, pt, n = 2, 64, 16, 700
    g = torch.Generator().manual_seed(5)
    k = torch.randn(n, n_head, head_dim, generator=g) * 0.1
    v = torch.randn(n, n_head, head_dim, generator=g)
    q = torch.randn(1, n_head, head_dim, generator=g)
    far = 3                                                      # in the first page
    k[far] = q[0] * 4.0                                          # score ~ 4 |q|^2 / 8 >> the rest
    pages = -(-n // pt)
    kp = torch.zeros(pages, n_head, pt, head_dim)
    vp = torch.zeros(pages, n_head, pt, head_dim)
    for i in range(pages):
        sl = slice(i * pt, min(n, (i + 1) * pt))
        kp[i, :, : sl.stop - sl.start] = k[sl].transpose(0, 1)
        vp[i, :, : sl.stop - sl.start] = v[sl].transpose(0, 1)
    cache = SimpleNamespace(k_pages=kp.to(dtype).cuda(), v_pages=vp.to(dtype).cuda(), group=0,
                            page_tokens=pt, window=None, writes=False)
    ctx = SimpleNamespace(block_tables=[torch.arange(pages, dtype=torch.int32)[None].cuda()],
                          token_request=torch.zeros(1, dtype=torch.int32).cuda(),
                          positions=torch.tensor([n - 1], dtype=torch.int32).cuda(),
                          decode_only=True, max_ctx_after=n)
    qkv = torch.cat([q.reshape(1, -1), torch.zeros(1, 2 * n_head * head_dim)], 1).to(dtype).cuda()
    got = ops.paged_attention(qkv, n_head, n_head, head_dim, 1 / math.sqrt(head_dim), cache, ctx)
    want = v[far].to(dtype).float().reshape(-1)
    assert (got.float().cpu()[0] - want).abs().max() < 2e-2


@pytest.mark.parametrize("dtype", DTYPES)
def test_kv_store_places_rows(ops, dtype):
    n_head, n_kv, d, pt, pages = 6, 2, 48, 8, 9
    qkv = randn(11, (n_head + 2 * n_kv) * d, dtype=dtype, seed=3)
    slots = torch.tensor([5, 70, 8, 9, 63, 0, 33, 34, 35, 71, -1], dtype=torch.int32).cuda()
    cache = SimpleNamespace(k_pages=torch.zeros(pages, n_kv, pt, d, dtype=dtype).cuda(),
                            v_pages=torch.zeros(pages, n_kv, pt, d, dtype=dtype).cuda(),
                            page_tokens=pt)
    ops.kv_store(qkv, n_head, n_kv, d, cache, slots)
    k = qkv[:, n_head * d: (n_head + n_kv) * d].reshape(11, n_kv, d)
    v = qkv[:, (n_head + n_kv) * d:].reshape(11, n_kv, d)
    want_k = torch.zeros_like(cache.k_pages)
    want_v = torch.zeros_like(cache.v_pages)
    for i, s in enumerate(slots.tolist()):
        if s >= 0:
            want_k[s // pt, :, s % pt] = k[i]
            want_v[s // pt, :, s % pt] = v[i]
    assert torch.equal(cache.k_pages, want_k) and torch.equal(cache.v_pages, want_v)


def test_gather_rows_and_argmax(ops):
    x = randn(40, 77, seed=1)
    rows = torch.tensor([3, 3, 39, 0], dtype=torch.int32).cuda()
    assert torch.equal(ops.gather_rows(x, rows), x[rows.long()])
    logits = randn(9, 50304, seed=2)
    logits[4, 50300] = 99.0
    logits[5, 17] = logits[5, 4000] = 50.0                     # a tie: the lower index wins
    got = ops.argmax(logits)
    assert got.tolist() == logits.argmax(-1).tolist() or got[5] == 17
    assert got[4] == 50300 and got[5] == 17
    limited = ops.argmax(logits, 50257)
    assert limited[4] == logits[4, :50257].argmax()


def _draws(ops, logits_row, temperature, top_k, top_p, n, seed=1234):
    rows = logits_row[None].expand(n, -1).contiguous()
    i32 = lambda v: torch.full((n,), v, dtype=torch.int32).cuda()          # noqa: E731
    f32 = lambda v: torch.full((n,), v, dtype=torch.float32).cuda()        # noqa: E731
    counter = torch.arange(n, dtype=torch.int32).cuda()
    return ops.sample(rows, f32(temperature), None if top_k is None else i32(top_k),
                      None if top_p is None else f32(top_p), i32(seed & 0xFFFF), i32(seed >> 16),
                      counter)


@pytest.mark.parametrize("vocab", [509, 50304])
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, None, None), (0.7, 5, None),
                                                     (1.3, None, 0.6), (0.9, 40, 0.8)])
def test_sampler_draws_from_the_reference_distribution(ops, vocab, temperature, top_k, top_p):
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(vocab, generator=g) * 2.5).cuda()
    want = plain_gpt.sampling_distribution(logits.cpu(), temperature, top_k, top_p)
    n = 40000
    ids = _draws(ops, logits, temperature, top_k, top_p, n).long().cpu()
    counts = torch.bincount(ids, minlength=vocab).double()
    # nothing outside the support (allowing the one token at the top-p edge to differ by rounding)
    outside = counts[want == 0].sum().item()
    assert outside <= (0 if top_p is None else 0.002 * n), outside
    # frequencies follow the probabilities: compare on the 20 likeliest tokens
    top = want.topk(20).indices
    freq = counts[top] / n
    sigma = (want[top] * (1 - want[top]) / n).sqrt()
    assert ((freq - want[top]).abs() <= 5 * sigma + 2e-3).all(), (freq, want[top])


def test_sampler_is_greedy_at_zero_and_repeatable_by_seed(ops):
    g = torch.Generator().manual_seed(4)
    logits = torch.randn(6, 1000, generator=g).cuda()
    zeros = torch.zeros(6).cuda()
    i32 = lambda v: torch.full((6,), v, dtype=torch.int32).cuda()          # noqa: E731
    got = ops.sample(logits, zeros, None, None, i32(1), i32(2), i32(3))
    assert got.tolist() == logits.argmax(-1).tolist()
    # mixed rows: greedy and stochastic side by side (tests/test_sampling.py:63-78)
    temps = torch.tensor([0.0, 1.0, 0.0, 1.0, 1.0, 0.0]).cuda()
    a = ops.sample(logits, temps, None, None, i32(7), i32(0), i32(5))
    b = ops.sample(logits, temps, None, None, i32(7), i32(0), i32(5))
    c = ops.sample(logits, temps, None, None, i32(8), i32(0), i32(5))
    assert a.tolist() == b.tolist()
    assert [a[i].item() for i in (0, 2, 5)] == [logits[i].argmax().item() for i in (0, 2, 5)]
    assert a.tolist() != c.tolist()
    # a row's draw does not depend on the rows beside it
    alone = ops.sample(logits[3:4].contiguous(), temps[3:4].contiguous(), None, None,
                       i32(7)[:1], i32(0)[:1], i32(5)[:1])
    assert alone[0] == a[3]
    # top_k = 1 is greedy whatever the temperature
    k1 = ops.sample(logits, torch.full((6,), 5.0).cuda(), i32(1), None, i32(7), i32(0), i32(5))
    assert k1.tolist() == logits.argmax(-1).tolist()


def test_refusals_are_clear(ops):
    from mini_gpt_inference_b200.kernels.library import KernelLibraryError

    with pytest.raises(KernelLibraryError, match="contiguous"):
        ops.layernorm(randn(4, 8).T, randn(4), None, 1e-5, torch.float32)
    with pytest.raises(KernelLibraryError, match="dtype"):
        ops.linear(randn(4, 8), randn(3, 8, dtype=torch.bfloat16), None, "none", torch.float32)
    with pytest.raises(KernelLibraryError, match="head_dim"):
        cache = SimpleNamespace(k_pages=torch.zeros(2, 1, 4, 512).cuda(), v_pages=torch.zeros(2, 1, 4, 512).cuda(),
                                group=0, page_tokens=4, window=None)
        ctx = SimpleNamespace(block_tables=[torch.zeros(1, 2, dtype=torch.int32).cuda()],
                              token_request=torch.zeros(1, dtype=torch.int32).cuda(),
                              positions=torch.zeros(1, dtype=torch.int32).cuda())
        ops.paged_attention(torch.zeros(1, 3 * 512).cuda(), 1, 1, 512, 1.0, cache, ctx)
