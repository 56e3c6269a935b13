"""Each part alone against its plain formula, at sizes of its own; and the framework's
generality: a toy mixer with per-request state of its own, a toy feed-forward that routes each
token to one of several experts, a toy position encoding and a toy architecture, all defined
here, are registered, built and stepped without touching the framework's files."""

from __future__ import annotations

import math
from dataclasses import dataclass

import pytest
import torch

import plain_gpt

from mini_gpt_inference_b200.cache import CacheManager, FixedStateSpec
from mini_gpt_inference_b200.cache.storage import CacheStorage
from mini_gpt_inference_b200.config import register_model
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry
from mini_gpt_inference_b200.parts import (FEED_FORWARDS, MIXERS, NORMS, LayerCall, LayerSpec,
                                           Mixer, ModelSpec, PartSpec, PositionEncoding,
                                           StepContext, TensorSpec, pre_norm_layer,
                                           register_arrangement, register_mixer,
                                           register_position_encoding)
from mini_gpt_inference_b200.parts.base import (EMBEDDINGS, HEADS, POSITION_ENCODINGS, FeedForward,
                                                register_feed_forward)
from mini_gpt_inference_b200.parts.block import stream_after
from mini_gpt_inference_b200.weights import random_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from mini_gpt_inference_b200.kernels.ops import default_ops

    return default_ops(DEV)


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def make_ctx(ops, dtype, lengths, manager=None, storage=None, ids=None):
    """A context in which request r brings `lengths[r]` tokens into an empty cache."""
    n = sum(lengths)
    token_request = [r for r, m in enumerate(lengths) for _ in range(m)]
    positions = [p for m in lengths for p in range(m)]
    starts = [sum(lengths[:r]) for r in range(len(lengths))]
    tables, slots = [], []
    if manager is not None:
        for g in range(len(manager.groups)):
            width = max(manager.pages_for(m) for m in lengths)
            table = torch.full((len(lengths), width), -1, dtype=torch.int32)
            slot = []
            for r, m in enumerate(lengths):
                manager.admit(f"q{r}")
                manager.reserve(f"q{r}", m)
                t = manager.block_table(f"q{r}", g)
                table[r, : len(t)] = torch.tensor(t, dtype=torch.int32)
                slot += [manager.slot_of(f"q{r}", g, p) for p in range(m)]
            tables.append(table.to(DEV))
            slots.append(i32(slot))
    return StepContext(
        ops=ops, act_dtype=dtype, num_tokens=n, num_requests=len(lengths),
        token_ids=i32(ids if ids is not None else [0] * n), positions=i32(positions),
        token_request=i32(token_request), req_q_start=i32(starts), req_q_len=i32(lengths),
        req_ctx_before=i32([0] * len(lengths)), req_state_slot=i32(list(range(len(lengths)))),
        block_tables=tables, slot_mapping=slots, logit_rows=i32(list(range(n))),
        host_q_len=list(lengths), host_ctx_before=[0] * len(lengths),
        host_state_slot=list(range(len(lengths))), max_q_len=max(lengths),
        max_ctx_after=max(lengths), decode_only=False, storage=storage)


def rel_err(got, want):
    """Largest difference relative to the largest wanted value: bfloat16 keeps 8 significant
    bits, so its error scales with the magnitude of what is computed."""
    return ((got.double().cpu() - want.double()).abs().max() / want.abs().max()).item()


REL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def bind_random(part, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    cpu, dev = {}, {}
    for name, spec in part.tensor_specs().items():
        t = torch.randn(spec.shape, generator=g) * (0.15 if spec.role == "matrix" else 1.0)
        store = dtype if spec.role == "matrix" else torch.float32
        cpu[name] = t.to(store).float()
        dev[name] = t.to(store).to(DEV)
    part.bind(dev)
    return cpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm_part(ops, dtype):
    part = NORMS.build(PartSpec("layernorm", {"width": 72, "eps": 2e-3, "bias": True}, "n"), "x.")
    assert set(part.tensor_specs()) == {"x.n.weight", "x.n.bias"}
    w = bind_random(part, dtype, 1)
    x = torch.randn(13, 72, generator=torch.Generator().manual_seed(2)) * 2 + 1
    got = part.forward(make_ctx(ops, dtype, [13]), x.to(DEV))
    want = plain_gpt.layer_norm(x.double(), w["x.n.weight"].double(), w["x.n.bias"].double(), 2e-3)
    assert got.dtype == dtype
    assert rel_err(got, want) <= REL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_mlp_part(ops, dtype):
    part = FEED_FORWARDS.build(PartSpec("dense_mlp", {"width": 40, "inner": 136, "bias": True}, "ff"), "")
    w = bind_random(part, dtype, 3)
    y = (torch.randn(9, 40, generator=torch.Generator().manual_seed(4))).to(dtype)
    residual = torch.randn(9, 40, generator=torch.Generator().manual_seed(5))
    res_dev = residual.to(DEV)
    res_dev = stream_after(part.forward(make_ctx(ops, dtype, [9]), y.to(DEV), res_dev), res_dev)
    want = residual.double() + plain_gpt.mlp(y.double(), {k: v.double() for k, v in w.items()}, "ff.")
    assert rel_err(res_dev, want) <= REL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_head,n_kv_head,head_dim,window", [(4, 4, 16, None), (6, 2, 32, None),
                                                              (2, 2, 48, 5)])
def test_attention_part(ops, dtype, n_head, n_kv_head, head_dim, window):
    width = 56
    part = MIXERS.build(PartSpec("causal_attention", {
        "width": width, "n_head": n_head, "n_kv_head": n_kv_head, "head_dim": head_dim,
        "bias": True, "window": window}, "attn"), "", position=None)
    w = bind_random(part, dtype, 6)
    lengths = [19, 1, 8]
    manager = CacheManager([part.cache_spec()], 8, 16, 4)
    storage = CacheStorage(manager, dtype, DEV)
    ctx = make_ctx(ops, dtype, lengths, manager, storage)
    y = torch.randn(sum(lengths), width, generator=torch.Generator().manual_seed(7)).to(dtype)
    residual = torch.zeros(sum(lengths), width, device=DEV)
    part.forward(ctx, ctx.cache_view(0), y.to(DEV), residual)
    row = 0
    for m in lengths:
        want = plain_gpt.causal_attention(y[row: row + m].double(), {k: v.double() for k, v in w.items()},
                                          "attn.", n_head, window=window, n_kv_head=n_kv_head)
        assert rel_err(residual[row: row + m], want) <= REL[dtype]
        row += m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_positions_and_head(ops, dtype):
    emb = EMBEDDINGS.build(PartSpec("token_embedding", {"vocab_size": 301, "width": 24}, "tok_emb"), "")
    pos = POSITION_ENCODINGS.build(PartSpec("learned_absolute", {"n_positions": 50, "width": 24}, "pos_emb"), "")
    head = HEADS.build(PartSpec("tied_head", {"vocab_size": 301, "width": 24, "tied_to": "tok_emb.weight"},
                                "lm_head"), "", embedding=emb)
    w = {**bind_random(emb, dtype, 8), **bind_random(pos, dtype, 9)}
    assert pos.max_positions == 50 and head.tensor_specs()["lm_head.weight"].optional_alias_of
    ids = [5, 300, 0, 17, 17, 299, 1]
    ctx = make_ctx(ops, dtype, [4, 3], ids=ids)
    x = emb.forward(ctx, pos)
    want = torch.cat([plain_gpt.embed(torch.tensor(ids[:4]), w, torch.float64),
                      plain_gpt.embed(torch.tensor(ids[4:]), w, torch.float64)])
    assert x.dtype == torch.float32 and (x.double().cpu() - want).abs().max() <= 1e-6
    y = torch.randn(7, 24, generator=torch.Generator().manual_seed(10)).to(dtype)
    logits = head.forward(ctx, y.to(DEV))
    assert logits.dtype == torch.float32
    assert (logits.double().cpu() - y.double() @ w["tok_emb.weight"].double().T).abs().max() <= 2e-5


# ---- toy parts, defined here only ------------------------------------------------------------
@register_mixer("toy_running_mean")
class RunningMeanMixer(Mixer):
    """Output at position t = gain * mean of the inputs at positions 0..t of the same request.
    Its state per request: the running sum of the inputs and the number of tokens so far."""

    def __init__(self, prefix, width, position=None):
        super().__init__(prefix)
        self.width = width
        self.gain = None

    def tensor_specs(self):
        return {self.prefix + "gain": TensorSpec((self.width,), "vector", "norm_gain")}

    def cache_spec(self):
        return FixedStateSpec((self.width + 1,), "float32")

    def forward(self, ctx, cache, y, residual32):
        start = 0
        for r, (n, before) in enumerate(zip(ctx.host_q_len, ctx.host_ctx_before)):
            slot = ctx.host_state_slot[r]
            if before == 0:
                cache.state[slot].zero_()                    # a new (or recomputed) request
            rows = y[start: start + n].float()
            sums = cache.state[slot, : self.width] + rows.cumsum(0)
            counts = cache.state[slot, self.width] + torch.arange(1, n + 1, device=y.device)
            residual32[start: start + n] += self.gain * sums / counts[:, None]
            if cache.writes:
                cache.state[slot, : self.width] = sums[-1]
                cache.state[slot, self.width] = counts[-1]
            start += n


@register_feed_forward("toy_top1_experts")
class Top1Experts(FeedForward):
    """Every token goes to the one expert whose router logit is largest (logits in 32-bit, ties
    to the lower index); an expert is ``proj(gelu(fc(y)))`` without biases."""

    def __init__(self, prefix, width, inner, experts):
        super().__init__(prefix)
        self.width, self.inner, self.experts = width, inner, experts

    def tensor_specs(self):
        specs = {self.prefix + "router.weight": TensorSpec((self.experts, self.width), "matrix")}
        for e in range(self.experts):
            specs[self.prefix + f"e{e}.fc.weight"] = TensorSpec((self.inner, self.width), "matrix")
            specs[self.prefix + f"e{e}.proj.weight"] = TensorSpec((self.width, self.inner), "matrix",
                                                                   "residual_proj")
        return specs

    def forward(self, ctx, y, residual32):
        choice = (y.float() @ self.router_weight.float().T).argmax(-1)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            h = ctx.ops.linear(y[rows].contiguous(), getattr(self, f"e{e}_fc_weight"), None, "gelu_tanh",
                               ctx.act_dtype)
            residual32[rows] += ctx.ops.linear(h, getattr(self, f"e{e}_proj_weight"), None, "none",
                                               torch.float32)


@register_position_encoding("toy_sign_flip")
class SignFlipPositions(PositionEncoding):
    """No table; flips the sign of q and k at odd positions (a stand-in for a rotation)."""

    def __init__(self, prefix=""):
        super().__init__(prefix)

    def rotate(self, ctx, qkv, n_head, n_kv_head, head_dim):
        sign = (1 - 2 * (ctx.positions % 2)).to(qkv.dtype)[:, None]
        qkv[:, : (n_head + n_kv_head) * head_dim] *= sign


@register_arrangement("toy_parallel")
def toy_parallel(ctx, layer, cache, residual32):
    """One norm feeds both branches: ``y = norm(x); x += mixer(y) + feed_forward(y)``."""
    y = layer.norm.forward(ctx, residual32)
    x = stream_after(layer.mixer.forward(ctx, cache, y, residual32), residual32)
    return stream_after(layer.feed_forward.forward(ctx, y, x), x)


toy_parallel.requires = ("norm", "mixer", "feed_forward")


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    width: int
    architecture: str = "ToyStateLM"

    @classmethod
    def from_dict(cls, raw, architecture=None):
        return cls(raw["vocab_size"], raw["width"])


TOY_WINDOW = 6


@register_model("ToyStateLM", config_class=ToyConfig)
def describe_toy(cfg: ToyConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("layernorm", {"width": cfg.width, "eps": 1e-5, "bias": False}, name)

    ff = PartSpec("dense_mlp", {"width": cfg.width, "inner": 2 * cfg.width, "bias": False}, "ff")
    mean = PartSpec("toy_running_mean", {"width": cfg.width}, "mix")
    windowed = PartSpec("causal_attention", {"width": cfg.width, "n_head": 2, "n_kv_head": 1,
                                             "head_dim": 16, "bias": False, "window": TOY_WINDOW}, "attn")
    # all keys, in pages of 8 from a pool of its own size: a second cache group beside the windowed one
    full = PartSpec("causal_attention", {"width": cfg.width, "n_head": 4, "n_kv_head": 2, "head_dim": 16,
                                         "bias": False, "cache_page_tokens": 8, "cache_pages": 9}, "attn")
    layers = (pre_norm_layer("l0.", norm("n1"), mean, norm("n2"), ff),
              pre_norm_layer("l1.", norm("n1"), windowed, norm("n2"), ff),
              pre_norm_layer("l2.", norm("n1"), mean, norm("n2"),
                             PartSpec("toy_top1_experts", {"width": cfg.width, "inner": 24, "experts": 3}, "moe")),
              LayerSpec("l3.", {"norm": norm("n"), "mixer": full, "feed_forward": ff}, "toy_parallel"))
    return ModelSpec(
        architecture="ToyStateLM", width=cfg.width, vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": cfg.width}, "emb"),
        position=PartSpec("toy_sign_flip", {}, ""),
        layers=layers,
        # layer 1 runs twice; its second run reads the cache its first run wrote
        layer_order=(LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 2), LayerCall(3, 3),
                     LayerCall(1, 1, writes_cache=False)),
        final_norm=norm("nf"),
        head=PartSpec("tied_head", {"vocab_size": cfg.vocab_size, "width": cfg.width,
                                    "tied_to": "emb.weight"}, "head"))


# ---- the toy model once more, whole sequences, no cache, plain torch in 64-bit -----------------
def plain_toy_logits(tokens, w, margins=None):
    """Logits of one whole sequence through the toy architecture, sharing nothing with the parts
    above but the formulas in their docstrings.  ``margins``: a list that receives, per token, the
    gap between the two largest router logits (a small gap means that rounding may pick another
    expert)."""
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    x = w["emb.weight"][torch.tensor(tokens)]
    counts = torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    pos = torch.arange(T)
    flip = (1 - 2 * (pos % 2)).double()[:, None]

    def ln(v, name):
        return plain_gpt.layer_norm(v, w[name + ".weight"], None, 1e-5)

    def running_mean(y, prefix):
        return w[prefix + "mix.gain"] * y.cumsum(0) / counts

    def qkv_of(y, prefix, n_head, n_kv):
        qkv = y @ w[prefix + "attn.qkv.weight"].T
        q = (qkv[:, : n_head * 16] * flip).reshape(T, n_head, 16)
        k = (qkv[:, n_head * 16: (n_head + n_kv) * 16] * flip).reshape(T, n_kv, 16)
        v = qkv[:, (n_head + n_kv) * 16:].reshape(T, n_kv, 16)
        return q, k, v

    def attend(q, k, v, prefix, window):
        n_head, n_kv = q.shape[1], k.shape[1]
        allowed = pos[None, :] <= pos[:, None]
        if window is not None:
            allowed &= pos[None, :] > pos[:, None] - window
        out = torch.zeros(T, n_head, 16, dtype=torch.float64)
        for h in range(n_head):
            s = (q[:, h] @ k[:, h // (n_head // n_kv)].T) / 4.0
            out[:, h] = torch.softmax(s.masked_fill(~allowed, float("-inf")), -1) @ v[:, h // (n_head // n_kv)]
        return out.reshape(T, -1) @ w[prefix + "attn.proj.weight"].T

    def dense(y, prefix):
        return plain_gpt.gelu_tanh(y @ w[prefix + "ff.fc.weight"].T) @ w[prefix + "ff.proj.weight"].T

    def experts(y, prefix):
        logits = y @ w[prefix + "moe.router.weight"].T
        if margins is not None:
            top = logits.sort(-1, descending=True).values
            margins.extend((top[:, 0] - top[:, 1]).tolist())
        out = torch.zeros_like(y)
        for t, e in enumerate(logits.argmax(-1).tolist()):
            out[t] = plain_gpt.gelu_tanh(y[t] @ w[prefix + f"moe.e{e}.fc.weight"].T) @ w[prefix + f"moe.e{e}.proj.weight"].T
        return out

    x = x + running_mean(ln(x, "l0.n1"), "l0.")
    x = x + dense(ln(x, "l0.n2"), "l0.")
    q, k1, v1 = qkv_of(ln(x, "l1.n1"), "l1.", 2, 1)            # keys and values of layer 1's first run
    x = x + attend(q, k1, v1, "l1.", TOY_WINDOW)
    x = x + dense(ln(x, "l1.n2"), "l1.")
    x = x + running_mean(ln(x, "l2.n1"), "l2.")
    x = x + experts(ln(x, "l2.n2"), "l2.")
    y = ln(x, "l3.n")                                           # one norm, two branches
    q, k, v = qkv_of(y, "l3.", 4, 2)
    x = x + attend(q, k, v, "l3.", None) + dense(y, "l3.")
    q, _, _ = qkv_of(ln(x, "l1.n1"), "l1.", 2, 1)               # second run: new queries, the old cache
    x = x + attend(q, k1, v1, "l1.", TOY_WINDOW)
    x = x + dense(ln(x, "l1.n2"), "l1.")
    return ln(x, "nf") @ w["emb.weight"].T


def test_toy_mixer_alone_matches_its_formula(ops):
    part = MIXERS.build(PartSpec("toy_running_mean", {"width": 12}, "mix"), "", position=None)
    part.bind({"mix.gain": torch.full((12,), 2.0, device=DEV)})
    manager = CacheManager([part.cache_spec()], 8, 4, 4)
    storage = CacheStorage(manager, torch.float32, DEV)
    ctx = make_ctx(ops, torch.float32, [5, 3], manager, storage)
    y = torch.randn(8, 12, device=DEV)
    residual = torch.zeros(8, 12, device=DEV)
    part.forward(ctx, ctx.cache_view(0), y, residual)
    want = torch.cat([2 * y[:5].cumsum(0) / torch.arange(1, 6, device=DEV)[:, None],
                      2 * y[5:].cumsum(0) / torch.arange(1, 4, device=DEV)[:, None]])
    assert torch.allclose(residual, want, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_routed_feed_forward_alone_matches_its_formula(ops, dtype):
    part = FEED_FORWARDS.build(PartSpec("toy_top1_experts", {"width": 40, "inner": 56, "experts": 4}, "moe"), "")
    w = bind_random(part, dtype, 17)
    ctx = make_ctx(ops, dtype, [9, 14])
    y = (torch.randn(23, 40, generator=torch.Generator().manual_seed(18)) * 2).to(dtype).to(DEV)
    residual = torch.zeros(23, 40, device=DEV)
    part.forward(ctx, y, residual)
    yd = y.double().cpu()
    choice = (y.float() @ part.router_weight.float().T).argmax(-1).cpu()     # as the part computes it
    assert len(set(choice.tolist())) >= 3, "the inputs were meant to reach several experts"
    want = torch.zeros(23, 40, dtype=torch.float64)
    for t in range(23):
        e = int(choice[t])
        h = plain_gpt.gelu_tanh(yd[t] @ w[f"moe.e{e}.fc.weight"].double().T)
        if dtype == torch.bfloat16:
            h = h.to(torch.bfloat16).double()
        want[t] = h @ w[f"moe.e{e}.proj.weight"].double().T
    assert rel_err(residual.cpu(), want) <= (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(ops, dtype):
    """Built from the registries alone, stepped whole and in portions with two requests side by
    side, and compared with the plain computation above: a mixer with state of its own (twice), a
    windowed attention layer that runs twice against one cache, a routed feed-forward, a layer
    with one norm and two branches, and two paged cache groups with different page sizes and
    pool sizes."""
    from mini_gpt_inference_b200.config import lookup
    from mini_gpt_inference_b200.parts import DecoderModel

    cfg = ToyConfig(vocab_size=97, width=32)
    family = lookup("ToyStateLM")
    model = DecoderModel(family.describe(cfg))
    specs = model.cache_specs()
    assert isinstance(specs[0], FixedStateSpec) and isinstance(specs[2], FixedStateSpec)
    # (a seed whose router logits have no near-ties on the two sequences below)
    tensors = random_tensors(model, 22, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    loaded = load_model(config=cfg, tensors=tensors, dtype=dtype, device=DEV)
    runner = make_runner(loaded, ops, page_tokens=4, num_pages=12, max_requests=3)
    groups = runner.manager.groups
    assert [(g.page_tokens, g.num_pages, g.layers) for g in groups] == [(4, 12, [1]), (8, 9, [3])]
    assert sorted(runner.manager.state_layers) == [0, 2]
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 97, (30,), generator=g).tolist()
    b = torch.randint(0, 97, (21,), generator=g).tolist()
    margins = []
    want_a, want_b = plain_toy_logits(a, tensors, margins), plain_toy_logits(b, tensors, margins)
    # routing is an argmax: the comparison is meaningful where rounding cannot flip it
    assert min(margins) > (1e-4 if dtype == "float32" else 2e-2), "choose weights with clearer routing"
    tol = 2e-5 if dtype == "float32" else 3e-2
    whole_a = runner.step([StepEntry("a", a, list(range(30)))])
    whole_b = runner.step([StepEntry("b", b, list(range(21)))])
    assert (whole_a.double().cpu() - want_a).abs().max() <= tol
    assert (whole_b.double().cpu() - want_b).abs().max() <= tol
    runner.finish("a")
    runner.finish("b")
    # the same two requests in portions, side by side, in fresh slots and pages
    got_a, got_b, pa, pb = [], [], 0, 0
    for na, nb in [(7, 1), (1, 9), (2, 1), (11, 2), (9, 8)]:
        out = runner.step([StepEntry("a2", a[pa: pa + na], list(range(na))),
                           StepEntry("b2", b[pb: pb + nb], list(range(nb)))])
        got_a.append(out[:na])
        got_b.append(out[na:])
        pa, pb = pa + na, pb + nb
        runner.manager.check()
    assert (torch.cat(got_a).double().cpu() - want_a).abs().max() <= tol
    assert (torch.cat(got_b).double().cpu() - want_b).abs().max() <= tol
    # the window (6) let pages go back early: 30 tokens never held more than 3 pages of 4 there;
    # the other group keeps every key: 30 + 21 tokens in pages of 8
    assert groups[0].pool.num_used <= 6 and groups[1].pool.num_used == 4 + 3
    # a slot that held state is given to a newcomer, which must start from zero: release one
    # request and recompute it beside the other
    runner.finish("a2")
    again = runner.step([StepEntry("a3", a[:17], list(range(17)))])
    assert (again.double().cpu() - want_a[:17]).abs().max() <= tol
    runner.finish("a3")
    runner.finish("b2")
    assert runner.manager.stats()["allocated_blocks"] == 0
