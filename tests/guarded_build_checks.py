"""Run by test_gpu_guards.py in a process of its own with MINIGPT_B200_GUARDS=1 (the build variant is
chosen when the kernel package is imported): drives the guarded build of the kernel library and
prints one JSON object with what it saw.

Every table that a bad index points beyond is a view of the first part of a larger tensor, so even
an access that a guard failed to stop would stay inside memory of this test; the part behind the
view must come out untouched.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import torch  # noqa: E402

from harness import PAGE_TOKENS, TOLERANCE, gpu_runner, make_tensors, plain_logits, tiny_config, tokens_for  # noqa: E402
from mini_gpt_inference_b200.config import GPTConfig  # noqa: E402
from mini_gpt_inference_b200.engine.runner import StepEntry  # noqa: E402
from mini_gpt_inference_b200.kernels.library import KernelLibraryError  # noqa: E402
from mini_gpt_inference_b200.kernels.ops import default_ops  # noqa: E402

ops = default_ops("cuda:0")
out: dict = {"guards": ops.guards}


def fault_of(run) -> str:
    """The message that check_indices raises after ``run``, or '' if it is quiet."""
    run()
    try:
        ops.check_indices()
    except KernelLibraryError as exc:
        return str(exc)
    return ""


# head size 64: the bfloat16 step runs the tensor-core projections and the prompt attention on them
HEAD64 = dict(vocab_size=1003, n_positions=700, n_layer=2, n_head=3, n_embd=192, n_inner=520, bias=True,
              layer_norm_epsilon=1e-5)


def engine_steps(tag: str) -> None:
    """A prompt in portions and some single tokens through the runner: right logits, quiet guards."""
    for which, dtype in (("A", "bfloat16"), ("B", "float32"), ("H", "bfloat16")):
        cfg = GPTConfig.from_dict(HEAD64) if which == "H" else tiny_config(which)
        tensors = make_tensors(cfg, 3, dtype, False)
        runner = gpu_runner(cfg, tensors, dtype, 16 if which == "H" else PAGE_TOKENS[which], 64)
        tokens = tokens_for(cfg, 300 if which == "H" else 45, 1)
        want = plain_logits(cfg, tensors, tokens)
        n, first = len(tokens), len(tokens) - 25
        got = [runner.step([StepEntry("r", tokens[:first], list(range(first)))]),
               runner.step([StepEntry("r", tokens[first: first + 13], list(range(13)))])]
        for t in range(first + 13, n):
            got.append(runner.step([StepEntry("r", tokens[t: t + 1], [0])]))
        diff = float((torch.cat(got).double().cpu() - want.double()).abs().max())
        runner.finish("r")
        ops.check_status()
        out[f"{tag}_{which}_{dtype}"] = {"diff": diff, "tolerance": TOLERANCE[dtype]}


engine_steps("before")

dev = "cuda:0"
i32 = dict(dtype=torch.int32, device=dev)

# ---- embedding: a token id beyond the vocabulary, a position beyond the table, a bad token source ----
big_tok = torch.randn(100, 16, device=dev)
big_pos = torch.randn(40, 16, device=dev)
tok, pos = big_tok[:50], big_pos[:20]
ids = torch.tensor([3, 77, 5], **i32)
positions = torch.tensor([0, 1, 2], **i32)
res = {}
out["token"] = fault_of(lambda: res.update(x=ops.embed(ids, positions, tok, pos)))
out["token_row_replaced"] = bool(torch.equal(res["x"][1], tok[0] + pos[1]) and torch.equal(res["x"][2], tok[5] + pos[2]))
out["position"] = fault_of(lambda: ops.embed(torch.tensor([1, 2], **i32), torch.tensor([4, 33], **i32), tok, pos))
previous = torch.tensor([9, 8, 7, 6], **i32)
out["source"] = fault_of(lambda: res.update(y=ops.embed(torch.tensor([1, 2], **i32), torch.tensor([0, 1], **i32), tok, pos,
                                                        source=torch.tensor([2, 11], **i32), previous=previous)))
out["source_row_kept"] = bool(torch.equal(res["y"][0], tok[7] + pos[0]) and torch.equal(res["y"][1], tok[2] + pos[1]))

# ---- row gather ----
big_x = torch.randn(12, 8, device=dev)
out["row"] = fault_of(lambda: ops.gather_rows(big_x[:6], torch.tensor([5, 9], **i32)))

# ---- cache rows: the page write as a kernel of its own and inside the projections ----
n_head, n_kv, d, pt, pages = 2, 2, 16, 8, 4


def fresh_cache(dtype):
    big_k = torch.zeros(2 * pages, n_kv, pt, d, dtype=dtype, device=dev)
    big_v = torch.zeros(2 * pages, n_kv, pt, d, dtype=dtype, device=dev)
    return big_k, big_v, SimpleNamespace(k_pages=big_k[:pages], v_pages=big_v[:pages], page_tokens=pt, writes=True,
                                         window=None, group=0)


def behind_untouched(big_k, big_v) -> bool:
    return bool((big_k[pages:] == 0).all() and (big_v[pages:] == 0).all())


for dtype in (torch.float32, torch.bfloat16):
    big_k, big_v, cache = fresh_cache(dtype)
    qkv = torch.randn(3, (n_head + 2 * n_kv) * d, device=dev).to(dtype)
    slots = torch.tensor([3, pages * pt + 5, -1], **i32)          # the second row points behind the pool
    name = "kv_store_" + str(dtype).split(".")[-1]
    out[name] = fault_of(lambda: ops.kv_store(qkv, n_head, n_kv, d, cache, slots))
    out[name + "_behind_untouched"] = behind_untouched(big_k, big_v)
    out[name + "_good_row_written"] = bool((cache.k_pages[0, :, 3] != 0).any())

for m, flags, name in ((3, {}, "skinny"), (40, {}, "cluster"), (200, {}, "tensor_cores"),
                       (3, {"stream_min_bytes": 0, "use_skinny": False, "use_cluster": False, "use_wide": False}, "stream"),
                       (3, {"stream_min_bytes": 0, "use_skinny": False, "use_cluster": False}, "wide")):
    big_k, big_v, cache = fresh_cache(torch.bfloat16)
    k = 64
    x = torch.randn(m, k, device=dev).bfloat16()
    w = (torch.randn((n_head + 2 * n_kv) * d, k, device=dev) / 8).bfloat16()
    slots = torch.full((m,), -1, **i32)
    slots[0], slots[m - 1] = 2, pages * pt + 1
    saved = {key: getattr(ops, key) for key in flags}
    for key, value in flags.items():
        setattr(ops, key, value)
    try:
        before = ops.launches
        out["sink_" + name] = fault_of(lambda: ops.linear_qkv(x, w, None, n_head, n_kv, d, cache, slots, torch.bfloat16))
        out["sink_" + name + "_one_launch"] = ops.launches == before + 1
    finally:
        for key, value in saved.items():
            setattr(ops, key, value)
    out["sink_" + name + "_behind_untouched"] = behind_untouched(big_k, big_v)
    out["sink_" + name + "_good_row_written"] = bool((cache.k_pages[0, :, 2] != 0).any())

# ---- attention: a page beyond the pool, a request beyond the block tables, a position beyond them ----
big_k, big_v, cache = fresh_cache(torch.bfloat16)
big_k.normal_()
big_v.normal_()
qkv = torch.randn(2, (n_head + 2 * n_kv) * d, device=dev).bfloat16()


def attention(table, requests, positions, decode):
    rows = torch.tensor(table + [[0] * len(table[0])] * 6, **i32)[: len(table)]     # (a view, like the other tables)
    ctx = SimpleNamespace(block_tables=[rows], token_request=torch.tensor(requests, **i32),
                          positions=torch.tensor(positions, **i32), decode_only=decode,
                          max_ctx_after=max(positions) + 1, extra={})
    return ops.paged_attention(qkv, n_head, n_kv, d, 0.25, cache, ctx)


good = [[0, 1, 2, 3], [3, 2, 1, 0]]
for decode, name in ((True, "split"), (False, "generic")):
    out[f"attention_{name}_quiet"] = fault_of(lambda: attention(good, [0, 1], [17, 9], decode))
    out[f"attention_{name}_page"] = fault_of(lambda: attention([[0, 1, pages + 2, 3], [3, 2, 1, 0]], [0, 1], [17, 9], decode))
    out[f"attention_{name}_request"] = fault_of(lambda: attention(good, [0, 5], [17, 9], decode))
    out[f"attention_{name}_position"] = fault_of(lambda: attention(good, [0, 1], [17, 4 * pt + 3], decode))

engine_steps("after")
print(json.dumps(out))
