#!/usr/bin/env python3
"""Serving benchmark: decode tokens per second of the GPT-2 style 50M decoder on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--sizes 50m|gpt2-small|gpt2-xl] [--layers L] [--batch B] [--context S]

A "step" is one decode step: every request of the batch advances by one token.  The default
run has the layer sizes of the 50M configuration (8 layers, width 512, 8 heads of 64, MLP
2048, vocabulary 50304, 2048 positions, biases on, tied head) with seeded random weights in
bfloat16, a batch of 8 and contexts that end at 2048 tokens.  One JSON line is printed:

* ``value``: decoded tokens per second from the device time of K decode steps (CUDA events
  around each step's work on the stream; L2 is flushed between steps, outside the events; a
  step takes the tokens that the step before sampled on the device, as the engine does in
  steady decoding, so the host prepares the next step while the device runs this one);
* ``e2e``: the same through ``LLMEngine.step()`` with host token ids in and out, wall clock;
* ``prefill``: one 2,048-token prompt; ``roofline``: bytes a decode step must read / its time;
* ``points``: decode at batch 1 and 64.

``--only serve`` prints a line of its own: 64 requests (prompts of 16 to 512 tokens, 256 greedy
tokens each) through ``LLMEngine.generate``, wall clock: the scheduler's mixed batches.

``--only kernels`` prints the device time of each function of the kernel library in one decode step
and one 2,048-token prompt (an event pair around every launch; the reference sums its kernels' time
from a profiler's trace, bench/bench_kernels.py:71-116).

``--sizes`` runs the same measurement at the layer sizes of GPT-2 small or GPT-2 XL (position
table of 1,024: the prefill step is then two whole prompts of 1,024 tokens).

The reference's own benchmark times decode the same way — prefill untimed, then per-token
steps (bench/bench_hardware.py:96-128) — on its static cache; ``--impl reference`` runs that
unmodified code from ``baseline/_ref`` at the same sizes.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes by name.  The default is the 50M model; the two others are the same architecture at
# the layer sizes of GPT-2 small and GPT-2 XL (random weights), for measurements at further sizes.
SIZES = {
    "50m": dict(vocab_size=50304, n_positions=2048, n_layer=8, n_head=8, n_embd=512, n_inner=2048,
                bias=True, layer_norm_epsilon=1e-5),
    "50m-long": dict(vocab_size=50304, n_positions=16384, n_layer=8, n_head=8, n_embd=512, n_inner=2048,
                     bias=True, layer_norm_epsilon=1e-5),
    "gpt2-small": dict(vocab_size=50257, n_positions=1024, n_layer=12, n_head=12, n_embd=768,
                       n_inner=3072, bias=True, layer_norm_epsilon=1e-5),
    "gpt2-xl": dict(vocab_size=50257, n_positions=1024, n_layer=48, n_head=25, n_embd=1600,
                    n_inner=6400, bias=True, layer_norm_epsilon=1e-5),
}
MODEL_NAMES = {"50m": "gpt2-style-50M", "50m-long": "gpt2-style-50M with a position table of 16384", "gpt2-small": "gpt2-small-sizes", "gpt2-xl": "gpt2-xl-sizes"}
MODEL = SIZES["50m"]
BASELINE_T4_DECODE_B8 = 1671.8      # tok/s, Tesla T4 fp16, context 8..40 (docs/BENCHMARKS.md:622)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PREFILL_TOKENS = 2048


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--sizes", choices=sorted(SIZES), default="50m",
                    help="layer sizes: the 50M model (default), the same with a position table of 16384 "
                         "(for contexts beyond 2048: give --context), or the same architecture at "
                         "the layer sizes of GPT-2 small / GPT-2 XL")
    ap.add_argument("--context", type=int, default=None, help="default: the position table's length")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--page-tokens", type=int, default=64)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and prefill")
    ap.add_argument("--only", choices=["all", "decode", "prefill", "serve", "kernels"], default="all",
                    help="a small case for profilers: only the device-timed decode steps, or only "
                         "the 2,048-token prefill (the printed line is then partial); serve: 64 "
                         "requests with prompts of 16 to 512 tokens and 256 generated tokens each "
                         "through LLMEngine.generate (mixed batches, wall clock)")
    args = ap.parse_args()
    global MODEL
    MODEL = SIZES[args.sizes]
    args.context = args.context or MODEL["n_positions"]
    args.layers = args.layers or MODEL["n_layer"]
    return args


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(raw.get(key), (int, float)):
                    out[key] = float(raw[key])
            return out, "measured"
        except (json.JSONDecodeError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML (read-only) every few
    milliseconds while a region is timed."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
               "sw_power_cap": 0x4}

    def __init__(self, index: int = 0, period_s: float = 0.005) -> None:
        self.index, self.period_s = index, period_s
        self.sm: list[int] = []
        self.reason_bits = 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None

    def start(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001 - no NVML: report that instead of clocks
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def _loop(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.sm.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period_s)

    def stop(self) -> dict:
        if self._nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._stop.set()
        self._thread.join(timeout=2)
        reasons = sorted(k for k, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(self.sm)}


# ---- this engine ---------------------------------------------------------------------------------
def build_engine(args, batch: int, max_tokens_per_request: int):
    import torch

    from mini_gpt_inference_b200 import EngineConfig, GPTConfig, LLMEngine
    from mini_gpt_inference_b200.config import lookup
    from mini_gpt_inference_b200.engine.build import load_model
    from mini_gpt_inference_b200.parts import DecoderModel
    from mini_gpt_inference_b200.weights import random_tensors

    cfg = GPTConfig.from_dict({**MODEL, "n_layer": args.layers})
    key = (args.sizes, args.layers, args.dtype)
    if key not in build_engine.cache:
        model = DecoderModel(lookup(cfg.architecture).describe(cfg))
        store = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
        tensors = random_tensors(model, 0, store)
        build_engine.cache[key] = load_model(config=cfg, tensors=tensors, dtype=args.dtype,
                                             device="cuda:0")
    loaded = build_engine.cache[key]
    pt = args.page_tokens
    pages = batch * ((max_tokens_per_request + pt - 1) // pt) + 4
    ecfg = EngineConfig(block_size=pt, num_blocks=pages, max_batch_size=max(batch, 1),
                        max_num_batched_tokens=2048, dtype=args.dtype, device="cuda:0")
    return cfg, LLMEngine(loaded, ecfg, seed=0)


build_engine.cache = {}


def metric_name(args) -> str:
    what = "GPT-2 style 50M" if args.sizes == "50m" else f"{args.sizes} layer sizes"
    return f"decode tok/s at batch {args.batch}, context {args.context} ({what}, random weights)"


def weight_bytes(cfg, dtype_bytes: int) -> int:
    """Bytes of every weight a decode step reads once: the matrices in the compute dtype, the
    vectors (biases, norm gains) in 32-bit, the embedding matrix once (as the output head)."""
    c, f, n_layer, v = cfg.n_embd, cfg.n_inner, cfg.n_layer, cfg.vocab_size
    matrices = n_layer * (3 * c * c + c * c + 2 * c * f) + v * c
    vectors = n_layer * (2 * c + (3 * c + c + f + c + 2 * c if cfg.bias else 0)) + (2 * c if cfg.bias else c)
    return matrices * dtype_bytes + vectors * 4


def kv_bytes(cfg, batch: int, context: float, dtype_bytes: int) -> float:
    return batch * context * 2 * cfg.n_layer * cfg.n_embd * dtype_bytes


def prefill_flops(cfg, tokens: int) -> float:
    c, f = cfg.n_embd, cfg.n_inner
    linear = 2.0 * tokens * cfg.n_layer * (3 * c * c + c * c + 2 * c * f)
    attention = cfg.n_layer * 2.0 * c * tokens * (tokens + 1)      # QK^T and PV over the causal half
    head = 2.0 * c * cfg.vocab_size                                  # logits of the last row only
    return linear + attention + head


def window_stats(per_window_ms: list) -> dict:
    """Median and interquartile range of the windows' mean step times."""
    ordered = sorted(per_window_ms)
    n = len(ordered)
    q1, q3 = ordered[n // 4], ordered[(3 * n) // 4 if n > 1 else 0]
    return {"count": n, "median_ms": round(statistics.median(ordered), 4),
            "iqr_ms": round(q3 - q1, 4), "min_ms": round(ordered[0], 4), "max_ms": round(ordered[-1], 4)}


def device_decode(args, batch: int, steps: int, warmup: int, clock_sampler=None, min_seconds: float = 0.5,
                  max_windows: int = 96, flush_l2: bool = True):
    """Windows of K decode steps of `batch` requests whose contexts end at args.context; device
    time.  A window prefills fresh requests (untimed), runs W warm-up steps and times exactly K
    steps with CUDA events around each step; windows are repeated until `min_seconds` of device
    time have been timed (at most `max_windows`).  Returns the mean step time of each window."""
    import torch

    from mini_gpt_inference_b200.config import SamplingParams
    from mini_gpt_inference_b200.engine.runner import StepEntry

    cfg, engine = build_engine(args, batch, args.context)
    runner, sampler = engine.runner, engine.sampler
    prompt_len = args.context - (steps + warmup)
    gen = torch.Generator().manual_seed(1)
    rids = [f"d{i}" for i in range(batch)]
    greedy = [SamplingParams(temperature=0.0)] * batch
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda:0") if flush_l2 else None
    feed = list(range(batch))
    per_window, launches, timed = [], 0, 0.0
    while len(per_window) < max_windows and (timed < min_seconds or not per_window):
        for rid in rids:                                   # prefill, untimed
            prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen).tolist()
            runner.step([StepEntry(rid, prompt, [])])
        last = torch.randint(0, cfg.vocab_size, (batch,), generator=gen).tolist()
        events, ids = [], None
        launches_before = getattr(runner.ops, "launches", 0)
        torch.cuda.synchronize()
        for step in range(steps + warmup):
            if flush is not None:
                flush.zero_()                              # evict L2 between steps, outside the events
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if step == warmup:
                torch.cuda.synchronize()
                launches_before = getattr(runner.ops, "launches", 0)
                if clock_sampler is not None and not per_window:
                    clock_sampler.start()                   # clocks of the timed steps of all windows
            start.record()
            if ids is None:
                logits = runner.step([StepEntry(rid, [tok], [0]) for rid, tok in zip(rids, last)], copy=False)
            else:
                # the tokens sampled by the step before are taken on the device, as the engine does
                # in steady decoding: the host prepares this step while the device runs the last one
                logits = runner.step([StepEntry(rid, [0], [0]) for rid in rids], copy=False,
                                     token_sources=feed, previous_ids=ids)
            ids = sampler.sample(logits, greedy, [0] * batch, [step] * batch,
                                 greedy_ids=runner.greedy_ids(batch), out=runner.sampled_ids[:batch])
            end.record()
            events.append((start, end))
        torch.cuda.synchronize()
        ids.tolist()                                       # device -> host: the last step's result
        times = [a.elapsed_time(b) for a, b in events[warmup:]]
        per_window.append(statistics.fmean(times))
        timed += sum(times) * 1e-3
        launches = getattr(runner.ops, "launches", 0) - launches_before
        for rid in rids:
            runner.finish(rid)
    clocks = clock_sampler.stop() if clock_sampler is not None else None
    runner.ops.check_status()
    mean_context = args.context - steps / 2.0
    return cfg, per_window, launches, mean_context, clocks


def e2e_decode(args, batch: int, steps: int, warmup: int, min_seconds: float = 0.3, max_windows: int = 48):
    """The same through LLMEngine.step(): host token ids in, sampled ids out, wall clock.  Windows
    of K steps on fresh requests, repeated like the device-timed ones; the median window counts."""
    import torch

    from mini_gpt_inference_b200 import Request, SamplingParams

    cfg, engine = build_engine(args, batch, args.context)
    # requests finish their prompts a few steps apart; leave room so that none runs out of
    # tokens inside the timed steps
    max_tokens = steps + warmup + batch + 8
    prompt_len = args.context - max_tokens
    gen = torch.Generator().manual_seed(2)
    rates, walls, total, window = [], [], 0.0, 0
    h2d = None
    while window < max_windows and (total < min_seconds or not rates):
        for i in range(batch):
            prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen).tolist()
            engine.add_request(Request(f"e{window}_{i}", prompt, SamplingParams(max_tokens=max_tokens,
                                                                                 temperature=0.0)))
        # prompts first (untimed), until every request is decoding
        while any(s.num_pending_tokens > 1 or s.num_computed_tokens == 0
                  for s in list(engine.scheduler.running) + list(engine.scheduler.waiting)):
            engine.step()
        for _ in range(warmup - 1):
            engine.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += len(engine.step())
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        h2d = engine.runner.last_h2d_bytes if hasattr(engine.runner, "last_h2d_bytes") else None
        while engine.has_unfinished_requests():
            engine.step()
        rates.append(produced / wall)
        walls.append(wall / steps * 1e3)
        total += wall
        window += 1
    return statistics.median(rates), statistics.median(walls), h2d, batch * 4, len(rates)


def prefill_once(args, reps: int = 6):
    """One step of 2,048 prompt tokens: one prompt where the position table holds it, else as
    many whole prompts of the table's length as make 2,048 tokens (two of 1,024)."""
    import torch

    from mini_gpt_inference_b200.engine.runner import StepEntry

    length = min(PREFILL_TOKENS, MODEL["n_positions"])
    count = PREFILL_TOKENS // length
    cfg, engine = build_engine(args, count, length)
    runner = engine.runner
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (length,), generator=gen).tolist() for _ in range(count)]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda:0")
    times = []
    for rep in range(reps):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        logits = runner.step([StepEntry(f"p{i}", p, [length - 1]) for i, p in enumerate(prompts)])
        end.record()
        torch.cuda.synchronize()
        assert logits.shape == (count, cfg.vocab_size)
        for i in range(count):
            runner.finish(f"p{i}")
        if rep >= min(2, reps - 1):
            times.append(start.elapsed_time(end))
    runner.ops.check_status()
    return cfg, statistics.median(times), length, count


def serve_mixed(args, requests: int = 64, new_tokens: int = 256) -> dict:
    """Many requests at once through the public entry point: prompts of 16 to 512 uniform random
    tokens, `new_tokens` greedy tokens each; the scheduler mixes prompt portions with decoding.
    Wall clock from the first add_request to the last token, host token ids in and out."""
    import torch

    from mini_gpt_inference_b200 import SamplingParams

    longest = min(512, MODEL["n_positions"] - new_tokens)
    cfg, engine = build_engine(args, requests, longest + new_tokens)
    gen = torch.Generator().manual_seed(4)
    lengths = torch.randint(16, longest + 1, (requests,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    params = SamplingParams(max_tokens=new_tokens, temperature=0.0)
    # Warm-up: as many other requests (other lengths, so no prompt step of the timed run has been seen
    # before) for a few tokens: a server that has been up for a minute has captured the decode graph
    # of every batch size it meets; the clock below does not pay for that once more.
    warm = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()
            for n in torch.randint(16, longest + 1, (requests,), generator=gen).tolist()]
    engine.generate(warm, SamplingParams(max_tokens=6, temperature=0.0))
    before = engine.stats()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    after = engine.stats()
    generated = sum(len(o["token_ids"]) for o in outs)
    return {"impl": "ours", "partial": "serve", "model": MODEL_NAMES[args.sizes], "requests": requests,
            "prompt_tokens": sum(lengths), "generated_tokens": generated, "seconds": round(wall, 4),
            "value": round(generated / wall, 1), "unit": "generated tokens/s",
            "warmup": f"{requests} other requests of 6 tokens (decode graphs exist before the clock starts)",
            "steps": after["steps"] - before["steps"],
            "preemptions": after["preemptions"] - before["preemptions"],
            "finish_reasons": sorted({o["finish_reason"] for o in outs})}


def kernel_times(args) -> dict:
    """Device time of each exported function of the kernel library in one decode step at the
    headline batch and in one 2,048-token prompt, launches issued one by one with an event before
    and after each (no CUDA graph, nothing overlaps: shares, not the step's time)."""
    import torch

    from mini_gpt_inference_b200.engine.runner import StepEntry
    from mini_gpt_inference_b200.kernels.timing import LaunchTimer

    batch = args.batch
    cfg, engine = build_engine(args, batch + 1, args.context)
    runner = engine.runner
    runner.use_cuda_graphs = False
    gen = torch.Generator().manual_seed(1)
    rids = [f"k{i}" for i in range(batch)]
    for rid in rids:
        runner.step([StepEntry(rid, torch.randint(0, cfg.vocab_size, (args.context - 4,), generator=gen).tolist(), [])])
    out = {"impl": "ours", "partial": "device time of each launch, issued one by one", "batch": batch,
           "context": args.context}
    for name, entries in (
            ("decode", lambda: [StepEntry(rid, [7], [0]) for rid in rids]),
            ("prefill", lambda: [StepEntry("kp", torch.randint(0, cfg.vocab_size, (min(PREFILL_TOKENS, args.context),),
                                                               generator=gen).tolist(), [min(PREFILL_TOKENS, args.context) - 1])])):
        for rep in range(3):                               # the third pass is the one reported
            with LaunchTimer(runner.ops) as timer:
                runner.step(entries())
            rows = timer.summary()
            if name == "prefill":
                runner.finish("kp")
        out[name] = [{"function": r.name, "calls": r.calls, "total_us": round(r.total_us, 1),
                      "mean_us": round(r.mean_us, 2), "share": round(r.share, 3)} for r in rows]
        out[name + "_total_us"] = round(sum(r.total_us for r in rows), 1)
    for rid in rids:
        runner.finish(rid)
    runner.ops.check_status()
    return out


def check_decode_logits(args) -> dict:
    """Outside every timed region: the decode step that the benchmark times (batch 8, contexts of
    2,048, the replayed graph) is run once on fixed tokens and its logits are compared with rows
    that the tests' plain implementation computed for the same weights and tokens
    (tests/golden/bench_decode_rows.json, written by tests/golden/make_bench_rows.py).  Raises if
    they differ by more than the bfloat16 tolerance of the tests (3% of the logits' spread)."""
    import torch

    from mini_gpt_inference_b200.engine.runner import StepEntry

    path = ROOT / "tests" / "golden" / "bench_decode_rows.json"
    if not path.is_file():
        return {"checked": False, "why": "tests/golden/bench_decode_rows.json is absent"}
    stored = json.loads(path.read_text())
    same = (args.sizes == "50m" and args.dtype == "bfloat16" and args.layers == stored["config"]["n_layer"]
            and all(MODEL[k] == v for k, v in stored["config"].items()))
    if not same:
        return {"checked": False, "why": "rows are stored for the default configuration only"}
    batch, length = stored["tokens"]["batch"], stored["tokens"]["length"]
    check_args = argparse.Namespace(**{**vars(args), "context": length})
    cfg, engine = build_engine(check_args, batch, length)
    runner = engine.runner
    gen = torch.Generator().manual_seed(stored["tokens"]["seed"])
    tokens = [torch.randint(0, cfg.vocab_size, (length,), generator=gen).tolist() for _ in range(batch)]
    for i, t in enumerate(tokens):
        runner.step([StepEntry(f"c{i}", t[:-1], [])])
    replays = runner.graph_replays
    logits = runner.step([StepEntry(f"c{i}", t[-1:], [0]) for i, t in enumerate(tokens)])
    torch.cuda.synchronize()
    runner.ops.check_status()
    columns = torch.tensor(stored["columns"], device=logits.device)
    got = logits[:, columns].double().cpu()
    want = torch.tensor(stored["logits"], dtype=torch.float64)
    diff = float((got - want).abs().max())
    tol = 0.03 * stored["logits_std"]
    for i in range(batch):
        runner.finish(f"c{i}")
    out = {"checked": True, "max_abs_diff": round(diff, 6), "tolerance": round(tol, 6),
           "argmax_equal": logits.argmax(-1).tolist() == stored["argmax"],
           "graph_replayed": runner.graph_replays == replays + 1}
    if not diff <= tol:
        raise SystemExit(f"bench.py: the decode step's logits differ from the plain implementation's: {out}")
    return out


def run_ours(args) -> dict:
    global MODEL
    import torch

    pk, peak_source = peaks()
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    if args.only == "prefill":
        cfg, pre_ms, _, _ = prefill_once(args)
        return {"impl": "ours", "partial": "prefill only", "prefill": {
            "value": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 4)}}
    if args.only == "serve":
        return serve_mixed(args)
    if args.only == "kernels":
        return kernel_times(args)
    if args.only == "decode":
        cfg, windows, launches, mean_ctx, clocks = device_decode(args, args.batch, args.steps, args.warmup,
                                                                 min_seconds=0.0)
        ms = statistics.median(windows)
        return {"impl": "ours", "partial": "decode only", "value": round(args.batch / (ms * 1e-3), 1),
                "ms_per_step": round(ms, 4), "gpu_launches": launches}

    def roofline_of(cfg, batch, mean_ctx, ms, nbytes=dtype_bytes):
        step_bytes = weight_bytes(cfg, nbytes) + kv_bytes(cfg, batch, mean_ctx, nbytes)
        return step_bytes, step_bytes / (ms * 1e-3) / 1e9

    cfg, windows, launches, mean_ctx, clocks = device_decode(args, args.batch, args.steps, args.warmup,
                                                             ClockSampler(0))
    ms = statistics.median(windows)                 # the median window of K steps is the reported one
    value = args.batch / (ms * 1e-3)
    step_bytes, achieved = roofline_of(cfg, args.batch, mean_ctx, ms)
    e2e_value, e2e_ms, h2d, d2h, e2e_windows = e2e_decode(args, args.batch, args.steps, args.warmup)
    line = {
        "metric": metric_name(args),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": round(value / BASELINE_T4_DECODE_B8, 2),
        "baseline_note": "published reference number is Tesla T4 fp16 at context 8..40 (1671.8 tok/s)",
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": MODEL_NAMES[args.sizes], "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single-gpu", "n_layer": args.layers, "n_layer_config": MODEL["n_layer"],
            "n_embd": cfg.n_embd, "n_head": cfg.n_head, "head_dim": cfg.head_dim,
            "n_inner": cfg.n_inner, "vocab_size": cfg.vocab_size, "n_positions": cfg.n_positions,
            "bias": cfg.bias, "tied_head": True, "page_tokens": args.page_tokens,
            "l2": "flushed between timed steps (256 MiB write)", "weights": "random seed 0",
            "mean_context": mean_ctx, "peaks": peak_source,
        },
        # windows of exactly K timed steps on freshly prefilled requests, repeated until half a
        # second of device time is timed; `value` is the median window
        "windows": window_stats(windows),
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "windows": e2e_windows},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "bytes_per_step": int(step_bytes), "of": peak_source},
    }
    if not args.no_points:
        points = {}
        small_k, small_w = min(args.steps, 64), max(3, min(args.warmup, 8))
        for b in (1, 64):
            _, t, _, ctx_b, _ = device_decode(args, b, small_k, small_w, min_seconds=0.25)
            ms_b = statistics.median(t)
            points[f"decode_b{b}"] = round(b / (ms_b * 1e-3), 1)
            points[f"decode_b{b}_roofline_frac"] = round(roofline_of(cfg, b, ctx_b, ms_b)[1] / pk["hbm_gbs"], 4)
        # the same step with whatever the step before left in L2 (no flush between steps)
        _, t, _, _, _ = device_decode(args, args.batch, small_k, small_w, min_seconds=0.1, flush_l2=False)
        points[f"decode_b{args.batch}_no_l2_flush"] = round(args.batch / (statistics.median(t) * 1e-3), 1)
        _, pre_ms, pre_len, pre_count = prefill_once(args)
        flops = pre_count * prefill_flops(cfg, pre_len)
        peak = pk["bf16_tflops"] if args.dtype == "bfloat16" else None
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                           "prompts": pre_count, "ms": round(pre_ms, 4),
                           "frac": round(flops / (pre_ms * 1e-3) / (peak * 1e12), 4) if peak else None,
                           "of": peak_source}
        if args.dtype == "bfloat16":
            # the true 32-bit path of the same model (FMA kernels, 32-bit weights and cache)
            args32 = argparse.Namespace(**{**vars(args), "dtype": "float32"})
            _, t, _, ctx32, _ = device_decode(args32, args.batch, min(args.steps, 16), 3, min_seconds=0.0,
                                              max_windows=2)
            ms32 = statistics.median(t)
            points[f"decode_b{args.batch}_fp32"] = round(args.batch / (ms32 * 1e-3), 1)
            points[f"decode_b{args.batch}_fp32_roofline_frac"] = round(
                roofline_of(cfg, args.batch, ctx32, ms32, 4)[1] / pk["hbm_gbs"], 4)
            _, pre32, _, _ = prefill_once(args32, reps=3)
            points["prefill_fp32_tok_s"] = round(PREFILL_TOKENS / (pre32 * 1e-3), 1)
            build_engine.cache.pop((args.sizes, args.layers, "float32"), None)     # give the memory back
        if args.sizes == "50m" and args.dtype == "bfloat16":
            # the same layers with a position table of 16384: the cache's share of a step grows eightfold
            keep, MODEL = MODEL, SIZES["50m-long"]
            try:
                args_long = argparse.Namespace(**{**vars(args), "sizes": "50m-long", "context": 16384})
                cfg_long, t, _, ctx_long, _ = device_decode(args_long, args.batch, min(args.steps, 32), 4,
                                                            min_seconds=0.0, max_windows=2)
                ms_long = statistics.median(t)
                points[f"decode_b{args.batch}_ctx16384"] = round(args.batch / (ms_long * 1e-3), 1)
                points[f"decode_b{args.batch}_ctx16384_roofline_frac"] = round(
                    roofline_of(cfg_long, args.batch, ctx_long, ms_long)[1] / pk["hbm_gbs"], 4)
                build_engine.cache.pop(("50m-long", args.layers, "bfloat16"), None)    # give the memory back
            finally:
                MODEL = keep
        serve = serve_mixed(args)
        points["serve_64_requests_tok_s"] = serve["value"]
        line["points"] = points
        line["logits_check"] = check_decode_logits(args)
    torch.cuda.synchronize()
    return line


# ---- the reference, unmodified, from baseline/_ref --------------------------------------------------
def run_reference(args) -> dict:
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "minigpt_infer").is_dir():
        return {"impl": "reference",
                "unavailable": "baseline/_ref is not installed (pip install --no-index --no-deps "
                               "--target baseline/_ref of the reference has not been run here)"}
    sys.path.insert(0, str(ref_root))
    try:
        import torch
        from minigpt_infer.batch import ForwardBatch
        from minigpt_infer.cache.static import StaticKVCache
        from minigpt_infer.config import GPTConfig as RefConfig
        from minigpt_infer.model import GPT
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    torch.manual_seed(0)
    cfg = RefConfig(vocab_size=MODEL["vocab_size"], block_size=args.context, n_layer=args.layers,
                    n_head=MODEL["n_head"], n_embd=MODEL["n_embd"], dropout=0.0, bias=MODEL["bias"])
    model = GPT(cfg).to(device="cuda", dtype=dtype).eval()
    batch, steps, warmup = args.batch, args.steps, args.warmup
    prompt_len = args.context - (steps + warmup)
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (batch, prompt_len), generator=gen).cuda()
    sampler = ClockSampler(0)
    with torch.no_grad():
        # the reference's decode-only timing (bench/bench_hardware.py:63-92): prefill untimed,
        # then one forward per token on the static cache, argmax on the device
        cache = StaticKVCache(n_layer=cfg.n_layer, n_head=cfg.n_head, head_dim=model.head_dim,
                              max_batch_size=batch, max_seq_len=cfg.block_size, device="cuda", dtype=dtype)
        pos = torch.arange(prompt_len, device="cuda").unsqueeze(0).expand(batch, -1)
        logits = model(ForwardBatch(input_ids=prompt, position_ids=pos, is_prefill=True, cache=cache))
        cache.advance(prompt_len, batch)
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
        times, wall = [], 0.0
        sampler.start()
        for step in range(steps + warmup):
            flush.zero_()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            next_id = torch.argmax(logits, dim=-1, keepdim=True)
            cur_len = int(cache.seq_lens[0].item())
            p = torch.full((batch, 1), cur_len, device="cuda", dtype=torch.long)
            logits = model(ForwardBatch(input_ids=next_id, position_ids=p, is_prefill=False, cache=cache))
            cache.advance(1, batch)
            end.record()
            host_ids = next_id.cpu()
            torch.cuda.synchronize()
            if step >= warmup:
                times.append(start.elapsed_time(end))
                wall += time.perf_counter() - t0
        clocks = sampler.stop()
        assert host_ids.shape == (batch, 1)
        # How much of a step the device is busy: the sum of the kernels' own durations over a few
        # further steps (the events above bracket the host's work between launches as well).  The
        # timed steps have filled the cache to its end, so these run on a second cache, right after
        # the same prompt.
        busy_ms = None
        try:
            from torch.profiler import ProfilerActivity, profile

            probe_steps = 3
            del cache
            cache = StaticKVCache(n_layer=cfg.n_layer, n_head=cfg.n_head, head_dim=model.head_dim,
                                  max_batch_size=batch, max_seq_len=cfg.block_size, device="cuda", dtype=dtype)
            logits = model(ForwardBatch(input_ids=prompt, position_ids=pos, is_prefill=True, cache=cache))
            cache.advance(prompt_len, batch)
            torch.cuda.synchronize()
            ran = 0
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(probe_steps):
                    next_id = torch.argmax(logits, dim=-1, keepdim=True)
                    cur_len = int(cache.seq_lens[0].item())
                    if cur_len >= cfg.block_size:
                        break
                    p = torch.full((batch, 1), cur_len, device="cuda", dtype=torch.long)
                    logits = model(ForwardBatch(input_ids=next_id, position_ids=p, is_prefill=False, cache=cache))
                    cache.advance(1, batch)
                    ran += 1
                torch.cuda.synchronize()
            total_us = sum(getattr(e, "self_device_time_total", 0.0) for e in prof.key_averages())
            busy_ms = round(total_us / 1e3 / ran, 4) if total_us and ran else None
        except Exception:  # noqa: BLE001 - no profiler on this machine: the figure is left out
            busy_ms = None
    ms = statistics.fmean(times)
    return {
        "metric": metric_name(args),
        "value": round(batch / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(batch / (ms * 1e-3) / BASELINE_T4_DECODE_B8, 2),
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic", "impl": "reference",
        "config": {"model": MODEL_NAMES[args.sizes], "global_batch": batch, "seq_len": args.context,
                   "parallelism": "single-gpu", "n_layer": args.layers, "n_layer_config": MODEL["n_layer"],
                   "path": "GPT + StaticKVCache, eager (bench/bench_hardware.py method)",
                   "l2": "flushed between timed steps (256 MiB write)"},
        "e2e": {"value": round(batch * steps / wall, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": batch * 8},
        "gpu_launches": 0, "clocks": clocks,
        # kernels' own time per step beside the event time: far below it means the arm waits for its host
        "device_busy_ms_per_step": busy_ms,
    }


def main() -> int:
    args = parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.context - args.steps - args.warmup - 80 < 2:
        print("steps + warmup must leave room for a prompt inside the context", file=sys.stderr)
        return 2
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
