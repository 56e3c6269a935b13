"""bench.py without a GPU: what it refuses, what its reference arm prints where the reference
cannot run, and the byte and flop counts behind the roofline figures."""

from __future__ import annotations

import importlib.util
import json
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_more_than_one_gpu_is_refused_with_one_line_and_code_2():
    run = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"], capture_output=True,
                         text=True, timeout=120)
    assert run.returncode == 2
    assert len(run.stdout.strip().splitlines()) == 1 and "single-GPU" in run.stdout


def test_reference_arm_says_unavailable_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        return                                   # on a GPU box the arm runs; covered by the bench itself
    run = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference"],
                         capture_output=True, text=True, timeout=300)
    assert run.returncode == 0
    line = json.loads(run.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_step_bytes_and_prefill_flops_of_the_50m_sizes():
    bench = _bench()
    m = bench.SIZES["50m"]
    cfg = SimpleNamespace(n_embd=m["n_embd"], n_inner=m["n_inner"], n_layer=m["n_layer"],
                          vocab_size=m["vocab_size"], bias=m["bias"])
    c, f, layers, v = 512, 2048, 8, 50304
    matrices = layers * (3 * c * c + c * c + 2 * c * f) + v * c          # position table is not read whole
    vectors = layers * (2 * c + 2 * c + 3 * c + c + f + c) + 2 * c      # norm gains and shifts, biases
    assert bench.weight_bytes(cfg, 2) == 2 * matrices + 4 * vectors
    # every parameter but the position table (2048 x 512): 52,024,320 in all
    assert matrices + vectors + 2048 * c == 52_024_320
    # keys and values: 2 x 8 layers x 512 x 2 bytes = 16 KiB a token
    assert bench.kv_bytes(cfg, 8, 2048, 2) == 8 * 2048 * 16 * 1024
    flops = bench.prefill_flops(cfg, 2048)
    linear = 2.0 * 2048 * layers * (4 * c * c + 2 * c * f)
    assert abs(flops - (linear + layers * 2.0 * c * 2048 * 2049 + 2.0 * c * v)) < 1.0
    assert 0.13e12 < flops < 0.14e12                                     # 0.137 TFLOP


def test_named_sizes_keep_the_default_and_name_every_size():
    bench = _bench()
    assert bench.MODEL is bench.SIZES["50m"]
    for name, sizes in bench.SIZES.items():
        assert sizes["n_embd"] % sizes["n_head"] == 0 and name in bench.MODEL_NAMES
        assert {"vocab_size", "n_positions", "n_layer", "n_head", "n_embd", "n_inner", "bias"} <= set(sizes)
