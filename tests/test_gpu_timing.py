"""The per-launch timer of the kernel library: it times every launch of a step that is issued
launch by launch, leaves the results alone and puts the library back."""

from __future__ import annotations

import pytest
import torch

from harness import PAGE_TOKENS, gpu_runner, make_tensors, tiny_config, tokens_for
from mini_gpt_inference_b200.engine.runner import StepEntry
from mini_gpt_inference_b200.kernels.timing import LaunchTimer, launches


def test_which_functions_launch():
    assert launches("mg_embed") and launches("mg_linear_wide") and launches("mg_zero_fill")
    assert not launches("mg_linear_wide_parts") and not launches("mg_mlp_fused_max_width")
    assert not launches("mg_set_device") and not launches("no_such_function")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_timed_launch_by_launch(dtype):
    cfg = tiny_config("A")
    tensors = make_tensors(cfg, 5, dtype, False)
    runner = gpu_runner(cfg, tensors, dtype, PAGE_TOKENS["A"], 64)
    runner.use_cuda_graphs = False
    ops = runner.ops
    tokens = tokens_for(cfg, 29, 11)
    plain = runner.step([StepEntry("a", tokens, [28])]).clone()
    runner.finish("a")
    library, before = ops.lib, ops.launches
    with LaunchTimer(ops) as timer:
        assert ops.lib is not library
        timed = runner.step([StepEntry("a", tokens, [28])]).clone()
    assert ops.lib is library
    assert torch.equal(timed, plain)                      # the same kernels ran on the same inputs
    rows = timer.summary()
    names = {r.name for r in rows}
    assert "mg_embed" in names and any(n.startswith("mg_paged_attention") or n.startswith("mg_attention") for n in names)
    assert any(n.startswith("mg_linear") or n == "mg_mlp_fused" for n in names)
    calls = sum(r.calls for r in rows)
    assert 0 < calls <= ops.launches - before             # (a call may launch two kernels)
    assert all(r.total_us > 0 and r.mean_us > 0 for r in rows)
    assert abs(sum(r.share for r in rows) - 1.0) < 1e-6
    assert rows == sorted(rows, key=lambda r: -r.total_us)
    assert "function" in timer.table() and "all" in timer.table()
    # one decode step of the same request, timed as well: it goes through the same wrapper
    with LaunchTimer(ops) as timer:
        runner.step([StepEntry("a", [3], [0])])
    assert sum(r.calls for r in timer.summary()) > 0
    runner.finish("a")
