"""The guarded build of the kernel library (MINIGPT_B200_GUARDS=1): its kernels check every index
they read from device memory, record the first one outside its table and skip the access, and the
engine's status check raises.  The build variant is fixed when the kernel package is imported, so
the checks run in a process of their own (tests/guarded_build_checks.py)."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from mini_gpt_inference_b200.kernels import library

ROOT = Path(__file__).resolve().parent.parent


def test_every_guarded_file_has_a_reader():
    for name in library.GUARDED_FILES:
        assert f"mg_{name}_index_fault" in library._SIGNATURES
    assert set(library.GUARD_CODES) == set(range(1, 8))


@pytest.mark.gpu
def test_guarded_build_catches_indices_outside_their_tables():
    env = dict(os.environ, MINIGPT_B200_GUARDS="1")
    proc = subprocess.run([sys.executable, str(ROOT / "tests" / "guarded_build_checks.py")], env=env,
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    seen = json.loads(proc.stdout.strip().splitlines()[-1])
    assert seen["guards"] is True
    # the engine's own steps: right logits, quiet guards, before and after the faults below
    for tag in ("before", "after"):
        for key in (f"{tag}_A_bfloat16", f"{tag}_B_float32", f"{tag}_H_bfloat16"):
            assert seen[key]["diff"] <= seen[key]["tolerance"], (key, seen[key])
    # each bad index is named with its value and its limit; the access was skipped or replaced
    assert "token id 77 is outside 0..49" in seen["token"] and seen["token_row_replaced"]
    assert "position 33 is outside 0..19" in seen["position"]
    assert "token source 11 is outside 0..3" in seen["source"] and seen["source_row_kept"]
    assert "row 9 is outside 0..5" in seen["row"]
    for name in ("kv_store_float32", "kv_store_bfloat16", "sink_skinny", "sink_cluster", "sink_tensor_cores",
                 "sink_stream", "sink_wide"):
        assert "cache row" in seen[name] and "is outside 0..31" in seen[name], (name, seen[name])
        assert seen[name + "_behind_untouched"], name
        assert seen[name + "_good_row_written"], name
    for name in ("skinny", "cluster", "tensor_cores", "stream", "wide"):
        assert seen[f"sink_{name}_one_launch"], name
    assert seen["sink_skinny"].startswith("a kernel met an index outside its table: linear_skinny")
    assert "linear_cluster" in seen["sink_cluster"] and "linear_tc" in seen["sink_tensor_cores"]
    for name in ("split", "generic"):
        assert seen[f"attention_{name}_quiet"] == ""
        assert "page 6 is outside 0..3" in seen[f"attention_{name}_page"], seen[f"attention_{name}_page"]
        assert "request 5 is outside 0..1" in seen[f"attention_{name}_request"]
        assert "position 35 is outside 0..31" in seen[f"attention_{name}_position"]
        assert f"attention_{name}" in seen[f"attention_{name}_page"]
