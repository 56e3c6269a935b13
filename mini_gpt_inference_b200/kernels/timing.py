"""Device time of every launch of the kernel library, by exported function.

The reference counts kernels and sums their device time from a profiler's trace
(bench/bench_kernels.py:71-116).  Here every kernel is launched through one of the library's
exported functions, so a pair of CUDA events around each call gives the same table without a
profiler::

    with LaunchTimer(ops) as timer:
        runner.step(entries)
    for row in timer.summary():
        print(row)

Only launches issued one by one are timed: while a step is being captured into a CUDA graph, and
when a captured step is replayed, no call passes through here (run the engine with
``use_cuda_graphs=False`` to see a step's kernels).  A launch timed alone neither overlaps its
neighbours nor starts while the kernel before it drains, so the times add up to more than the step
takes when it is replayed: compare shares.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .library import _P, _SIGNATURES


def launches(name: str) -> bool:
    """Whether the exported function ``name`` launches kernels (its last parameter is the stream)."""
    sig = _SIGNATURES.get(name)
    return sig is not None and len(sig) >= 3 and sig[-1] is _P


@dataclass
class LaunchRow:
    name: str            # exported function
    calls: int
    total_us: float
    mean_us: float
    share: float         # of the device time of all timed calls


class _TimedLibrary:
    def __init__(self, lib, records, device) -> None:
        self._lib, self._records, self._device = lib, records, device

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not launches(name):
            return fn
        records, device = self._records, self._device

        def timed(*args):
            if torch.cuda.is_current_stream_capturing():
                return fn(*args)
            stream = torch.cuda.current_stream(device)
            first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            first.record(stream)
            code = fn(*args)
            last.record(stream)
            records.append((name, first, last))
            return code

        return timed


class LaunchTimer:
    """While the block runs, ``ops.lib`` is a wrapper that brackets every launching call with events."""

    def __init__(self, ops) -> None:
        self.ops = ops
        self._records: list = []
        self._lib = None

    def __enter__(self) -> "LaunchTimer":
        self._lib = self.ops.lib
        self.ops.lib = _TimedLibrary(self._lib, self._records, self.ops.device)
        return self

    def __exit__(self, *exc) -> None:
        self.ops.lib = self._lib

    def summary(self) -> list[LaunchRow]:
        """One row per exported function, longest total first (waits for the device)."""
        torch.cuda.synchronize(self.ops.device)
        totals: dict[str, list] = {}
        for name, first, last in self._records:
            entry = totals.setdefault(name, [0, 0.0])
            entry[0] += 1
            entry[1] += first.elapsed_time(last) * 1e3
        whole = sum(v[1] for v in totals.values()) or 1.0
        rows = [LaunchRow(name, calls, total, total / calls, total / whole)
                for name, (calls, total) in totals.items()]
        return sorted(rows, key=lambda r: -r.total_us)

    def table(self) -> str:
        rows = self.summary()
        lines = [f"{'function':34s} {'calls':>6s} {'total us':>10s} {'mean us':>9s} {'share':>7s}"]
        for r in rows:
            lines.append(f"{r.name:34s} {r.calls:6d} {r.total_us:10.1f} {r.mean_us:9.2f} {r.share:7.1%}")
        lines.append(f"{'all':34s} {sum(r.calls for r in rows):6d} {sum(r.total_us for r in rows):10.1f}")
        return "\n".join(lines)
