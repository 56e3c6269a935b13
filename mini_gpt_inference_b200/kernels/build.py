"""Build the CUDA kernel library for sm_100a, in the tree, with nvcc alone.

Each ``csrc/*.cu`` is compiled to an object (in parallel) and linked into one shared
library under ``csrc/_build/``.  Nothing of torch is compiled in: the library exports
plain C functions that take device pointers, so a build takes seconds per file.  A
stamp of the sources' contents decides whether a rebuild is needed; a fresh checkout
builds at first use and prints a line per file while it does.  If the package folder
cannot be written, the build goes to a per-user temporary folder.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libminigpt_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# MINIGPT_B200_STAMPS=1 builds a tracing variant (in a folder of its own) whose kernels record
# time stamps at their phases (MG_STAMP in common.cuh); the ordinary build has none of it.
STAMPS = os.environ.get("MINIGPT_B200_STAMPS", "") not in ("", "0")
if STAMPS:
    NVCC_FLAGS = NVCC_FLAGS + ["-DMG_STAMPS"] + os.environ.get("MINIGPT_B200_STAMPS_FLAGS", "").split()
# MINIGPT_B200_GUARDS=1 builds a guarded variant (in a folder of its own) whose kernels check every
# index they read from device memory before they use it (MG_GUARDED in common.cuh).
GUARDS = os.environ.get("MINIGPT_B200_GUARDS", "") not in ("", "0")
if GUARDS:
    NVCC_FLAGS = NVCC_FLAGS + ["-DMG_GUARDS"]


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc not found: the CUDA kernel library cannot be built "
                     "(set NVCC or put nvcc on PATH)")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _build_dir() -> Path:
    d = CSRC / ("_build" + ("_stamps" if STAMPS else "") + ("_guards" if GUARDS else ""))
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"minigpt_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[mini_gpt_inference_b200] {msg}", file=sys.stderr, flush=True)


def library_path(verbose: bool = True, force: bool = False) -> Path:
    """Path of the built library, building it first if the sources changed."""
    bdir = _build_dir()
    lib = bdir / LIB_NAME
    stamp_file = bdir / "stamp.txt"
    stamp = _stamp()
    if not force and lib.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return lib
    nvcc = _nvcc()
    srcs = sources()
    _say(f"building {LIB_NAME} for sm_100a from {len(srcs)} files in {bdir}", verbose)
    t0 = time.time()

    def compile_one(src: Path) -> Path:
        obj = bdir / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        t = time.time()
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
        _say(f"  compiled {src.name} ({time.time() - t:.1f}s)", verbose)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = bdir / (LIB_NAME + f".tmp{os.getpid()}")
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    stamp_file.write_text(stamp)
    _say(f"built {lib} in {time.time() - t0:.1f}s", verbose)
    return lib


if __name__ == "__main__":
    print(library_path(force="--force" in sys.argv))
