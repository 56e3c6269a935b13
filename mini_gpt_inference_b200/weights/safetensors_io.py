"""Minimal reader and writer for the safetensors container.

The format: 8 bytes little-endian header length, a JSON header mapping each tensor name
to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of
the header), then the raw little-endian data.  The reference loads a pickled training
checkpoint instead (src/minigpt_infer/loader.py:63-85); this engine reads tensors by
name from ``model.safetensors`` and never unpickles anything.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Mapping

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path: str | Path) -> tuple[dict, int]:
    """Return (header dict without ``__metadata__``, byte offset where data begins)."""
    path = Path(path)
    with open(path, "rb") as f:
        first = f.read(8)
        if len(first) != 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", first)
        size = path.stat().st_size
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not JSON: {exc}") from exc
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    header.pop("__metadata__", None)
    spans = []
    for name, info in header.items():
        if not isinstance(info, dict):
            raise SafetensorsError(f"{path}: entry {name!r} of the header is not an object")
        dtype, shape, offsets = info.get("dtype"), info.get("shape"), info.get("data_offsets")
        if not isinstance(dtype, str) or dtype not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")

        def is_int(v):
            return isinstance(v, int) and not isinstance(v, bool)

        if not isinstance(shape, list) or not all(is_int(d) and d >= 0 for d in shape):
            raise SafetensorsError(f"{path}: tensor {name!r} has a malformed shape {shape!r}")
        if (not isinstance(offsets, list) or len(offsets) != 2 or not all(is_int(v) for v in offsets)
                or not 0 <= offsets[0] <= offsets[1]):
            raise SafetensorsError(f"{path}: tensor {name!r} has malformed data_offsets {offsets!r}")
        begin, end = offsets
        count = 1
        for d in shape:
            count *= d
        width = torch.empty((), dtype=_DTYPES[dtype]).element_size()
        if end - begin != count * width or 8 + n + end > size:
            raise SafetensorsError(f"{path}: tensor {name!r} has inconsistent offsets")
        if end > begin:
            spans.append((begin, end, name))
    spans.sort()
    for (_, end_a, a), (begin_b, _, b) in zip(spans, spans[1:]):
        if begin_b < end_a:
            raise SafetensorsError(f"{path}: tensors {a!r} and {b!r} overlap in the file")
    return header, 8 + n


def load_file(path: str | Path) -> dict[str, torch.Tensor]:
    """All tensors of a file, as CPU tensors that own their memory."""
    path = Path(path)
    header, base = read_header(path)
    out: dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        with mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as mm:
            for name, info in header.items():
                begin, end = info["data_offsets"]
                dtype = _DTYPES[info["dtype"]]
                if end == begin:
                    out[name] = torch.empty(info["shape"], dtype=dtype)
                    continue
                raw = bytearray(mm[base + begin: base + end])
                out[name] = torch.frombuffer(raw, dtype=dtype).reshape(info["shape"])
    return out


def save_file(tensors: Mapping[str, torch.Tensor], path: str | Path,
              metadata: Mapping[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        data = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(data)]}
        offset += len(data)
        blobs.append(data)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * ((8 - len(head) % 8) % 8)
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for data in blobs:
            f.write(data)
