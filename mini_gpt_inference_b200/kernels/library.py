"""Load the kernel library and declare its C functions.

The library is the only way the engine computes: if it cannot be built or loaded, or
if the device is not sm_100, importing the kernel set fails with a clear error.  There
is no fallback.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

from .build import library_path

_P = c_void_p
_I = c_int
_F = c_float

_SIGNATURES = {
    "mg_device_arch": [_I],
    "mg_set_device": [_I],
    "mg_set_dependent_launch": [_I],
    "mg_guards_enabled": [],
    "mg_embed": [_P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _P],
    "mg_layernorm": [_P, _P, _P, _P, _I, _I, _F, _I, _P],
    "mg_gather_rows": [_P, _P, _P, _I, _I, _I, _P],
    "mg_gather_tokens": [_P, _P, _P, _I, _I, _P],
    "mg_kv_store": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "mg_linear_simt": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "mg_linear_skinny": [_P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P,
                         _I, _I, _I, _I, _I, _P, _P, _I, _P],
    "mg_linear_skinny_ctas": [_I, _I],
    "mg_linear_stream": [_P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P,
                         _I, _I, _I, _I, _I, _P, _P, _I, _I, _P, _P],
    "mg_linear_stream_parts": [_I],
    "mg_linear_wide": [_P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P,
                       _I, _I, _I, _I, _I, _P, _P, _I, _P, _I, _P, _P],
    "mg_linear_wide_parts": [_I, _I, _I, _I],
    "mg_argmax_merge": [_P, _P, _P, _I, _I, _P],
    "mg_linear_cluster": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "mg_linear_tc": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "mg_paged_attention_generic": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "mg_paged_attention_split": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I,
                                 _F, _I, _I, _P, _P],
    "mg_attention_prefill_tc": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                ctypes.c_longlong, _I, _I, _F, _I, _P, _P],
    "mg_copy_ints": [_P, _P, _I, _P],
    "mg_argmax": [_P, _P, _I, _I, _I, _P],
    "mg_argmax_wide": [_P, _P, _P, _P, _I, _I, _I, _P],
    "mg_wait_probe": [_I, _P, _P],
    "mg_mlp_fused_max_width": [],
    "mg_mlp_fused": [_P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _P],
    "mg_zero_fill": [_P, ctypes.c_longlong, _P],
    "mg_sample": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
}


# exported readers of the kernel files' index guards: mg_<name>_index_fault(long long[4])
GUARDED_FILES = ("elementwise", "linear_skinny", "linear_stream", "linear_wide", "linear_cluster", "linear_tc",
                 "attention_generic", "attention_split", "attention_prefill")
for _name in GUARDED_FILES:
    _SIGNATURES[f"mg_{_name}_index_fault"] = [_P]
GUARD_CODES = {1: "token id", 2: "position", 3: "cache row", 4: "page", 5: "request", 6: "row", 7: "token source"}

UNSUPPORTED = -3     # a kernel refused the sizes; the caller may take another path


class KernelLibraryError(RuntimeError):
    pass


_lib = None


def load(verbose: bool = True):
    """The loaded library (built first if needed), with argument types declared."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path(verbose=verbose)
    try:
        lib = ctypes.CDLL(str(path))
    except OSError as exc:
        raise KernelLibraryError(f"cannot load the kernel library {path}: {exc}") from exc
    lib.mg_last_error.restype = ctypes.c_char_p
    lib.mg_last_error.argtypes = []
    for name, argtypes in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise KernelLibraryError(f"the kernel library lacks {name}; rebuild it") from None
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.mg_attention_prefill_scratch_floats.argtypes = [c_int, c_int]
    lib.mg_attention_prefill_scratch_floats.restype = ctypes.c_longlong
    lib.mg_argmax_parts.argtypes = [c_int]
    lib.mg_argmax_parts.restype = c_int
    lib.mg_attention_split_count.argtypes = [c_int, c_int, c_int]
    lib.mg_attention_split_count.restype = c_int
    lib.mg_attention_split_keys.argtypes = [c_int]
    lib.mg_attention_split_keys.restype = c_int
    lib.mg_attention_split_launches.argtypes = [c_int, c_int, c_int, c_int]
    lib.mg_attention_split_launches.restype = c_int
    lib.mg_mlp_pack_elements.argtypes = [c_int, c_int]
    lib.mg_mlp_pack_elements.restype = ctypes.c_longlong
    lib.mg_attention_split_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mg_attention_split_scratch_floats.restype = ctypes.c_longlong
    _lib = lib
    return lib


def declare(name: str, argtypes) -> None:
    """Declare a further function (used by kernels added after the table above)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().mg_last_error().decode(errors="replace")
        raise KernelLibraryError(f"{what} failed ({code}): {msg}")
