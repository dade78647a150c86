"""ctypes binding of libsfmonarch.so (the C ABI declared in include/sfmonarch.h).

The library is the only compute path: if it is missing it is built with nvcc, and if
that fails the import raises.  There is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libsfmonarch.so"

# name -> (restype, argtypes); must list every symbol of include/sfmonarch.h
SIGNATURES = {
    "sfm_version": (C.c_int, []),
    "sfm_error_string": (C.c_char_p, [C.c_int]),
    "sfm_build_maps": (C.c_int, [C.c_void_p, C.c_void_p] + [C.c_int] * 6),
    "sfm_rope_table": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_double]),
    "sfm_rope_cache_write": (C.c_int, [C.c_void_p] * 6 + [C.c_int64, C.c_void_p] + [C.c_int] * 12 + [C.c_void_p]),
    "sfm_rope_apply": (C.c_int, [C.c_void_p] * 3 + [C.c_int] * 8 + [C.c_void_p]),
    "sfm_monarch_workspace_bytes": (C.c_size_t, [C.c_int] * 11 + [C.c_size_t]),
    "sfm_monarch_fwd": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                  C.c_void_p, C.c_size_t] + [C.c_int] * 10 + [C.c_float, C.c_int, C.c_size_t,
                                                                             C.c_void_p]),
    "sfm_monarch_nocache_fwd": (C.c_int, [C.c_void_p] * 7 + [C.c_size_t] + [C.c_int] * 9 +
                                [C.c_float, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "sfm_dense_fwd": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p] +
                      [C.c_int] * 5 + [C.c_float, C.c_void_p]),
    "sfm_monarch_fwd_static": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p] +
                               [C.c_int] * 10 + [C.c_float, C.c_int, C.c_void_p]),
    "sfm_static_scratch_bytes": (C.c_size_t, []),
    "sfm_norm_rope_cache_write": (C.c_int, [C.c_void_p] * 5 + [C.c_float] + [C.c_void_p] * 3 + [C.c_int64, C.c_void_p] +
                                  [C.c_int] * 12 + [C.c_void_p]),
    "sfm_rope_cache_write_roll": (C.c_int, [C.c_void_p] * 5 + [C.c_float] + [C.c_void_p] * 3 + [C.c_int64, C.c_void_p] +
                                  [C.c_int] * 14 + [C.c_void_p]),
    "sfm_norm_rope_token_slice": (C.c_int, [C.c_void_p] * 5 + [C.c_float] + [C.c_void_p] * 4 + [C.c_int] * 8 + [C.c_void_p]),
    "sfm_rope_cache_write_gather": (C.c_int, [C.c_void_p] * 3 + [C.c_int, C.c_int] + [C.c_void_p] * 3 +
                                    [C.c_int64, C.c_void_p] + [C.c_int] * 12 + [C.c_void_p]),
    "sfm_monarch_fwd_scatter": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                          C.c_int, C.c_int, C.c_void_p, C.c_size_t] + [C.c_int] * 10 +
                                [C.c_float, C.c_size_t, C.c_void_p]),
    "sfm_monarch_bwd_workspace_bytes": (C.c_size_t, [C.c_int] * 10 + [C.c_size_t]),
    "sfm_monarch_bwd": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64] + [C.c_void_p] * 5 +
                        [C.c_size_t] + [C.c_int] * 10 + [C.c_float, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "sfm_workspace_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sfm_static_scratch_status": (C.c_int, [C.c_void_p]),
    "sfm_dense_status": (C.c_int, [C.c_void_p]),
    "sfm_launch_count": (C.c_longlong, []),
    "sfm_profile_enable": (C.c_int, [C.c_int]),
    "sfm_profile_read": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "sfm_probe_dsmem_store": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sfm_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        from . import build as _build
        _build.build()
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class SfmError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    """Raise for a non-zero return code: ValueError for argument errors, RuntimeError otherwise."""
    if rc == 0:
        return
    msg = load().sfm_error_string(rc).decode()
    if rc in (-1, -2, -3, -4, -5, -8):
        raise ValueError(f"{what}: {msg} (code {rc})")
    raise SfmError(f"{what}: {msg} (code {rc})")
