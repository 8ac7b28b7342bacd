"""ctypes binding of libpq_b200.so (the C ABI declared in include/pq_b200.h).

The library is the only implementation of the hot path: when it is missing, loading fails with a
RuntimeError that says how to build it -- there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent / "libpq_b200.so"

PQ_OK = 0
PQ_ERR_TIMEOUT = 6
DTYPE_BF16 = 0
DTYPE_FP16 = 1
GEMM_WORKSPACE_BYTES = 256

_lib: Optional[ctypes.CDLL] = None

# name -> (restype, argtypes); mirrors include/pq_b200.h
SIGNATURES = {
    "pq_version": (c_int, []),
    "pq_status_str": (c_char_p, [c_int]),
    "pq_last_cuda_error": (c_int, []),
    "pq_set_option": (c_int, [c_char_p, c_int]),
    "pq_get_option": (c_int, [c_char_p, POINTER(c_int)]),
    "pq_quant_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "pq_quant_rows_cat": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int64, c_void_p, c_void_p,
                                  c_void_p]),
    "pq_lowrank_down_cat": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_void_p, c_int64, c_int,
                                    c_void_p, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "pq_adaln_quant_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                    ctypes.c_float, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "pq_gather_quant_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p,
                                     c_void_p, c_void_p]),
    "pq_gather_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                               c_void_p]),
    "pq_quant_rows_g32": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "pq_dequant_epilogue": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                                    c_void_p]),
    "pq_int8_gemm": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                             c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int,
                             c_void_p, c_int, c_int64, c_int64, c_int64, c_int64,
                             c_void_p, c_size_t, c_void_p, c_void_p]),
    "pq_int8_gemm_ex": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int,
                                c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int,
                                c_void_p, c_size_t, c_void_p]),
    "pq_int8_gemm_gated": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                   c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int,
                                   c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int,
                                   c_void_p, c_size_t, c_void_p]),
    "pq_int8_gemm_bcast": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                   c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int,
                                   c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int,
                                   c_void_p, c_size_t, c_void_p]),
    "pq_int8_gemm_grouped": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                     c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int,
                                     c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                                     c_void_p, c_size_t, c_void_p]),
    "pq_lowrank_down": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int64, c_int64,
                                c_void_p, c_size_t, c_void_p]),
    "pq_unpack_int4": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "pq_int8_gemm_g32": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "pq_scatter_rows": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "pq_noalloc_scratch_bytes": (c_size_t, []),
    "pq_int8_linear_noalloc": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                       c_int64, c_int64, c_int64, c_int64, POINTER(c_void_p), c_void_p]),
    "pq_read_status_word": (c_int, [c_void_p, POINTER(c_int32), c_int, c_void_p]),
    "pq_wait_probe": (c_int, [c_void_p, c_size_t, c_int, c_void_p]),
    "pq_i8_mma_issue_loop": (c_int, [c_int, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
}


def load() -> ctypes.CDLL:
    """Loads the shared library once and attaches the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the sm_100a CUDA library has not been built. "
            "Run `python -m pyraquant_b200.build` (needs nvcc). There is no fallback path.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError here = header and library out of step
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_str(rc: int) -> str:
    return load().pq_status_str(int(rc)).decode()


def check(rc: int, what: str) -> None:
    if rc != PQ_OK:
        lib = load()
        extra = f" (cudaError {lib.pq_last_cuda_error()})" if rc == 5 else ""
        raise RuntimeError(f"{what}: {status_str(rc)}{extra}")


def set_option(key: str, value: int) -> None:
    check(load().pq_set_option(key.encode(), int(value)), f"pq_set_option({key})")


def get_option(key: str) -> int:
    v = c_int(0)
    check(load().pq_get_option(key.encode(), ctypes.byref(v)), f"pq_get_option({key})")
    return int(v.value)
