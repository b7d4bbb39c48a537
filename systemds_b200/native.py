"""ctypes binding of ``libsystemds_cla.so`` (the C ABI declared in ``include/systemds_cla.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsystemds_cla.so")

ERR_NAMES = {-1: "BAD_HANDLE", -2: "BAD_ARG", -3: "UNSUPPORTED", -4: "SHAPE", -5: "CUDA", -6: "STATE", -7: "NOMEM",
             -8: "DEVICE_CHECK"}


class CLAError(RuntimeError):
    """A C-ABI call returned a negative status (the Java side rethrows these as DMLCompressionException)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"CLA_ERR_{ERR_NAMES.get(code, code)}: {msg}")
        self.code = code


class cla_stats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("n_rows", "n_cols", "n_groups", "device_bytes", "index_bytes", "calls_rmm",
                                         "calls_lmm", "calls_tsmm", "calls_mmchain", "calls_decompress",
                                         "kernel_launches")] + [("last_kernel_ms", C.c_double),
                                                                 ("main_kernel_ms", C.c_double),
                                                                 ("main_kernel_count", C.c_int64)]


_P, _I32, _I64 = C.c_void_p, C.c_int32, C.c_int64
# name -> argument types; every function returns int64
SIGNATURES = {
    "cla_create": [_I32, _I32, _I32],
    "cla_destroy": [_I64],
    "cla_finalize": [_I64, _I32],
    "cla_last_error": [C.c_char_p, _I64],
    "cla_stats_get": [_I64, C.POINTER(cla_stats)],
    "cla_set_profile": [_I64, _I32],
    "cla_measure_fp64_peaks": [_I32, _P, _P],
    "cla_add_group_ddc": [_I64, _P, _I32, _P, _I32, _I32, _P, _P, _I64],
    "cla_add_group_sdc": [_I64, _P, _I32, _P, _I32, _P, _I32, _I32, _I32, _P, _I64, _I64, _I32, _P, _P],
    "cla_add_group_rle": [_I64, _P, _I32, _P, _I32, _P, _P, _I64],
    "cla_add_group_ole": [_I64, _P, _I32, _P, _I32, _P, _P, _I64],
    "cla_add_group_uncompressed": [_I64, _P, _I32, _P],
    "cla_add_group_ddc_dev": [_I64, _P, _I32, _P, _I32, _I32, _P, _I64],
    "cla_add_group_uncompressed_dev": [_I64, _P, _I32, _P],
    "cla_add_group_const": [_I64, _P, _I32, _P],
    "cla_add_group_empty": [_I64, _P, _I32],
    "cla_rmm": [_I64, _P, _I32, _I32, _P],
    "cla_rmm_overlapping": [_I64, _P, _I32, _I32],
    "cla_rmm_overlapping_dev": [_I64, _P, _I32, _I32, _P],
    "cla_lmm": [_I64, _P, _I32, _P],
    "cla_read_block": [_P, _I64, _P, _P],
    "cla_tsmm": [_I64, _P],
    "cla_tmm": [_I64, _I64, _P],
    "cla_mmchain": [_I64, _P, _P, _I32, _P],
    "cla_decompress": [_I64, _P],
    "cla_unary_agg": [_I64, _I32, _P],
    "cla_rmm_dev": [_I64, _P, _I32, _I32, _P, _P],
    "cla_lmm_dev": [_I64, _P, _I32, _P, _P],
    "cla_lmm_vec_noalloc_dev": [_I64, _P, _P, _P],
    "cla_tsmm_dev": [_I64, _P, _P],
    "cla_decompress_dev": [_I64, _P, _P],
    "cla_tmm_dev": [_I64, _I64, _P, _P],
    "cla_mmchain_dev": [_I64, _P, _P, _I32, _P, _P, _P],
    "cla_comm_create": [_I32, _I32, _I32, _I64, _P],
    "cla_comm_connect": [_I64, _P],
    "cla_comm_set_timeout_ms": [_I64, _I64],
    "cla_allreduce_dev": [_I64, _P, _I64, _P],
    "cla_comm_status": [_I64],
    "cla_comm_destroy": [_I64],
    "cla_group_decode": [_I64, _I32, _P],
    "cla_group_counts": [_I64, _I32, _P],
}

_lib = None


def lib() -> C.CDLL:
    """Load the shared library (once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m systemds_b200.build` (needs nvcc). "
                               "There is no CPU fallback for the compressed products.")
        l = C.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = _I64
        _lib = l
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(1024)
    lib().cla_last_error(buf, 1024)
    return buf.value.decode("utf-8", "replace")


def check(rc: int) -> int:
    if rc < 0:
        raise CLAError(int(rc), last_error())
    return int(rc)


def ptr(a) -> C.c_void_p:
    """Address of a numpy array (or None)."""
    if a is None:
        return C.c_void_p(0)
    return C.c_void_p(a.ctypes.data)
