"""ctypes binding of ``libtessel_b200.so`` (the C ABI of ``include/tessel_b200.h``).

There is no fallback: if the library is missing, importing the symbols raises
with the build command, and every compute call needs a B200.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TESSEL_B200_LIB selects another build of the same ABI (the trace build of tessel_b200/build.py).
SO = os.environ.get("TESSEL_B200_LIB") or os.path.join(HERE, "libtessel_b200.so")

# Every symbol include/tessel_b200.h declares: (name, restype, argtypes).
_u64p = C.POINTER(C.c_uint64)
SYMBOLS = [
    ("tb200_init", C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    ("tb200_destroy", None, [C.c_void_p]),
    ("tb200_last_error", C.c_char_p, [C.c_void_p]),
    ("tb200_alloc", C.c_int, [C.c_void_p, C.c_size_t, _u64p]),
    ("tb200_free", C.c_int, [C.c_void_p, C.c_uint64]),
    ("tb200_write", C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_void_p, C.c_size_t]),
    ("tb200_write_async", C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_void_p, C.c_size_t]),
    ("tb200_read", C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_void_p, C.c_size_t]),
    ("tb200_host_alloc", C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    ("tb200_host_free", C.c_int, [C.c_void_p, C.c_void_p]),
    ("tb200_kernel", C.c_int,
     [C.c_void_p, C.c_char_p, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.c_int, C.POINTER(C.c_int32)]),
    ("tb200_launch", C.c_int, [C.c_void_p, C.c_int32, _u64p, C.c_int]),
    ("tb200_tune", C.c_int, [C.c_void_p, C.c_int32, _u64p, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
    ("tb200_capture_begin", C.c_int, [C.c_void_p]),
    ("tb200_capture_end", C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
    ("tb200_replay", C.c_int, [C.c_void_p, C.c_int32]),
    ("tb200_sync", C.c_int, [C.c_void_p]),
    ("tb200_time_begin", C.c_int, [C.c_void_p]),
    ("tb200_time_end", C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    ("tb200_profile", C.c_int, [C.c_void_p, C.c_int]),
    ("tb200_phase", C.c_int, [C.c_void_p, C.c_char_p]),
    ("tb200_profile_rows", C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    ("tb200_profile_row", C.c_int,
     [C.c_void_p, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), _u64p, C.POINTER(C.c_double)]),
    ("tb200_launch_count", C.c_int, [C.c_void_p, _u64p]),
    ("tb200_set_stream", C.c_int, [C.c_void_p, C.c_void_p]),
    ("tb200_get_stream", C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    ("tb200_comm_id", C.c_int, [C.c_void_p, C.c_void_p]),
    ("tb200_comm_init", C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    ("tb200_allreduce", C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_int]),
    ("tb200_ipc_export", C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    ("tb200_ipc_import", C.c_int, [C.c_void_p, C.c_void_p, _u64p]),
    ("tb200_tp_sizes", C.c_int, [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    ("tb200_tp_table", C.c_int,
     [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, _u64p, _u64p, _u64p, C.c_uint64, C.c_uint64, C.c_uint64]),
    ("tb200_memset", C.c_int, [C.c_void_p, C.c_uint64, C.c_int, C.c_size_t]),
    ("tb200_decode_attention_static", C.c_int,
     [C.c_void_p, C.POINTER(C.c_int32), C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
      C.c_float]),
    ("tb200_rng_seed", C.c_uint64, [C.c_uint64]),
    ("tb200_rng_uniform", None, [_u64p, C.c_void_p, C.c_size_t]),
]

COMM_ID_BYTES = 128

_lib = None


def lib() -> C.CDLL:
    """The loaded library. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO):
            raise RuntimeError(
                f"{SO} is missing: build it with `python -m tessel_b200.build` "
                "(nvcc, sm_100a). There is no CPU path.")
        l = C.CDLL(SO)
        for name, res, args in SYMBOLS:
            f = getattr(l, name)
            f.restype = res
            f.argtypes = args
        _lib = l
    return _lib
