"""ctypes binding of libmpserve_b200.so (the C ABI declared in include/mpserve_b200.h)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libmpserve_b200.so"

MPS_OK = 0
MPS_ERR_INVALID = -1
MPS_ERR_UNSUPPORTED = -2
MPS_ERR_WORKSPACE = -3

_p = C.c_void_p
_i64 = C.c_int64
_i32 = C.c_int32


class BucketTensor(C.Structure):
    """struct mps_bucket_tensor"""

    _fields_ = [
        ("ctx_bytes", _p), ("bitstream", _p), ("bitstream_words", _i64),
        ("decode_syms", _p), ("decode_lens", _p), ("num_tables", _i64),
        ("bucket_table", _p), ("bucket_col_start", _p), ("bucket_col_len", _p),
        ("bucket_row_offsets", _p), ("row_indices", _p), ("group_col_start", _p), ("num_rows", _i64),
        ("thread_startbit", _p), ("bucket_bit_base", _p), ("num_buckets", _i64),
        ("k", _i32), ("group_size", _i32), ("mode", _i32), ("reserved", _i32),
        ("n", _i64), ("m", _i64), ("out", _p),
    ]


_PROTOS = {
    "mps_abi_version": (C.c_int, []),
    "mps_last_error": (C.c_char_p, []),
    "mps_cuda_clock_rate_khz": (_i64, []),
    "mps_workspace_bytes": (C.c_size_t, []),
    "mps_decode_fp8": (C.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _p, _p, _p, _i64, _p, _p, _i64, _i32, _i64, _i64,
                                 _i64, _p, _p, C.c_size_t, _p]),
    "mps_decode_fp8_noalloc": (C.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _p, _p, _p, _i64, _p, _p, _i64, _i32, _i64, _i64,
                                         _i64, _p, _p]),
    "mps_decode_awq_int4_bucket": (C.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _p, _p, _p, _i64, _p, _p, _i64, _i32,
                                             _i64, _i64, _i64, _p, _p, C.c_size_t, _p]),
    "mps_decode_awq_int4_bucket_by_scale": (C.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _p, _p, _i64, _p, _p, _i64,
                                                      _i32, _i64, _i64, _i64, _i64, _p, _p, C.c_size_t, _p]),
    "mps_decode_awq_shared_table": (C.c_int, [_p, _i64, _p, _p, _i64, _p, _i64, _p, _p, _p, _p, _i64, _p, _p, _p, _i64,
                                              _i64, _p, _p]),
    "mps_bucket_batch_plan": (C.c_int, [C.POINTER(BucketTensor), C.c_int, C.POINTER(_i64), C.POINTER(_i32),
                                        C.POINTER(_i32)]),
    "mps_decode_bucket_batch": (C.c_int, [_p, _p, C.c_int, _i64, _i32, _i32, _i32, _p, C.c_size_t, _p]),
    "mps_decode_bucket_tensor": (C.c_int, [C.POINTER(BucketTensor), _p, C.c_size_t, _p]),
    "mps_decode_status": (C.c_int, [_p, C.c_size_t, _p, C.POINTER(_i32)]),
    "mps_selftest_stalled_decode": (C.c_int, [C.POINTER(BucketTensor), _i32, C.c_uint32, _p, C.c_size_t, _p]),
    "mps_checksum_u16": (C.c_int, [_p, _i64, _p, _p]),
    "mps_build_workspace_bytes": (C.c_size_t, [_i64, _i64]),
    "mps_build_analyze": (C.c_int, [_p, _p, _p, _p, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _i64, _p, C.c_size_t, _p,
                                    C.POINTER(_i64), C.POINTER(_i64)]),
    "mps_build_codebooks": (C.c_int, [_p, _p, _p, _p, _p, _p]),
    "mps_build_bucket_table": (C.c_int, [_p, _p, _i64, _p, _p]),
    "mps_build_bucket_unique": (C.c_int, [_p, _i64, _p, _p, _p, _p]),
    "mps_build_rect_layout": (C.c_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i32, _p, _p, _p, C.POINTER(_i64)]),
    "mps_build_rect_emit": (C.c_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i32, _p, _p, _p, _i64, _p]),
    "mps_build_shared_codebooks": (C.c_int, [_p, _p, _i64, _p, _p, _p]),
    "mps_build_shared_layout": (C.c_int, [_p, _p, _p, _p, _i32, _i64, _i64, _i64, _p, _p, _p, C.POINTER(_i64),
                                          C.POINTER(_i64)]),
    "mps_build_shared_emit": (C.c_int, [_p, _p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library; raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mpserve_b200.build` "
                "(there is no CPU or PyTorch fallback for the decode path)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _PROTOS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def exported_names() -> list[str]:
    return sorted(_PROTOS)


def check(rc: int) -> None:
    """Map a C-ABI return code to the exception class the reference binding would raise."""
    if rc == MPS_OK:
        return
    msg = load().mps_last_error().decode(errors="replace")
    if rc == MPS_ERR_INVALID:
        raise ValueError(msg)
    if rc == MPS_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"{msg} (code {rc})")
