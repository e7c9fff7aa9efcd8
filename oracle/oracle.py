"""ctypes front end of the CPU oracle (``huff_oracle.c``).

TEST INFRASTRUCTURE ONLY: the parity tests, the smoke entry and the CPU-baseline leg of the
benchmark import this module; nothing in the product package does.

All functions take and return numpy arrays.  Encoders return a dict keyed exactly like the dicts of
the reference's Python bindings (kernel/wrapper.cpp:182-209, 258-321, 419-454); dtypes are the
unsigned ones the reference returns (uint16 / uint32 / uint64 where it says ``_u16/_u32/_u64``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "liborc.so"

_DTYPES = [np.uint8, np.uint16, np.int16, np.int32, np.uint32, np.int64, np.uint64]


class _Tensor(C.Structure):
    _fields_ = [
        ("name", C.c_char * 48),
        ("dtype", C.c_int),
        ("ndim", C.c_int),
        ("shape", C.c_int64 * 2),
        ("data", C.c_void_p),
    ]


class _Result(C.Structure):
    _fields_ = [
        ("ntensors", C.c_int),
        ("err_kind", C.c_int),
        ("err", C.c_char * 256),
        ("t", _Tensor * 24),
    ]


def build_library(force: bool = False) -> Path:
    """Compile ``huff_oracle.c`` into ``_build/liborc.so`` (gcc, a second or two)."""
    src = _HERE / "huff_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "_build/liborc.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build_library()
        _lib = C.CDLL(str(_LIB_PATH))
        for fn in ("orc_build_fp8", "orc_build_awq_bucket", "orc_build_awq_by_scale", "orc_build_awq_shared"):
            getattr(_lib, fn).restype = C.POINTER(_Result)
        _lib.orc_free.argtypes = [C.POINTER(_Result)]
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Threads of the decode loops from now on, whatever OMP_NUM_THREADS said when the OpenMP runtime
    started (torchrun exports OMP_NUM_THREADS=1 to its ranks)."""
    lib().orc_set_num_threads(C.c_int(int(n)))


def set_substream_limit(n: int = 1024) -> None:
    """Most sub-streams per bucket ``build_fp8`` accepts from now on (1024, the reference's limit, unless a
    test of the library's finer sub-streams raises it)."""
    lib().orc_set_substream_limit(C.c_int64(int(n)))


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype != dtype:
        if a.dtype.itemsize == np.dtype(dtype).itemsize:
            a = a.view(dtype)
        else:
            raise TypeError(f"expected {np.dtype(dtype)}, got {a.dtype}")
    return a


def _take(res_p) -> dict:
    res = res_p.contents
    try:
        if res.err_kind == 1:
            raise ValueError(res.err.decode())
        if res.err_kind == 2:
            raise RuntimeError(res.err.decode())
        out = {}
        for i in range(res.ntensors):
            t = res.t[i]
            dt = np.dtype(_DTYPES[t.dtype])
            shape = tuple(int(t.shape[j]) for j in range(t.ndim))
            numel = int(np.prod(shape)) if shape else 1
            if numel > 0:
                buf = (C.c_char * (numel * dt.itemsize)).from_address(t.data)
                arr = np.frombuffer(buf, dtype=dt).reshape(shape).copy()
            else:
                arr = np.zeros(shape, dtype=dt)
            out[t.name.decode()] = arr
        return out
    finally:
        lib().orc_free(res_p)


def _scale_args(scales: np.ndarray):
    s = _c(scales, np.uint16)
    nd = s.ndim
    if nd > 2:
        raise ValueError("scales must have at most 2 dims")
    d0 = s.shape[0] if nd >= 1 else 1
    d1 = s.shape[1] if nd >= 2 else 1
    return s, C.c_int(nd), C.c_int64(d0), C.c_int64(d1)


def build_fp8(bf16_bits, fp8_u8, scales_u16, max_len=12, threads_per_block=256) -> dict:
    """huffman_build_fp8_decode_tables (kernel/wrapper.cpp:419-454, build_huffman.cu:292-969)."""
    b = _c(bf16_bits, np.uint16)
    if b.ndim != 2:
        raise ValueError("bucket packing requires bf16_params to be 2D [n,m]")
    f = _c(fp8_u8, np.uint8)
    if f.size != b.size:
        raise ValueError("bf16_params and fp8_params must have same numel")
    s, nd, d0, d1 = _scale_args(scales_u16)
    n, m = b.shape
    return _take(lib().orc_build_fp8(_ptr(b), _ptr(f), _ptr(s), nd, d0, d1, C.c_int64(n), C.c_int64(m),
                                     C.c_int64(int(max_len)), C.c_int64(int(threads_per_block))))


def build_awq_bucket(bf16_bits, int4_u8, scales_u16, max_len=11, threads_per_block=256) -> dict:
    """huffman_build_awq_int4_bucket_decode_tables (wrapper.cpp:258-288, build_huffman.cu:1582-2126)."""
    b = _c(bf16_bits, np.uint16)
    q = _c(int4_u8, np.uint8)
    if b.ndim != 2:
        raise ValueError("bf16_params must be 2D [n,m]")
    if q.shape != b.shape:
        raise ValueError("int4_values_u8 shape must match bf16_params")
    s, nd, d0, d1 = _scale_args(scales_u16)
    n, m = b.shape
    return _take(lib().orc_build_awq_bucket(_ptr(b), _ptr(q), _ptr(s), nd, d0, d1, C.c_int64(n), C.c_int64(m),
                                            C.c_int64(int(max_len)), C.c_int64(int(threads_per_block))))


def build_awq_by_scale(bf16_bits, int4_u8, scales_u16, max_len=11, threads=256, group_cap=1024) -> dict:
    """huffman_build_awq_int4_bucket_decode_tables_by_scale (wrapper.cpp:290-321, build_huffman.cu:1074-1580)."""
    b = _c(bf16_bits, np.uint16)
    q = _c(int4_u8, np.uint8)
    if b.ndim != 2:
        raise ValueError("bf16_params must be 2D [n,m]")
    if q.shape != b.shape:
        raise ValueError("int4_values_u8 shape must match bf16_params")
    s, nd, d0, d1 = _scale_args(scales_u16)
    n, m = b.shape
    return _take(lib().orc_build_awq_by_scale(_ptr(b), _ptr(q), _ptr(s), nd, d0, d1, C.c_int64(n), C.c_int64(m),
                                              C.c_int64(int(max_len)), C.c_int64(int(threads)),
                                              C.c_int64(int(group_cap))))


def build_awq_shared(bf16_bits, int4_u8, scales_u16, max_len=11) -> dict:
    """huffman_build_awq_decode_tables (wrapper.cpp:182-209, build_huffman.cu:2157-2633)."""
    b = _c(bf16_bits, np.uint16)
    q = _c(int4_u8, np.uint8)
    if b.ndim != 2:
        raise ValueError("bf16_params must be 2D [n,m]")
    if q.shape != b.shape:
        raise ValueError("int4_values_u8 shape must match bf16_params")
    s, nd, d0, d1 = _scale_args(scales_u16)
    n, m = b.shape
    return _take(lib().orc_build_awq_shared(_ptr(b), _ptr(q), _ptr(s), nd, d0, d1, C.c_int64(n), C.c_int64(m),
                                            C.c_int64(int(max_len))))


def package_merge(weights, max_len: int) -> np.ndarray:
    """Code lengths of the ascending-sorted weights (build_huffman.cu:46-118)."""
    w = np.ascontiguousarray(np.asarray(weights, dtype=np.int64))
    lens = np.zeros(len(w), dtype=np.int32)
    rc = lib().orc_package_merge(_ptr(w), C.c_int(len(w)), C.c_int(int(max_len)), _ptr(lens))
    if rc == 1:
        raise ValueError("package-merge: invalid argument")
    if rc == 2:
        raise RuntimeError("package-merge: not enough packages")
    return lens


def decode_fp8(fp8_u8, art: dict, n: int, m: int, out=None) -> np.ndarray:
    """CPU decode of the FP8 bucket format; returns BF16 bit patterns ``uint16[n,m]``."""
    f = _c(fp8_u8, np.uint8)
    bs = _c(art["bitstream_u64"], np.uint64)
    syms = _c(art["decode_syms_u16"], np.uint16)
    lens = _c(art["decode_lens_u8"], np.uint8)
    bt = _c(art["bucket_table_i32"], np.int32)
    cs = _c(art["bucket_col_start_i32"], np.int32)
    cl = _c(art["bucket_col_len_i32"], np.int32)
    ro = _c(art["bucket_row_offsets_i32"], np.int32)
    ri = _c(art["row_indices_i32"], np.int32)
    tsb = _c(art["bucket_thread_startbit_u32"], np.uint32)
    bb = _c(art["bucket_bit_base_i64"], np.int64)
    B, k = bt.shape[0], tsb.shape[1] - 1
    if out is None:
        out = np.zeros((n, m), dtype=np.uint16)
    lib().orc_decode_fp8(_ptr(f), _ptr(bs), C.c_int64(bs.size), _ptr(syms), _ptr(lens), _ptr(bt), _ptr(cs), _ptr(cl),
                         _ptr(ro), _ptr(ri), _ptr(tsb), _ptr(bb), C.c_int64(B), C.c_int64(k), C.c_int64(n),
                         C.c_int64(m), _ptr(out))
    return out


def decode_awq_bucket(int4_u8, art: dict, n: int, m: int) -> np.ndarray:
    q = _c(int4_u8, np.uint8)
    bs = _c(art["bitstream_u64"], np.uint64)
    syms = _c(art["decode_syms_u16"], np.uint16)
    lens = _c(art["decode_lens_u8"], np.uint8)
    bt = _c(art["bucket_table_i32"], np.int32)
    cs = _c(art["bucket_col_start_i32"], np.int32)
    cl = _c(art["bucket_col_len_i32"], np.int32)
    ro = _c(art["bucket_row_offsets_i32"], np.int32)
    ri = _c(art["row_indices_i32"], np.int32)
    tsb = _c(art["bucket_thread_startbit_u32"], np.uint32)
    bb = _c(art["bucket_bit_base_i64"], np.int64)
    B, k = bt.shape[0], tsb.shape[1] - 1
    out = np.zeros((n, m), dtype=np.uint16)
    lib().orc_decode_awq_bucket(_ptr(q), _ptr(bs), C.c_int64(bs.size), _ptr(syms), _ptr(lens), _ptr(bt), _ptr(cs),
                                _ptr(cl), _ptr(ro), _ptr(ri), _ptr(tsb), _ptr(bb), C.c_int64(B), C.c_int64(k),
                                C.c_int64(n), C.c_int64(m), _ptr(out))
    return out


def decode_awq_by_scale(int4_u8, art: dict, n: int, m: int, group_size: int) -> np.ndarray:
    q = _c(int4_u8, np.uint8)
    bs = _c(art["bitstream_u64"], np.uint64)
    syms = _c(art["decode_syms_u16"], np.uint16)
    lens = _c(art["decode_lens_u8"], np.uint8)
    bt = _c(art["bucket_table_i32"], np.int32)
    go = _c(art["bucket_group_offsets_i32"], np.int32)
    gr = _c(art["group_rows_i32"], np.int32)
    gc = _c(art["group_col_start_i32"], np.int32)
    tsb = _c(art["bucket_thread_startbit_u32"], np.uint32)
    bb = _c(art["bucket_bit_base_i64"], np.int64)
    B, k = bt.shape[0], tsb.shape[1] - 1
    out = np.zeros((n, m), dtype=np.uint16)
    lib().orc_decode_awq_by_scale(_ptr(q), _ptr(bs), C.c_int64(bs.size), _ptr(syms), _ptr(lens), _ptr(bt), _ptr(go),
                                  _ptr(gr), _ptr(gc), _ptr(tsb), _ptr(bb), C.c_int64(B), C.c_int64(k), C.c_int64(n),
                                  C.c_int64(m), C.c_int64(int(group_size)), _ptr(out))
    return out


def decode_awq_shared(art: dict, out_len: int, max_len: int = 11) -> np.ndarray:
    bs = _c(art["bitstream_u64"], np.uint64)
    syms = _c(art["decode_syms_i16"], np.int16)
    nb = _c(art["decode_nbits_u8"], np.uint8)
    sbb = _c(art["scale_bit_base_i64"], np.int64)
    cst = _c(art["chunk_startbit_rel_u32"], np.uint32)
    cob = _c(art["chunk_out_base_u32"], np.uint32)
    cm = _c(art["chunk_meta_u32"], np.uint32)
    csi = _c(art["chunk_scale_id_i32"], np.int32)
    oi = _c(art["out_idx_i32"], np.int32)
    so = _c(art["stream_chunk_ofs_i64"], np.int64)
    si = _c(art["stream_chunk_ids_i32"], np.int32)
    out = np.zeros(out_len, dtype=np.int16)
    lib().orc_decode_awq_shared(_ptr(bs), C.c_int64(bs.size), _ptr(syms), _ptr(nb), C.c_int64(syms.shape[1]),
                                _ptr(sbb), _ptr(cst), _ptr(cob), _ptr(cm), _ptr(csi), _ptr(oi), _ptr(so), _ptr(si),
                                C.c_int64(syms.shape[0]), C.c_int64(int(out_len)), C.c_int(int(max_len)), _ptr(out))
    return out
