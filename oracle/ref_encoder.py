"""Loader for the reference's own CPU encoder compiled by ``oracle/build_ref.sh``.

TEST INFRASTRUCTURE ONLY.  Used to pin ``huff_oracle.c`` byte-for-byte, to generate the golden
fixtures, and as the timed "reference" CPU encode baseline.  ``available()`` is False on machines
where ``oracle/_ref`` was never built.

The dict keys follow the reference's Python bindings (kernel/wrapper.cpp:190-203, 268-281,
301-313, 429-446); values are the torch CPU tensors the reference returns.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

_REF_DIR = Path(__file__).resolve().parent / "_ref"

FP8_KEYS = [
    "decode_syms_u16", "decode_lens_u8", "table_scale_u16", "table_fp8_u16", "bucket_scale_u16",
    "bucket_row_offsets_i32", "row_indices_i32", "bucket_table_i32", "bucket_col_start_i32",
    "bucket_col_len_i32", "bucket_thread_startbit_u32", "bucket_bit_base_i64", "bitstream_u64",
    "shape_nmk_i64", "bucket_U_i32", "bucket_unique_gid_i32", "bucket_fp8_uidx_i16",
]
AWQ_BUCKET_KEYS = [
    "decode_syms_u16", "decode_lens_u8", "table_scale_u16", "table_qv_u16", "bucket_scale_u16",
    "bucket_row_offsets_i32", "row_indices_i32", "bucket_table_i32", "bucket_col_start_i32",
    "bucket_col_len_i32", "bucket_thread_startbit_u32", "bucket_bit_base_i64", "bitstream_u64",
    "shape_nmk_i64",
]
AWQ_BY_SCALE_KEYS = [
    "decode_syms_u16", "decode_lens_u8", "table_scale_u16", "table_qv_u16", "bucket_scale_u16",
    "bucket_group_offsets_i32", "group_rows_i32", "group_col_start_i32", "bucket_table_i32",
    "bucket_thread_startbit_u32", "bucket_bit_base_i64", "bitstream_u64", "shape_nmkg_i64",
]
AWQ_SHARED_KEYS = [
    "decode_syms_i16", "decode_nbits_u8", "scale_values_u16", "scale_bit_base_i64",
    "chunk_startbit_rel_u32", "chunk_out_base_u32", "chunk_meta_u32", "chunk_scale_id_i32",
    "out_idx_i32", "stream_chunk_ofs_i64", "stream_chunk_ids_i32", "bitstream_u64",
]

_mod = None


def _find():
    if not _REF_DIR.is_dir():
        return None
    for p in sorted(_REF_DIR.glob("mpserve_ref_build*.so")):
        return p
    return None


def available() -> bool:
    return _find() is not None


def module():
    global _mod
    if _mod is None:
        import torch  # noqa: F401  (the extension links against libtorch)

        path = _find()
        if path is None:
            raise RuntimeError("oracle/_ref is not built; run oracle/build_ref.sh where the reference tree exists")
        spec = importlib.util.spec_from_file_location("mpserve_ref_build", str(path))
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod


class _quiet_stdout:
    """The reference encoder prints one line per bucket to C stdout; keep test logs readable."""

    def __enter__(self):
        sys.stdout.flush()
        self._saved = os.dup(1)
        self._null = os.open(os.devnull, os.O_WRONLY)
        os.dup2(self._null, 1)

    def __exit__(self, *exc):
        os.dup2(self._saved, 1)
        os.close(self._null)
        os.close(self._saved)


def build_fp8(bf16, fp8_u8, scales, max_len=12, threads_per_block=256) -> dict:
    with _quiet_stdout():
        out = module().build_fp8(bf16, fp8_u8, scales, int(max_len), int(threads_per_block))
    return dict(zip(FP8_KEYS, out))


def build_awq_bucket(bf16, int4_u8, scales_u16, max_len=11, threads_per_block=256) -> dict:
    with _quiet_stdout():
        out = module().build_awq_bucket(bf16, int4_u8, scales_u16, int(max_len), int(threads_per_block))
    return dict(zip(AWQ_BUCKET_KEYS, out))


def build_awq_by_scale(bf16, int4_u8, scales_u16, max_len=11, threads=256, group_cap=1024) -> dict:
    with _quiet_stdout():
        out = module().build_awq_by_scale(bf16, int4_u8, scales_u16, int(max_len), int(threads), int(group_cap))
    return dict(zip(AWQ_BY_SCALE_KEYS, out))


def build_awq_shared(bf16, int4_u8, scales_u16, max_len=11) -> dict:
    with _quiet_stdout():
        out = module().build_awq_shared(bf16, int4_u8, scales_u16, int(max_len))
    return dict(zip(AWQ_SHARED_KEYS, out))
