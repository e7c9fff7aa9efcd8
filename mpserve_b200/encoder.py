"""Sidecar builders (the ``huffman_build_*`` entry points).  GPU implementation pending in this
build; the calls fail loudly rather than fall back to a CPU path."""
from __future__ import annotations


def _missing(name: str):
    raise NotImplementedError(f"{name}: the GPU sidecar builder is not part of this build of libmpserve_b200.so")


def build_fp8(bf16_params, fp8_params, scales, max_len, threads_per_block):
    _missing("huffman_build_fp8_decode_tables")


def build_awq_bucket(bf16_params, int4_values_u8, scales_u16, max_len, threads_per_block):
    _missing("huffman_build_awq_int4_bucket_decode_tables")


def build_awq_by_scale(bf16_values, int4_values, scales_u16, max_len, threads, group_cap):
    _missing("huffman_build_awq_int4_bucket_decode_tables_by_scale")


def build_awq_shared(bf16_params, int4_values_u8, scales_u16, max_len):
    _missing("huffman_build_awq_decode_tables")
