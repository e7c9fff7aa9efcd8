"""Bit-exact parity at the shapes of the benchmark configurations that the other GPU tests do not reach:
the size sweep (config 3), the Llama-3-8B linears as AWQ INT4 in every sidecar layout (config 4) and the
tensor-parallel shard shapes of the Llama-3-70B-shaped model at TP=8 (config 5).

Inputs are seeded synthetic weights with the shapes, distributions and quantisers the configurations
name (mpserve_b200/workloads.py); sidecars are built on the GPU by this library's builder, whose
artifacts the encoder tests pin byte for byte to the reference encoder.  Where the CPU oracle finishes
in seconds the decode is compared with the oracle's decode of the same sidecar as well; at the full
sizes it is compared with the source tensor (the codec is lossless: decode(encode(w)) == w), and the
device checksum of the output with the checksum of the source.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from mpserve_b200 import api, util
from mpserve_b200 import workloads as wl
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

FP8_KEYS = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_col_start_i32",
            "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32", "bucket_thread_startbit_u32",
            "bucket_bit_base_i64")
BYSCALE_KEYS = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_group_offsets_i32",
                "group_rows_i32", "group_col_start_i32", "bucket_thread_startbit_u32", "bucket_bit_base_i64")
SHARED_KEYS = ("bitstream_u64", "decode_syms_i16", "decode_nbits_u8", "scale_bit_base_i64", "chunk_startbit_rel_u32",
               "chunk_out_base_u32", "chunk_meta_u32", "chunk_scale_id_i32", "out_idx_i32", "stream_chunk_ofs_i64",
               "stream_chunk_ids_i32")


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def _same(out: torch.Tensor, src: torch.Tensor) -> None:
    assert torch.equal(out.view(torch.uint16), src.view(torch.uint16))
    got = api.checksum_u16(out).cpu()
    want = api.checksum_u16(src.contiguous()).cpu()
    assert torch.equal(got, want)


def _fp8_roundtrip(n, m, dist, mode, seed, dev, with_oracle):
    import MPServe_cuda

    c = wl.quantize_fp8(wl.random_weight(n, m, seed, dist, device=dev), mode)
    art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=1024)
    out = MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *[art[k] for k in FP8_KEYS], n, m, 7)
    torch.cuda.synchronize()
    _same(out, c.bf16)
    if with_oracle:
        host = {k: v.cpu().numpy() for k, v in art.items()}
        want = orc.decode_fp8(c.fp8_u8.cpu().numpy(), host, n, m)
        np.testing.assert_array_equal(util.bf16_bits(out), want)
    assert api.decode_timed_out(dev) is False


# ---- config 3: single tensors by size, N(0, 0.02) and Student-t(4) x 0.02, per-channel scales ----------------

@pytest.mark.parametrize("dist", ["normal", "student_t"])
@pytest.mark.parametrize("n,m", [(128, 256), (2048, 4096), (16384, 8192)], ids=["64KB", "16MB", "256MB"])
def test_size_sweep_points(dev, n, m, dist):
    _fp8_roundtrip(n, m, dist, "channel", 11, dev, with_oracle=n * m <= 2048 * 4096)


def test_size_sweep_largest_point(dev):
    """1 GB of BF16 output from one call: 32-bit element offsets, long bitstreams, thousands of buckets."""
    _fp8_roundtrip(32768, 16384, "normal", "channel", 11, dev, with_oracle=False)


# ---- config 5: the five shard shapes of the 70B-shaped model at TP=8 -------------------------------------------

@pytest.mark.parametrize("name,n,m", [("q/o (column parallel)", 1024, 8192), ("k/v", 128, 8192), ("o (row parallel)", 8192, 1024),
                                      ("gate/up", 3584, 8192), ("down", 8192, 3584)], ids=lambda v: str(v))
def test_tp8_shard_shapes(dev, name, n, m):
    _fp8_roundtrip(n, m, "normal", "channel", 500 + n % 97, dev, with_oracle=n * m <= 1024 * 8192)


@pytest.mark.parametrize("n,m", [(5, 3584), (3, 1552), (7, 2064), (130, 1040), (64, 3600)], ids=lambda v: str(v))
def test_rows_that_split_steps_with_a_ragged_last_step(dev, n, m):
    """Rows longer than a step that do not hold whole steps (widths that are multiples of 16 but not of
    1024), in buckets whose element count is no multiple of the sub-streams either: the last step holds an
    element for the first sub-streams only.  One scale for the whole tensor, so a bucket is up to 128 rows."""
    _fp8_roundtrip(n, m, "normal", "tensor", 77 + n, dev, with_oracle=True)


def test_tp8_shards_in_one_plan(dev):
    """All seven shards of one layer of a TP=8 rank through one persistent launch."""
    import MPServe_cuda

    entries, srcs = [], []
    for i, (name, n, m) in enumerate(wl.layer_linears(wl.LLAMA3_70B)):
        sn, sm = wl.tp_shard_shape(name, n, m, 8)
        c = wl.quantize_fp8(wl.random_weight(sn, sm, 900 + i, "normal", device=dev), "channel")
        art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=1024)
        entries.append((c.fp8_u8, {k: art[k] for k in FP8_KEYS}, None))
        srcs.append(c.bf16)
    plan = api.BucketDecodePlan(entries, mode=0)
    outs = plan.decode()
    torch.cuda.synchronize()
    for o, s in zip(outs, srcs):
        _same(o, s)
    assert api.decode_timed_out(dev) is False


# ---- config 4: an 8B-shaped linear as INT4 AWQ (group 128), every layout -----------------------------------------

@pytest.mark.parametrize("layout", ["byscale", "bucket", "shared"])
@pytest.mark.parametrize("name,n,m", [("k_proj", 1024, 4096), ("o_proj", 4096, 4096)], ids=["k_proj", "o_proj"])
def test_awq_8b_shapes(dev, layout, name, n, m):
    import MPServe_cuda

    c = wl.quantize_awq(wl.random_weight(n, m, 100, "normal", device=dev), 128)
    if layout == "bucket":
        art = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables(c.bf16, c.int4_u8, c.scales_u16, max_len=11,
                                                                       threads_per_block=256)
        out = MPServe_cuda.huffman_decode_awq_int4_bucket(c.int4_u8, *[art[k] for k in FP8_KEYS], n, m, 11)
    elif layout == "shared":
        art = MPServe_cuda.huffman_build_awq_decode_tables(c.bf16, c.int4_u8, c.scales_u16, max_len=11)
        out = MPServe_cuda.huffman_decode_awq_shared_table(*[art[k] for k in SHARED_KEYS], n * m, 11)
        out = out.view(torch.bfloat16).view(n, m)
    else:
        art = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables_by_scale(c.bf16, c.int4_u8, c.scales_u16,
                                                                                max_len=11, threads=256, group_cap=1024)
        out = MPServe_cuda.huffman_decode_awq_int4_bucket_by_scale(c.int4_u8, *[art[k] for k in BYSCALE_KEYS], n, m, 11,
                                                                   int(art["shape_nmkg_i64"][3]))
    torch.cuda.synchronize()
    _same(out, c.bf16)
    if layout == "byscale" and n * m <= 1024 * 4096:
        host = {k: (v.cpu().numpy() if isinstance(v, torch.Tensor) else v) for k, v in art.items()}
        want = orc.decode_awq_by_scale(c.int4_u8.cpu().numpy(), host, n, m, int(art["shape_nmkg_i64"][3]))
        np.testing.assert_array_equal(util.bf16_bits(out), want)
