"""Host-side pieces of the sidecar builder (no GPU): bucket lists made from the scale tensor must be
the ones the reference encoder makes (checked through the oracle, itself pinned to the reference)."""
import numpy as np
import pytest
import torch

from mpserve_b200 import api, encoder
from mpserve_b200 import workloads as wl
from oracle import oracle as orc


def _case(n, m, mode, seed=3, block=(64, 128)):
    c = wl.quantize_fp8(wl.random_weight(n, m, seed, "normal"), mode, block)
    art = orc.build_fp8(c.bf16.view(torch.uint16).numpy(), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 64)
    return c, art


@pytest.mark.parametrize("n,m,mode", [(300, 256, "channel"), (64, 128, "tensor"), (256, 512, "block"), (1, 64, "tensor"),
                                      (257, 64, "tensor")])
def test_rect_buckets_match_reference_layout(n, m, mode):
    c, art = _case(n, m, mode)
    smode, nb0, nb1, sb0, sb1 = encoder._scale_mode(c.scales_u16, n, m, True)
    b_scale, b_ofs, rows, cs, cl = encoder.rect_buckets(c.scales_u16.numpy(), smode, n, m, nb0, nb1, sb0, sb1)
    np.testing.assert_array_equal(b_scale, art["bucket_scale_u16"])
    np.testing.assert_array_equal(b_ofs, art["bucket_row_offsets_i32"])
    np.testing.assert_array_equal(rows, art["row_indices_i32"])
    np.testing.assert_array_equal(cs, art["bucket_col_start_i32"])
    np.testing.assert_array_equal(cl, art["bucket_col_len_i32"])


@pytest.mark.parametrize("kind,cap", [("group", 1024), ("group", 7), ("row", 3), ("scalar", 1024)])
def test_ragged_buckets_match_reference_layout(kind, cap):
    n, m = 64, 512
    c = wl.quantize_awq(wl.random_weight(n, m, 5, "normal"), 128)
    sc = c.scales_u16
    if kind == "row":
        sc = sc[:, 0].contiguous()
    elif kind == "scalar":
        sc = sc[:1, 0].contiguous().reshape(1)
    art = orc.build_awq_by_scale(c.bf16.view(torch.uint16).numpy(), c.int4_u8.numpy(), sc.numpy(), 11, 64, cap)
    smode, nb0, nb1, sb0, sb1 = encoder._scale_mode(sc, n, m, False)
    b_scale, b_ofs, rows, cols, gsize = encoder.ragged_buckets(sc.numpy(), smode, n, m, nb1, sb0, sb1, cap)
    np.testing.assert_array_equal(b_scale, art["bucket_scale_u16"])
    np.testing.assert_array_equal(b_ofs, art["bucket_group_offsets_i32"])
    np.testing.assert_array_equal(rows, art["group_rows_i32"])
    np.testing.assert_array_equal(cols, art["group_col_start_i32"])
    assert gsize == int(art["shape_nmkg_i64"][3])


def test_scale_mode_rules_follow_the_reference():
    n, m = 8, 16
    u16 = lambda *shape: torch.zeros(shape, dtype=torch.uint16)
    assert encoder._scale_mode(u16(1), n, m, True)[0] == 0
    assert encoder._scale_mode(u16(n), n, m, True)[0] == 1
    assert encoder._scale_mode(u16(n, 1), n, m, True)[0] == 1          # FP8: any shape with n elements is per-row
    assert encoder._scale_mode(u16(2, 4), n, m, True)[0] == 1          # 8 elements == n: still per-row
    assert encoder._scale_mode(u16(2, 2), n, m, True)[0] == 2
    with pytest.raises(ValueError):
        encoder._scale_mode(u16(n, m), n, m, True)                      # per-element: no bucket packing
    with pytest.raises(ValueError):
        encoder._scale_mode(u16(3), n, m, True)
    with pytest.raises(ValueError):
        encoder._scale_mode(u16(3, 5), n, m, False)


def test_builder_argument_checks_without_gpu():
    import MPServe_cuda

    w = torch.zeros((4, 8), dtype=torch.bfloat16)
    q = torch.zeros((4, 8), dtype=torch.uint8)
    s = torch.zeros(1, dtype=torch.uint16)
    with pytest.raises(ValueError, match="bfloat16"):
        MPServe_cuda.huffman_build_fp8_decode_tables(w.float(), q, s, 7, 32)
    with pytest.raises(ValueError, match="threads_per_block"):
        MPServe_cuda.huffman_build_fp8_decode_tables(w, q, s, 7, 4096)
    with pytest.raises(ValueError, match=r"threads_per_block must be in \[1, 1024\]"):
        MPServe_cuda.huffman_build_fp8_decode_tables(w, q, s, 7, 1025)   # the reference's limit under the reference's name
    with pytest.raises(ValueError, match=r"threads_per_block must be in \[1, 8192\]"):
        api.build_fp8_fine_substreams(w, q, s, 7, api.MAX_SUBSTREAMS + 1)
    with pytest.raises(ValueError, match="max_len"):
        MPServe_cuda.huffman_build_fp8_decode_tables(w, q, s, 16, 32)
    with pytest.raises(ValueError, match="same numel"):
        MPServe_cuda.huffman_build_fp8_decode_tables(w, q[:2], s, 7, 32)
    with pytest.raises(ValueError, match="uint16"):
        MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables(w, q, s.to(torch.int32), 11, 32)
    with pytest.raises(ValueError, match="group_cap"):
        MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables_by_scale(w, q, s, 11, 32, 0)
