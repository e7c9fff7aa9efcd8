"""The GPU sidecar builder against the CPU oracle and the reference encoder's golden artifacts:
every returned tensor byte-identical."""
import numpy as np
import pytest
import torch

from mpserve_b200 import workloads as wl
from oracle import oracle as orc
from tests._util import golden_names

pytestmark = pytest.mark.gpu


def _np(t):
    return t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def _same(got: dict, want: dict, tag: str):
    assert set(got) == set(want), (sorted(got), sorted(want))
    for k, w in want.items():
        g = _np(got[k].cpu())
        assert g.dtype == w.dtype and g.shape == w.shape, (tag, k, g.dtype, w.dtype, g.shape, w.shape)
        np.testing.assert_array_equal(g, w, err_msg=f"{tag}:{k}")


@pytest.mark.parametrize("name", golden_names("fp8"))
def test_fp8_builder_matches_reference_golden(golden_cases, name):
    import MPServe_cuda

    g = golden_cases[name]
    p = g.params
    got = MPServe_cuda.huffman_build_fp8_decode_tables(
        torch.from_numpy(g.bf16).view(torch.bfloat16), torch.from_numpy(g.ctx), torch.from_numpy(g.scales),
        max_len=p["max_len"], threads_per_block=p["threads_per_block"])
    g.check_artifacts({k: _np(v) for k, v in got.items()})


@pytest.mark.parametrize("name", [n for n in golden_names("awq") if n.endswith("_bucket")])
def test_awq_bucket_builder_matches_reference_golden(golden_cases, name):
    import MPServe_cuda

    g = golden_cases[name]
    p = g.params
    got = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables(
        torch.from_numpy(g.bf16).view(torch.bfloat16), torch.from_numpy(g.ctx), torch.from_numpy(g.scales),
        max_len=p["max_len"], threads_per_block=p["threads_per_block"])
    g.check_artifacts({k: _np(v) for k, v in got.items()})


FP8_CASES = [
    (512, 1024, "normal", "tensor", 7, 1024),
    (300, 4096, "normal", "channel", 7, 1024),
    (256, 512, "student_t", "block", 7, 256),
    (1024, 1024, "student_t", "tensor", 7, 1024),
    (129, 1000, "normal", "channel", 7, 1024),
    (3, 5, "normal", "tensor", 7, 32),
    (512, 512, "normal", "tensor", 5, 128),     # many ESC contexts at a short max_len
    (512, 512, "normal", "tensor", 12, 256),
    (2048, 2048, "student_t", "tensor", 7, 1024),
]


@pytest.mark.parametrize("case", FP8_CASES, ids=lambda c: "x".join(map(str, c)))
def test_fp8_builder_matches_oracle(case):
    import MPServe_cuda

    n, m, dist, mode, L, k = case
    c = wl.quantize_fp8(wl.random_weight(n, m, 300 + n + m, dist), mode)
    want = orc.build_fp8(c.bf16.view(torch.uint16).numpy(), c.fp8_u8.numpy(), c.scales_u16.numpy(), L, k)
    got = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=L, threads_per_block=k)
    _same(got, want, str(case))


@pytest.mark.parametrize("scale_kind,L", [("group", 11), ("row", 11), ("scalar", 11), ("scalar", 6), ("row", 8)])
def test_awq_bucket_builder_matches_oracle(scale_kind, L):
    import MPServe_cuda

    n, m = 128, 512
    c = wl.quantize_awq(wl.random_weight(n, m, 55, "student_t" if L != 11 else "normal"), 128)
    sc = c.scales_u16
    if scale_kind == "row":
        sc = sc[:, 0].contiguous()
    elif scale_kind == "scalar":
        sc = sc[:1, 0].contiguous().reshape(1)
    want = orc.build_awq_bucket(c.bf16.view(torch.uint16).numpy(), c.int4_u8.numpy(), sc.numpy(), L, 256)
    got = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables(c.bf16, c.int4_u8, sc, max_len=L,
                                                                   threads_per_block=256)
    _same(got, want, f"{scale_kind} L={L}")


@pytest.mark.parametrize("name", [n for n in golden_names("awq") if n.endswith("_byscale")])
def test_awq_by_scale_builder_matches_reference_golden(golden_cases, name):
    import MPServe_cuda

    g = golden_cases[name]
    p = g.params
    got = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables_by_scale(
        torch.from_numpy(g.bf16).view(torch.bfloat16), torch.from_numpy(g.ctx), torch.from_numpy(g.scales),
        max_len=p["max_len"], threads=p["threads"], group_cap=p["group_cap"])
    g.check_artifacts({k: _np(v) for k, v in got.items()})


@pytest.mark.parametrize("scale_kind,L,cap", [("group", 11, 1024), ("row", 11, 5), ("scalar", 11, 1024),
                                                 ("scalar", 6, 3), ("row", 8, 1024)])
def test_awq_by_scale_builder_matches_oracle(scale_kind, L, cap):
    import MPServe_cuda

    n, m = 128, 512
    c = wl.quantize_awq(wl.random_weight(n, m, 56, "student_t" if L != 11 else "normal"), 128)
    sc = c.scales_u16
    if scale_kind == "row":
        sc = sc[:, 0].contiguous()
    elif scale_kind == "scalar":
        sc = sc[:1, 0].contiguous().reshape(1)
    want = orc.build_awq_by_scale(c.bf16.view(torch.uint16).numpy(), c.int4_u8.numpy(), sc.numpy(), L, 256, cap)
    got = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables_by_scale(c.bf16, c.int4_u8, sc, max_len=L,
                                                                            threads=256, group_cap=cap)
    _same(got, want, f"{scale_kind} L={L}")


@pytest.mark.parametrize("name", [n for n in golden_names("awq") if n.endswith("_shared")])
def test_awq_shared_builder_matches_reference_golden(golden_cases, name):
    import MPServe_cuda

    g = golden_cases[name]
    got = MPServe_cuda.huffman_build_awq_decode_tables(
        torch.from_numpy(g.bf16).view(torch.bfloat16), torch.from_numpy(g.ctx), torch.from_numpy(g.scales),
        max_len=g.params["max_len"])
    g.check_artifacts({k: _np(v) for k, v in got.items()})


@pytest.mark.parametrize("scale_kind,L,dist", [("group", 11, "normal"), ("row", 11, "normal"), ("scalar", 11, "normal"),
                                                ("scalar", 6, "student_t"), ("row", 8, "student_t"),
                                                ("group", 9, "student_t")])
def test_awq_shared_builder_matches_oracle(scale_kind, L, dist):
    import MPServe_cuda

    n, m = 128, 512
    c = wl.quantize_awq(wl.random_weight(n, m, 57, dist), 128)
    sc = c.scales_u16
    if scale_kind == "row":
        sc = sc[:, 0].contiguous()
    elif scale_kind == "scalar":
        sc = sc[:1, 0].contiguous().reshape(1)
    want = orc.build_awq_shared(c.bf16.view(torch.uint16).numpy(), c.int4_u8.numpy(), sc.numpy(), L)
    got = MPServe_cuda.huffman_build_awq_decode_tables(c.bf16, c.int4_u8, sc, max_len=L)
    _same(got, want, f"{scale_kind} L={L}")


@pytest.mark.parametrize("n,m", [(256, 1024), (2048, 4096)])   # the larger one spans many grid strides
def test_awq_shared_build_then_decode_on_device(n, m):
    import MPServe_cuda

    dev = torch.device("cuda:0")
    c = wl.quantize_awq(wl.random_weight(n, m, 58, "normal"), 128)
    d = MPServe_cuda.huffman_build_awq_decode_tables(c.bf16.to(dev), c.int4_u8.to(dev), c.scales_u16.to(dev), max_len=11)
    assert all(v.is_cuda for k, v in d.items() if k != "scale_values_u16")
    out = MPServe_cuda.huffman_decode_awq_shared_table(
        d["bitstream_u64"], d["decode_syms_i16"], d["decode_nbits_u8"], d["scale_bit_base_i64"],
        d["chunk_startbit_rel_u32"], d["chunk_out_base_u32"], d["chunk_meta_u32"], d["chunk_scale_id_i32"],
        d["out_idx_i32"], d["stream_chunk_ofs_i64"], d["stream_chunk_ids_i32"], n * m, 11)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16).reshape(n, m).cpu(), c.bf16.view(torch.uint16))


def test_build_then_decode_roundtrip_on_device():
    """Encoder output fed straight to the decoder, everything resident on the GPU."""
    import MPServe_cuda
    from mpserve_b200 import util

    dev = torch.device("cuda:0")
    n, m = 1024, 4096
    c = wl.quantize_fp8(wl.random_weight(n, m, 9, "normal"), "channel")
    art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16.to(dev), c.fp8_u8.to(dev), c.scales_u16.to(dev),
                                                       max_len=7, threads_per_block=1024)
    assert art["bitstream_u64"].is_cuda
    out = MPServe_cuda.huffman_decode_fp8(*util.decode_fp8_args(c.fp8_u8.to(dev), art, n, m, 7))
    torch.cuda.synchronize()
    assert torch.equal(out.cpu().view(torch.uint16), c.bf16.view(torch.uint16))


@pytest.mark.parametrize("n,m,k", [(14336, 4096, 1024),    # widest weight of an 8B-shaped layer
                                   (8192, 3584, 1024),     # row-parallel shard whose rows do not hold whole steps
                                   (4096, 4096, 256)])     # the reference builder's default sub-stream count
def test_full_size_build_decode_checksum_on_device(n, m, k):
    """Full-size tensors, everything on the GPU: the builder's sidecar decodes back to the source bit for
    bit (a lossless round trip does not depend on the size), and the device checksum agrees with torch."""
    import MPServe_cuda
    from mpserve_b200 import api, util

    dev = torch.device("cuda:0")
    c = wl.quantize_fp8(wl.random_weight(n, m, 4242, "normal", device=dev), "channel")
    art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=k)
    out = MPServe_cuda.huffman_decode_fp8(*util.decode_fp8_args(c.fp8_u8, art, n, m, 7))
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16))
    acc = api.checksum_u16(out)
    assert int(acc.cpu()[0]) % (1 << 64) == int(c.bf16.view(torch.uint16).to(torch.int64).sum()) % (1 << 64)


def test_bucket_unique_lists_with_repeats_and_holes():
    """The first-appearance list of a bucket's tables, on a table with repeated ids (inside one group of
    32 contexts and across groups), absent contexts and the extremes of zero and 256 distinct ids; the
    expected result is the sequential scan of build_huffman.cu:748-783 written as a Python loop."""
    import ctypes as C

    from mpserve_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    B = 37
    bt = rng.integers(-1, 40, size=(B, 256), dtype=np.int32)           # many repeats, some holes
    bt[0] = -1                                                          # no table at all
    bt[1] = np.arange(256, dtype=np.int32)[::-1] + 1000                 # all distinct
    bt[2] = 7                                                           # a single id
    bt[3] = np.repeat(np.arange(8, dtype=np.int32), 32)                 # one id per group of 32
    bt[4] = np.tile(np.arange(32, dtype=np.int32), 8)                   # every group repeats the first
    bt[5:9] = rng.integers(-1, 100000, size=(4, 256), dtype=np.int32)   # mostly distinct
    want_u = np.zeros(B, np.int32)
    want_list = np.full((B, 256), -1, np.int32)
    want_idx = np.full((B, 256), -1, np.int16)
    for b in range(B):
        seen: dict[int, int] = {}
        for i in range(256):
            g = int(bt[b, i])
            if g < 0:
                continue
            if g not in seen:
                seen[g] = len(seen)
                want_list[b, seen[g]] = g
            want_idx[b, i] = seen[g]
        want_u[b] = len(seen)
    bt_d = torch.from_numpy(bt).to(dev)
    U = torch.full((B,), -7, dtype=torch.int32, device=dev)
    uniq = torch.full((B, 256), -7, dtype=torch.int32, device=dev)
    uidx = torch.full((B, 256), -7, dtype=torch.int16, device=dev)
    _lib.check(lib.mps_build_bucket_unique(bt_d.data_ptr(), B, U.data_ptr(), uniq.data_ptr(), uidx.data_ptr(),
                                           C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(U.cpu().numpy(), want_u)
    np.testing.assert_array_equal(uniq.cpu().numpy(), want_list)
    np.testing.assert_array_equal(uidx.cpu().numpy(), want_idx)
