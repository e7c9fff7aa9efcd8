"""Parity of the CUDA decoders (called through the MPServe_cuda surface -> C ABI) with the CPU
oracle, the golden fixtures of the reference encoder, and the original BF16 tensors.  Bit-exact."""
import os

import numpy as np
import pytest
import torch

from mpserve_b200 import api, util
from mpserve_b200 import workloads as wl
from oracle import oracle as orc
from tests._util import golden_names

pytestmark = pytest.mark.gpu

CONFIGS = [(256, 4), (512, 2), (256, 1), (256, 2), (128, 8), (128, 4), (512, 1)]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from mpserve_b200 import _lib

    _lib.load()  # fail loudly when the extension is missing
    return torch.device("cuda:0")


@pytest.fixture
def force_config():
    """Pin the decode path: ("direct",) = the per-sub-stream kernel that reads the tables in place,
    (threads, chains) = the persistent kernel in that shape, nothing = the library's own choice."""
    def _set(threads=None, chains=None):
        direct = None
        if threads == "direct":
            threads, direct = None, 1
        elif threads is not None:
            direct = 0
        for k, v in (("MPS_DECODE_THREADS", threads), ("MPS_DECODE_CHAINS", chains), ("MPS_DECODE_DIRECT", direct)):
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = str(v)

    yield _set
    _set(None, None)


DIRECT = ("direct", None)


def _u16(t):
    return t.view(torch.uint16).numpy()


def _fp8_decode(ctx_np, art, n, m, dev):
    import MPServe_cuda

    d = util.artifacts_to_device(art, dev)
    ctx = torch.from_numpy(np.ascontiguousarray(ctx_np)).to(dev)
    out = MPServe_cuda.huffman_decode_fp8(*util.decode_fp8_args(ctx, d, n, m, 7))
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (n, m)
    return util.bf16_bits(out)


def _encode_golden(g):
    p = g.params
    if g.kind == "fp8":
        return orc.build_fp8(g.bf16, g.ctx, g.scales, p["max_len"], p["threads_per_block"])
    if g.kind == "awq_bucket":
        return orc.build_awq_bucket(g.bf16, g.ctx, g.scales, p["max_len"], p["threads_per_block"])
    if g.kind == "awq_by_scale":
        return orc.build_awq_by_scale(g.bf16, g.ctx, g.scales, p["max_len"], p["threads"], p["group_cap"])
    return orc.build_awq_shared(g.bf16, g.ctx, g.scales, p["max_len"])


# ---------------------------------------------------------------------------------------------
# FP8
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", golden_names("fp8"))
@pytest.mark.parametrize("cfg", [None, DIRECT, (256, 4), (512, 1), (128, 8)], ids=str)
def test_fp8_golden(golden_cases, dev, force_config, name, cfg):
    g = golden_cases[name]
    art = _encode_golden(g)
    g.check_artifacts(art)  # the inputs of this decode ARE the reference encoder's bytes
    if cfg:
        force_config(*cfg)
    n, m = g.bf16.shape
    got = _fp8_decode(g.ctx, art, n, m, dev)
    np.testing.assert_array_equal(got, orc.decode_fp8(g.ctx, art, n, m))
    np.testing.assert_array_equal(got, g.bf16)


FP8_SEEDED = [
    # n, m, dist, scale mode, k
    (512, 1024, "normal", "tensor", 1024),
    (300, 4096, "normal", "channel", 1024),
    (256, 2048, "student_t", "channel", 1024),
    (256, 512, "student_t", "block", 256),      # 128x128 blocks: col_len < k_eff multiples
    (129, 1000, "normal", "channel", 1024),     # m % 8 != 0 for some paths, odd row count
    (64, 250, "normal", "tensor", 1024),        # m % 4 != 0 -> generic path
    (200, 3, "normal", "tensor", 256),          # m < 4
    (1, 4096, "normal", "tensor", 1024),
    (2048, 256, "normal", "tensor", 64),        # small k
    (1024, 1024, "normal", "tensor", 1),        # k = 1
    (512, 768, "normal", "channel", 32),
    # rows that do not hold a whole number of steps (m % k != 0): a step spans two rows, and the last step
    # of a bucket may be ragged
    (300, 3584, "normal", "channel", 1024),
    (200, 1536, "normal", "tensor", 1024),
    (77, 2064, "student_t", "channel", 1024),
    (130, 1040, "normal", "tensor", 1024),
    (64, 400, "normal", "tensor", 256),
    (256, 3584, "student_t", "tensor", 512),
]


@pytest.mark.parametrize("case", FP8_SEEDED, ids=lambda c: "x".join(map(str, c)))
def test_fp8_seeded_all_configs(dev, force_config, case):
    n, m, dist, mode, k = case
    c = wl.quantize_fp8(wl.random_weight(n, m, 100 + n + m, dist), mode)
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, k)
    want = orc.decode_fp8(c.fp8_u8.numpy(), art, n, m)
    np.testing.assert_array_equal(want, _u16(c.bf16))
    for cfg in [None, DIRECT] + CONFIGS:
        force_config(*(cfg or (None, None)))
        got = _fp8_decode(c.fp8_u8.numpy(), art, n, m, dev)
        np.testing.assert_array_equal(got, want, err_msg=f"config {cfg}")


def test_fp8_esc_large(dev, force_config):
    """Heavy-tailed per-tensor case: contexts of fp8 codes around zero hold > 128 distinct values."""
    n, m = 2048, 2048
    c = wl.quantize_fp8(wl.random_weight(n, m, 7, "student_t"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    assert ((art["decode_lens_u8"] & 0x88) != 0).any(), "case was meant to contain ESC tables"
    for cfg in (None, DIRECT, (256, 4), (512, 2), (256, 1)):
        force_config(*(cfg or (None, None)))
        got = _fp8_decode(c.fp8_u8.numpy(), art, n, m, dev)
        np.testing.assert_array_equal(got, _u16(c.bf16), err_msg=f"config {cfg}")


def test_fp8_config1_full_size_roundtrip(dev):
    """One 4096x4096 linear weight at full size, N(0,0.02), per-tensor scale, k=1024."""
    n = m = 4096
    c = wl.quantize_fp8(wl.random_weight(n, m, 0, "normal"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    got = _fp8_decode(c.fp8_u8.numpy(), art, n, m, dev)
    np.testing.assert_array_equal(got, _u16(c.bf16))


def test_no_bounded_wait_runs_out_in_normal_operation(dev):
    """Waits in the kernels are bounded and report through the workspace; nothing may report here."""
    n, m = 512, 2048
    c = wl.quantize_fp8(wl.random_weight(n, m, 21, "normal"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    for _ in range(3):
        np.testing.assert_array_equal(_fp8_decode(c.fp8_u8.numpy(), art, n, m, dev), _u16(c.bf16))
    assert api.decode_timed_out(dev) is False


def test_bounded_wait_runs_out_and_is_reported(dev):
    """The give-up path, made to happen on the host's request and without any fault: the producer leaves the
    context bytes of one block out (mps_selftest_stalled_decode), the decoding warps' wait runs out after a
    few thousand polls, the kernel stops taking work, drains what it has in flight and returns; the status
    call says so once, and the very next decode on the same workspace is bit-exact."""
    n, m = 1024, 4096
    c = wl.quantize_fp8(wl.random_weight(n, m, 77, "normal"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    d = util.artifacts_to_device(art, dev)
    ctx = c.fp8_u8.to(dev)
    assert api.decode_timed_out(dev) is False
    out = torch.zeros((n, m), dtype=torch.bfloat16, device=dev)
    api.selftest_stalled_decode(ctx, d, out, stall_block=1, polls=20000)
    torch.cuda.synchronize()
    assert api.decode_timed_out(dev) is True        # reported ...
    assert api.decode_timed_out(dev) is False       # ... once
    assert not np.array_equal(util.bf16_bits(out), _u16(c.bf16))   # the stalled decode did stop early
    for _ in range(2):                               # and left the workspace and the GPU in working order
        np.testing.assert_array_equal(_fp8_decode(c.fp8_u8.numpy(), art, n, m, dev), _u16(c.bf16))
    assert api.decode_timed_out(dev) is False


def test_fp8_repeated_calls_reuse_workspace(dev):
    n, m = 256, 1024
    c = wl.quantize_fp8(wl.random_weight(n, m, 3, "normal"), "channel")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    for _ in range(5):
        np.testing.assert_array_equal(_fp8_decode(c.fp8_u8.numpy(), art, n, m, dev), _u16(c.bf16))


@pytest.mark.parametrize("cfg", [DIRECT, (256, 1)], ids=str)
def test_fp8_missing_table_decodes_zero(dev, force_config, cfg):
    """A context without a table (gid = -1) yields zeros and consumes nothing, as in the reference
    kernel (decode_huffman.cu:252-264); the oracle does the same."""
    n, m = 64, 256
    c = wl.quantize_fp8(wl.random_weight(n, m, 5, "normal"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 256)
    art["bucket_table_i32"][:, 0x30:0x38] = -1
    force_config(*cfg)
    want = orc.decode_fp8(c.fp8_u8.numpy(), art, n, m)
    got = _fp8_decode(c.fp8_u8.numpy(), art, n, m, dev)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("cfg", [DIRECT, (256, 1)], ids=str)
def test_fp8_corrupt_metadata_is_contained(dev, force_config, cfg):
    """Out-of-range rows / windows / offsets must not fault: such buckets are skipped or clamped."""
    n, m = 64, 256
    c = wl.quantize_fp8(wl.random_weight(n, m, 6, "normal"), "channel")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 256)
    bad = dict(art)
    bad["row_indices_i32"] = art["row_indices_i32"].copy()
    bad["row_indices_i32"][0] = n + 1000
    bad["bucket_col_len_i32"] = art["bucket_col_len_i32"].copy()
    bad["bucket_col_len_i32"][-1] = m + 7
    bad["bucket_thread_startbit_u32"] = art["bucket_thread_startbit_u32"].copy()
    bad["bucket_thread_startbit_u32"][1, :] = 0xFFFFFF00
    force_config(*cfg)
    _fp8_decode(c.fp8_u8.numpy(), bad, n, m, dev)  # completes; content of the bad buckets is unspecified
    # the context is still healthy afterwards
    np.testing.assert_array_equal(_fp8_decode(c.fp8_u8.numpy(), art, n, m, dev), _u16(c.bf16))


def test_fp8_argument_validation(dev):
    import MPServe_cuda

    n, m = 16, 64
    c = wl.quantize_fp8(wl.random_weight(n, m, 1, "normal"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 32)
    d = util.artifacts_to_device(art, dev)
    ctx = c.fp8_u8.to(dev)
    args = list(util.decode_fp8_args(ctx, d, n, m, 7))
    with pytest.raises(ValueError, match="max_len must be 7"):
        MPServe_cuda.huffman_decode_fp8(*args[:-1], 12)
    with pytest.raises(ValueError, match="numel must equal"):
        MPServe_cuda.huffman_decode_fp8(*args[:-3], n + 1, m, 7)
    bad = list(args)
    bad[1] = d["bitstream_u64"].view(torch.int64)
    with pytest.raises(ValueError, match="uint64"):
        MPServe_cuda.huffman_decode_fp8(*bad)
    bad = list(args)
    bad[4] = d["bucket_table_i32"][:, :128].contiguous()
    with pytest.raises(ValueError, match=r"\[B,256\]"):
        MPServe_cuda.huffman_decode_fp8(*bad)


@pytest.mark.parametrize("cfg", [(256, 4), (256, 1)], ids=str)
def test_fp8_tables_in_any_order(dev, force_config, cfg):
    """The reference encoder numbers a bucket's tables consecutively in context order, which the decoder
    uses (one bulk copy of the run, expanded in place); a sidecar whose tables are stored in another
    order, or that shares a table between contexts, must decode just the same through the other path."""
    n, m = 512, 4096
    c = wl.quantize_fp8(wl.random_weight(n, m, 21, "normal"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    want = _u16(c.bf16)
    force_config(*cfg)
    np.testing.assert_array_equal(_fp8_decode(c.fp8_u8.numpy(), art, n, m, dev), want)
    G = art["decode_syms_u16"].shape[0]
    perm = np.random.default_rng(3).permutation(G)            # new position of every table
    shuffled = dict(art)
    shuffled["decode_syms_u16"] = np.empty_like(art["decode_syms_u16"])
    shuffled["decode_lens_u8"] = np.empty_like(art["decode_lens_u8"])
    shuffled["decode_syms_u16"][perm] = art["decode_syms_u16"]
    shuffled["decode_lens_u8"][perm] = art["decode_lens_u8"]
    bt = art["bucket_table_i32"].copy()
    bt[bt >= 0] = perm[bt[bt >= 0]].astype(np.int32)
    shuffled["bucket_table_i32"] = bt
    np.testing.assert_array_equal(_fp8_decode(c.fp8_u8.numpy(), shuffled, n, m, dev), want)
    # a run of consecutive ids that does not start at the first context's table: reversed order
    rev = dict(art)
    rev["decode_syms_u16"] = art["decode_syms_u16"][::-1].copy()
    rev["decode_lens_u8"] = art["decode_lens_u8"][::-1].copy()
    bt = art["bucket_table_i32"].copy()
    bt[bt >= 0] = (G - 1 - bt[bt >= 0]).astype(np.int32)
    rev["bucket_table_i32"] = bt
    np.testing.assert_array_equal(_fp8_decode(c.fp8_u8.numpy(), rev, n, m, dev), want)


def test_fp8_checked_arguments_are_remembered_but_rechecked_when_they_change(dev):
    """A second call with the same tensor objects skips the argument checks; a tensor changed in place
    between two calls (another dtype, another shape, other storage) is checked again in full."""
    import MPServe_cuda
    from mpserve_b200 import api

    n, m = 256, 1024
    c = wl.quantize_fp8(wl.random_weight(n, m, 8, "normal"), "tensor")
    art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    d = util.artifacts_to_device(art, dev)
    args = list(util.decode_fp8_args(c.fp8_u8.to(dev), d, n, m, 7))
    want = _u16(c.bf16)
    api._fp8_checked.clear()
    np.testing.assert_array_equal(util.bf16_bits(MPServe_cuda.huffman_decode_fp8(*args)), want)
    assert len(api._fp8_checked) == 1
    memo = next(iter(api._fp8_checked.values()))
    assert memo.still_holds(args[:11])
    np.testing.assert_array_equal(util.bf16_bits(MPServe_cuda.huffman_decode_fp8(*args)), want)
    assert len(api._fp8_checked) == 1 and next(iter(api._fp8_checked.values())) is memo

    table = args[4]
    kept = table.data
    table.data = kept.to(torch.int64)                       # same object, another dtype
    assert not memo.still_holds(args[:11])
    with pytest.raises(ValueError, match="int32"):
        MPServe_cuda.huffman_decode_fp8(*args)
    table.data = kept[:, :128].contiguous()                 # same object, another shape
    with pytest.raises(ValueError, match=r"\[B,256\]"):
        MPServe_cuda.huffman_decode_fp8(*args)
    table.data = kept.clone()                               # same object, same facts, other storage
    assert not memo.still_holds(args[:11])
    np.testing.assert_array_equal(util.bf16_bits(MPServe_cuda.huffman_decode_fp8(*args)), want)
    # a new tensor object is a new entry, never a stale hit
    fresh = list(args)
    fresh[4] = kept.clone()
    np.testing.assert_array_equal(util.bf16_bits(MPServe_cuda.huffman_decode_fp8(*fresh)), want)


def test_fp8_batch_plan_matches_single(dev):
    # per-channel tensors of this size have tiny buckets (decoded one by one, in place); the per-tensor
    # ones have full 128-row buckets and share the persistent launch
    shapes = [(256, 1024, "channel"), (512, 512, "tensor"), (1024, 256, "channel"), (8, 4096, "channel"),
              (1024, 2048, "tensor")]
    entries, wants = [], []
    for i, (n, m, mode) in enumerate(shapes):
        c = wl.quantize_fp8(wl.random_weight(n, m, 40 + i, "normal"), mode)
        art = orc.build_fp8(_u16(c.bf16), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
        entries.append((c.fp8_u8.to(dev), util.artifacts_to_device(art, dev), None))
        wants.append(_u16(c.bf16))
    plan = api.BucketDecodePlan(entries, mode=0)
    assert plan._direct and plan.total_items > 0, "the case was meant to exercise both kernels"
    for _ in range(2):
        outs = plan.decode()
        torch.cuda.synchronize()
        for o, w in zip(outs, wants):
            np.testing.assert_array_equal(util.bf16_bits(o), w)
        for o in outs:
            o.zero_()


# ---------------------------------------------------------------------------------------------
# AWQ
# ---------------------------------------------------------------------------------------------

def _awq_decode(kind, ctx_np, art, n, m, dev, L=11):
    import MPServe_cuda

    d = util.artifacts_to_device(art, dev)
    ctx = torch.from_numpy(np.ascontiguousarray(ctx_np)).to(dev)
    if kind == "awq_bucket":
        out = MPServe_cuda.huffman_decode_awq_int4_bucket(
            ctx, d["bitstream_u64"], d["decode_syms_u16"], d["decode_lens_u8"], d["bucket_table_i32"],
            d["bucket_col_start_i32"], d["bucket_col_len_i32"], d["bucket_row_offsets_i32"], d["row_indices_i32"],
            d["bucket_thread_startbit_u32"], d["bucket_bit_base_i64"], n, m, L)
    elif kind == "awq_by_scale":
        out = MPServe_cuda.huffman_decode_awq_int4_bucket_by_scale(
            ctx, d["bitstream_u64"], d["decode_syms_u16"], d["decode_lens_u8"], d["bucket_table_i32"],
            d["bucket_group_offsets_i32"], d["group_rows_i32"], d["group_col_start_i32"],
            d["bucket_thread_startbit_u32"], d["bucket_bit_base_i64"], n, m, L, int(art["shape_nmkg_i64"][3]))
    else:
        out = MPServe_cuda.huffman_decode_awq_shared_table(
            d["bitstream_u64"], d["decode_syms_i16"], d["decode_nbits_u8"], d["scale_bit_base_i64"],
            d["chunk_startbit_rel_u32"], d["chunk_out_base_u32"], d["chunk_meta_u32"], d["chunk_scale_id_i32"],
            d["out_idx_i32"], d["stream_chunk_ofs_i64"], d["stream_chunk_ids_i32"], n * m, L)
        torch.cuda.synchronize()
        assert out.dtype == torch.int16
        return out.cpu().numpy().view(np.uint16).reshape(n, m)
    torch.cuda.synchronize()
    return util.bf16_bits(out)


@pytest.mark.parametrize("name", golden_names("awq"))
@pytest.mark.parametrize("cfg", [DIRECT, (256, 1)], ids=str)
def test_awq_golden(golden_cases, dev, force_config, name, cfg):
    g = golden_cases[name]
    force_config(*cfg)
    art = _encode_golden(g)
    g.check_artifacts(art)
    n, m = g.bf16.shape
    got = _awq_decode(g.kind, g.ctx, art, n, m, dev, g.params["max_len"])
    np.testing.assert_array_equal(got, g.bf16)


@pytest.mark.parametrize("scale_kind", ["group", "row", "scalar"])
def test_awq_seeded(dev, force_config, scale_kind):
    n, m = 256, 1024
    c = wl.quantize_awq(wl.random_weight(n, m, 77, "normal"), 128)
    sc = c.scales_u16.numpy()
    if scale_kind == "row":
        sc = np.ascontiguousarray(sc[:, 0])
    elif scale_kind == "scalar":
        sc = np.ascontiguousarray(sc[:1, 0])
    q, b = c.int4_u8.numpy(), _u16(c.bf16)
    arts = {
        "awq_bucket": orc.build_awq_bucket(b, q, sc, 11, 256),
        "awq_by_scale": orc.build_awq_by_scale(b, q, sc, 11, 256, 1024),
        "awq_shared": orc.build_awq_shared(b, q, sc, 11),
    }
    for kind, art in arts.items():
        for cfg in (None, DIRECT, (256, 1), (128, 4)):
            force_config(*(cfg or (None, None)))
            got = _awq_decode(kind, q, art, n, m, dev)
            np.testing.assert_array_equal(got, b, err_msg=f"{kind} {cfg}")


# ---------------------------------------------------------------------------------------------
# checksum
# ---------------------------------------------------------------------------------------------

def test_checksum_matches_numpy(dev):
    rng = np.random.default_rng(0)
    a = rng.integers(0, 65536, size=1_000_003, dtype=np.uint16)
    acc = api.checksum_u16(torch.from_numpy(a).to(dev).view(torch.bfloat16))
    torch.cuda.synchronize()
    got = acc.cpu().numpy().view(np.uint64)
    want_sum = np.uint64(a.astype(np.uint64).sum())
    want_xor = np.bitwise_xor.reduce(a.astype(np.uint64) * (np.arange(a.size, dtype=np.uint64) + np.uint64(1)))
    assert got[0] == want_sum and got[1] == want_xor
