"""Host side of a decode launch (no GPU): which tensors get work items, how many, and the launch shape
(`mps_bucket_batch_plan` reads sizes from host descriptors and dereferences no device pointer; without a
device it plans for 148 SMs)."""
import ctypes as C

import pytest

from mpserve_b200 import _lib


@pytest.fixture(autouse=True)
def no_overrides(monkeypatch):
    for name in ("MPS_DECODE_THREADS", "MPS_DECODE_CHAINS", "MPS_DECODE_DIRECT"):
        monkeypatch.delenv(name, raising=False)


def _tensor(n, m, buckets, k, mode=0, group_size=0):
    t = _lib.BucketTensor()
    fake = 0x10000   # never dereferenced by the planner; aligned like anything a CUDA allocator returns
    for name in ("ctx_bytes", "bitstream", "decode_syms", "decode_lens", "bucket_table", "bucket_col_start",
                 "bucket_col_len", "bucket_row_offsets", "row_indices", "group_col_start", "thread_startbit",
                 "bucket_bit_base", "out"):
        setattr(t, name, fake)
    t.bitstream_words, t.num_tables, t.num_rows, t.num_buckets = 1 << 20, buckets * 200, n, buckets
    t.k, t.group_size, t.mode, t.n, t.m = k, group_size, mode, n, m
    return t


def _plan(tensors):
    lib = _lib.load()
    arr = (_lib.BucketTensor * len(tensors))(*tensors)
    prefix = (C.c_int64 * (len(tensors) + 1))()
    threads, chains = C.c_int32(0), C.c_int32(0)
    rc = lib.mps_bucket_batch_plan(arr, len(tensors), prefix, C.byref(threads), C.byref(chains))
    return rc, list(prefix), threads.value, chains.value


def test_whole_model_takes_the_widest_items():
    tensors = [_tensor(4096, 4096, 111, 1024) for _ in range(64)] + [_tensor(14336, 4096, 190, 1024) for _ in range(32)]
    rc, prefix, threads, chains = _plan(tensors)
    assert rc == 0 and (threads, chains) == (256, 4)
    assert prefix[1] - prefix[0] == 111 and prefix[-1] == 64 * 111 + 32 * 190   # one item per bucket


@pytest.mark.parametrize("k,shape,items", [(1024, (256, 1), 128), (2048, (256, 2), 128), (4096, (256, 4), 128),
                                           (8192, (256, 4), 256), (256, (256, 1), 32)])
def test_lone_weight_of_few_buckets(k, shape, items):
    """32 buckets: narrower items while every item still finds an SM of its own; buckets that are several
    items each (more sub-streams than an item holds) are not cut further than that."""
    rc, prefix, threads, chains = _plan([_tensor(4096, 4096, 32, k)])
    assert rc == 0 and (threads, chains) == shape and prefix[1] == items


def test_whole_buckets_are_halved_up_to_the_sm_count_only():
    assert _plan([_tensor(8192, 8192, 129, 1024)])[2:] == (256, 2)   # 129 items at full width: halve once
    assert _plan([_tensor(8192, 8192, 188, 1024)])[2:] == (256, 4)   # more buckets than SMs: full width


def test_tensors_of_tiny_buckets_get_no_items():
    awq_rect = _tensor(4096, 4096, 4096 * 4096 // 128, 256, mode=1)      # one bucket per 128-element group
    small = _tensor(128, 256, 67, 1024)                                  # under one step per sub-stream
    two_steps = _tensor(512, 1024, 171, 1024)                            # 3066 elements per bucket
    five_steps = _tensor(512, 1024, 100, 1024)                           # 5242 elements per bucket
    big = _tensor(4096, 4096, 111, 1024)
    rc, prefix, threads, chains = _plan([big, big, small, two_steps, five_steps])
    assert rc == 0 and (threads, chains) == (256, 4) and prefix == [0, 111, 222, 222, 222, 322]
    lib = _lib.load()
    arr = (_lib.BucketTensor * 1)(awq_rect)
    pre = (C.c_int64 * 2)()
    th, ch = C.c_int32(0), C.c_int32(0)
    assert lib.mps_bucket_batch_plan(arr, 1, pre, C.byref(th), C.byref(ch)) == 0 and pre[1] == 0


@pytest.mark.parametrize("k", [0, -1, 8193])
def test_sub_stream_count_is_checked(k):
    rc, _, _, _ = _plan([_tensor(4096, 4096, 32, k)])
    assert rc == _lib.MPS_ERR_INVALID
    assert b"invalid k" in _lib.load().mps_last_error()


def test_null_pointer_and_mode_mismatch_are_refused():
    t = _tensor(4096, 4096, 32, 1024)
    t.out = None
    assert _plan([t])[0] == _lib.MPS_ERR_INVALID
    by_scale = _tensor(4096, 4096, 462, 256, mode=2, group_size=0)      # by-scale groups need their size
    assert _plan([by_scale])[0] == _lib.MPS_ERR_INVALID


def test_decode_argument_check_takes_finer_sub_streams():
    """The Python-side check of the rectangular decode calls: up to MAX_SUBSTREAMS sub-streams per bucket."""
    import torch

    from mpserve_b200 import api

    B = 3
    i32 = lambda n: torch.zeros(n, dtype=torch.int32)
    args = lambda k: (i32(B), i32(B), i32(B + 1), i32(7), torch.zeros((B, k + 1), dtype=torch.uint32),
                      torch.zeros(B + 1, dtype=torch.int64), B)
    assert api._check_rect(*args(1024)) == 1024
    assert api._check_rect(*args(api.MAX_SUBSTREAMS)) == api.MAX_SUBSTREAMS
    with pytest.raises(ValueError, match="invalid k"):
        api._check_rect(*args(api.MAX_SUBSTREAMS + 1))


@pytest.mark.parametrize("n,m,k", [(64, 512, 2048), (9, 1000, 4096), (3, 5, 8192)])
def test_oracle_round_trip_with_the_limit_lifted(n, m, k):
    """The checker of the finer sub-streams: the oracle's layout code takes any sub-stream count once its
    argument check (the reference's, 1024) is lifted, and its decode restores the source."""
    import numpy as np
    import torch

    from mpserve_b200 import workloads as wl
    from oracle import oracle as orc

    c = wl.quantize_fp8(wl.random_weight(n, m, 5 + n, "normal"), "channel")
    bits = c.bf16.view(torch.uint16).numpy()
    with pytest.raises(ValueError, match="1024"):
        orc.build_fp8(bits, c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, k)
    orc.set_substream_limit(8192)
    try:
        art = orc.build_fp8(bits, c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, k)
    finally:
        orc.set_substream_limit(1024)
    assert art["bucket_thread_startbit_u32"].shape[1] == k + 1
    np.testing.assert_array_equal(orc.decode_fp8(c.fp8_u8.numpy(), art, n, m), bits)
