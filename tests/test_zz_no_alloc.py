"""The non-allocating FP8 decode entry point against the regular one.

Some callers of this library cannot allocate device memory at call time -- a plugin living inside
another framework's memory pool, a process with a fixed memory budget that forbids cudaMalloc after
start-up, a latency-critical loop -- so they cannot hand the decoder its queue workspace.
``mps_decode_fp8_noalloc`` keeps that workspace inside the library image instead.  This test calls
it through the C ABI, twice in a row (the second call finds whatever the first left in the shared
scratch), and wants bit-identical output to ``mps_decode_fp8`` both times.

Collected last on purpose: a failure here cannot hide the results of the other GPU tests.
"""
import numpy as np
import pytest
import torch

from mpserve_b200 import _lib, util
from mpserve_b200 import workloads as wl
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _args(ctx, d, n, m, out):
    return (ctx.data_ptr(), d["bitstream_u64"].data_ptr(), d["bitstream_u64"].numel(), d["decode_syms_u16"].data_ptr(),
            d["decode_lens_u8"].data_ptr(), d["decode_syms_u16"].size(0), d["bucket_table_i32"].data_ptr(),
            d["bucket_col_start_i32"].data_ptr(), d["bucket_col_len_i32"].data_ptr(),
            d["bucket_row_offsets_i32"].data_ptr(), d["row_indices_i32"].data_ptr(), d["row_indices_i32"].numel(),
            d["bucket_thread_startbit_u32"].data_ptr(), d["bucket_bit_base_i64"].data_ptr(),
            d["bucket_table_i32"].size(0), d["bucket_thread_startbit_u32"].size(1) - 1, n, m, 7, out.data_ptr())


@pytest.mark.parametrize("shape,mode", [((384, 2048), "channel"), ((100, 250), "tensor")])
def test_noalloc_matches_regular_entry_twice(shape, mode):
    assert torch.cuda.is_available()
    lib = _lib.load()
    dev = torch.device("cuda:0")
    n, m = shape
    c = wl.quantize_fp8(wl.random_weight(n, m, 4242, "normal"), mode)
    bits = c.bf16.view(torch.uint16).numpy()
    art = orc.build_fp8(bits, c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
    d = util.artifacts_to_device(art, dev)
    ctx = c.fp8_u8.to(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    ref = torch.zeros((n, m), dtype=torch.bfloat16, device=dev)
    ws = torch.zeros(int(lib.mps_workspace_bytes()) // 4, dtype=torch.int32, device=dev)
    _lib.check(lib.mps_decode_fp8(*_args(ctx, d, n, m, ref), ws.data_ptr(), ws.numel() * 4, stream))
    torch.cuda.synchronize()
    want = util.bf16_bits(ref)
    np.testing.assert_array_equal(want, bits)

    for call in range(2):
        out = torch.zeros((n, m), dtype=torch.bfloat16, device=dev)
        _lib.check(lib.mps_decode_fp8_noalloc(*_args(ctx, d, n, m, out), stream))
        torch.cuda.synchronize()
        np.testing.assert_array_equal(util.bf16_bits(out), want, err_msg=f"call {call}")
    # a caller of this entry has no workspace to ask about; the status call takes NULL for the library's own
    from mpserve_b200 import api

    assert api.noalloc_decode_timed_out(dev) is False


def test_noalloc_rejects_oversized_input():
    lib = _lib.load()
    dev = torch.device("cuda:0")
    z = torch.zeros(16, dtype=torch.int64, device=dev)
    p = z.data_ptr()
    too_many = (1 << 20) + 1
    rc = lib.mps_decode_fp8_noalloc(p, p, 1, p, p, 1, p, p, p, p, p, 1, p, p, too_many, 1024, 4, 4, 7, p,
                                    torch.cuda.current_stream(dev).cuda_stream)
    assert rc == _lib.MPS_ERR_INVALID
    assert b"maximum" in lib.mps_last_error()
