"""Sidecars with more than the reference's 1024 sub-streams per bucket (api.build_fp8_fine_substreams):
the builder byte for byte against the CPU oracle with the reference's argument check lifted (the layout
code it restates, build_huffman.cu:811-918, does not depend on the number), the decoders bit for bit
against the oracle's decode and the source tensor.  The reference itself refuses such sidecars
(build_huffman.cu:313, decode_huffman.cu:695), so there is no golden vector for them."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from mpserve_b200 import api, util
from mpserve_b200 import workloads as wl
from oracle import oracle as orc
from tests.test_configs_gpu import FP8_KEYS
from tests.test_encode_gpu import _same

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


@pytest.fixture()
def lifted_oracle():
    orc.set_substream_limit(api.MAX_SUBSTREAMS)
    yield
    orc.set_substream_limit(1024)


CASES = [
    (256, 2048, "normal", "tensor", 7, 2048),
    (512, 1024, "normal", "tensor", 7, 4096),
    (300, 1000, "normal", "channel", 7, 2048),       # ragged widths, buckets with fewer elements than sub-streams
    (129, 4096, "student_t", "channel", 7, 4096),
    (256, 512, "student_t", "block", 7, 1536),       # not a power of two
    (512, 512, "normal", "tensor", 5, 8192),         # many ESC contexts at a short max_len
    (3, 5, "normal", "tensor", 7, 8192),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c)))
def test_builder_and_decoder_against_the_oracle(dev, lifted_oracle, case):
    import MPServe_cuda

    n, m, dist, mode, L, k = case
    c = wl.quantize_fp8(wl.random_weight(n, m, 700 + n + m, dist), mode)
    want = orc.build_fp8(c.bf16.view(torch.uint16).numpy(), c.fp8_u8.numpy(), c.scales_u16.numpy(), L, k)
    got = api.build_fp8_fine_substreams(c.bf16, c.fp8_u8, c.scales_u16, max_len=L, substreams=k)
    _same(got, want, str(case))
    assert got["bucket_thread_startbit_u32"].shape[1] == k + 1
    if L != 7:
        return   # the FP8 decoder reads 7-bit tables only, like the reference's
    fp8 = c.fp8_u8.to(dev)
    out = MPServe_cuda.huffman_decode_fp8(fp8, *[got[key].to(dev) for key in FP8_KEYS], n, m, 7)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu().view(torch.uint16), c.bf16.view(torch.uint16))
    ref = orc.decode_fp8(c.fp8_u8.numpy(), want, n, m)
    np.testing.assert_array_equal(util.bf16_bits(out), ref)
    assert api.decode_timed_out(dev) is False


@pytest.mark.parametrize("k", [2048, 4096, 8192])
def test_lone_weight_with_a_per_tensor_scale(dev, k):
    """The case finer sub-streams are for: 4096 x 4096, 32 buckets.  Through the per-tensor call and through
    a plan, with the launch shapes the library picks for them."""
    import MPServe_cuda

    n = m = 4096
    c = wl.quantize_fp8(wl.random_weight(n, m, 7, "normal", device=dev), "tensor")
    art = api.build_fp8_fine_substreams(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, substreams=k)
    out = MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *[art[key] for key in FP8_KEYS], n, m, 7)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16))
    plan = api.BucketDecodePlan([(c.fp8_u8, {key: art[key] for key in FP8_KEYS}, None)], mode=0)
    assert plan.total_items == 32 * -(-k // (plan.threads * plan.chains))
    got = plan.decode()[0]
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.uint16), c.bf16.view(torch.uint16))
    assert torch.equal(api.checksum_u16(got).cpu(), api.checksum_u16(c.bf16).cpu())
    assert api.decode_timed_out(dev) is False


def test_per_channel_weight_with_fine_substreams(dev):
    """Rows that hold a whole number of steps only in part: 14336 columns under 4096 sub-streams."""
    import MPServe_cuda

    n, m = 512, 14336
    c = wl.quantize_fp8(wl.random_weight(n, m, 21, "normal", device=dev), "channel")
    art = api.build_fp8_fine_substreams(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, substreams=4096)
    out = MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *[art[key] for key in FP8_KEYS], n, m, 7)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16))
    assert api.decode_timed_out(dev) is False
