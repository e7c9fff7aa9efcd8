"""The reference's own CUDA decoder as a second checker (gate: new decode == reference kernel's decode).

``oracle/build_ref_decode.sh`` compiles kernel/decode_huffman.cu, unmodified, for sm_100a; the built
module travels with the repository, the reference tree is not needed to run these tests.  The shipped
kernel is only correct on part of the input space (no ESC tables, no bitstream of 3072..10240 words,
no bucket narrower than its sub-stream count); ``oracle/ref_decoder.py`` refuses everything else on the
host, and the cases here were chosen from reading the kernel: every index it forms stays inside the
tensors it is given, and it has no wait.
"""
from __future__ import annotations

import pytest
import torch

from mpserve_b200 import workloads as wl
from oracle import ref_decoder as ref

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref.available(), reason="oracle/_ref holds no reference decoder")]

KEYS = ref.ORDER


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


@pytest.mark.parametrize("n,m,mode,k", [(4096, 4096, "tensor", 1024), (4096, 4096, "tensor", 256),
                                        (14336, 4096, "channel", 1024)],
                         ids=["config1-k1024", "config1-k256", "gate_up-per-channel"])
def test_same_output_as_the_reference_kernel(dev, n, m, mode, k):
    import MPServe_cuda

    c = wl.quantize_fp8(wl.random_weight(n, m, 77, "normal", device=dev), mode)
    art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=k)
    assert ref.refusal(art, n, m) is None
    mine = MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *[art[x] for x in KEYS], n, m, 7)
    torch.cuda.synchronize()
    theirs = ref.decode_fp8(c.fp8_u8, art, n, m)
    torch.cuda.synchronize()
    assert theirs.dtype == torch.bfloat16 and tuple(theirs.shape) == (n, m)
    assert torch.equal(mine.view(torch.uint16), theirs.view(torch.uint16))
    assert torch.equal(mine.view(torch.uint16), c.bf16.view(torch.uint16))


def test_unsafe_sidecars_are_refused_on_the_host(dev):
    import MPServe_cuda

    # 128 x 1024 at about 4 bits per element: a bitstream of about 8192 words, inside the range the kernel overruns on
    c = wl.quantize_fp8(wl.random_weight(128, 1024, 3, "normal", device=dev), "tensor")
    art = dict(MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=1024))
    words = int(art["bitstream_u64"].numel())
    assert 3072 < words < 10240 and "overrun" in ref.refusal(art, 128, 1024)
    with pytest.raises(ValueError, match="not given to the reference kernel"):
        ref.decode_fp8(c.fp8_u8, art, 128, 1024)
    esc = dict(art)
    esc["decode_lens_u8"] = art["decode_lens_u8"].clone()
    esc["decode_lens_u8"][0, 0] |= 0x08
    esc["bitstream_u64"] = torch.zeros(20000, dtype=torch.uint64, device=dev)
    assert "ESC" in ref.refusal(esc, 128, 1024)
