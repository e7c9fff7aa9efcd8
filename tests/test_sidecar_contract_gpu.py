"""The sidecar's on-disk contract and the plugin's call sequence on the real kernels.

The fixture under tests/golden/tiny_llama_sidecar was written by the reference's own compressor
script and encoder (tests/golden/make_sidecar_fixture.py); the reference tree is not needed to run
these tests.  They do what scripts/mpserve_vllm_fp8_huffman.py does with such a shard -- load the
signed-dtype tensors, re-view them (plugin:457-472), call ``MPServe_cuda.huffman_decode_fp8``
positionally per shard (plugin:474-489), ``torch.cat`` fused layers (plugin:526-543), ``torch.matmul``
(plugin:657-661) -- and check every weight bit for bit against the BF16 checkpoint it was made from.
tests/test_reference_plugin_cpu.py drives the unmodified plugin itself over the same fixture on the host.
"""
from __future__ import annotations

import pytest
import torch

from tests._util import GOLDEN_DIR

pytestmark = pytest.mark.gpu

FIXTURE = GOLDEN_DIR / "tiny_llama_sidecar"
PREFIX = "model.layers.0"
ORDER = ("fp8_u8", "bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_col_start_i32",
         "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32", "bucket_thread_startbit_u32",
         "bucket_bit_base_i64")


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def stored():
    from safetensors.torch import load_file

    return load_file(str(FIXTURE / "huffman_fp8.safetensors")), load_file(str(FIXTURE / "expected_bf16.safetensors"))


def _plugin_decode_one(module_tensors: dict, dev, max_len=7):
    """The body of the plugin's _decode_one, restated: re-view, make contiguous, positional call."""
    import MPServe_cuda

    t = {k: v.to(dev) for k, v in module_tensors.items()}
    fp8 = t["fp8_u8"]
    assert fp8.dim() == 2
    n, m = int(fp8.shape[0]), int(fp8.shape[1])
    bs = t["bitstream_u64"]
    assert bs.dtype == torch.int64            # as the compressor stored it
    bs = bs.view(torch.uint64)
    syms = t["decode_syms_u16"]
    assert syms.dtype == torch.int16
    syms = syms.view(torch.uint16)
    tsb = t["bucket_thread_startbit_u32"]
    assert tsb.dtype == torch.int32
    tsb = tsb.view(torch.uint32)
    return MPServe_cuda.huffman_decode_fp8(
        fp8.contiguous(), bs.contiguous(), syms.contiguous(), t["decode_lens_u8"].contiguous(),
        t["bucket_table_i32"].contiguous(), t["bucket_col_start_i32"].contiguous(), t["bucket_col_len_i32"].contiguous(),
        t["bucket_row_offsets_i32"].contiguous(), t["row_indices_i32"].contiguous(), tsb.contiguous(),
        t["bucket_bit_base_i64"].contiguous(), n, m, max_len)


def _module(sidecar: dict, name: str) -> dict:
    return {leaf: sidecar[f"{PREFIX}.{name}.huff_{leaf}"] for leaf in ORDER}


@pytest.mark.parametrize("name", ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                                  "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"])
def test_every_module_of_the_reference_sidecar_decodes(stored, dev, name):
    sidecar, expected = stored
    w = _plugin_decode_one(_module(sidecar, name), dev)
    want = expected[f"{PREFIX}.{name}.weight"]
    assert w.dtype == torch.bfloat16 and tuple(w.shape) == tuple(want.shape)
    assert torch.equal(w.cpu().view(torch.uint16), want.view(torch.uint16))


@pytest.mark.parametrize("parts", [("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"),
                                   ("mlp.gate_proj", "mlp.up_proj")])
def test_fused_layer_as_the_plugin_builds_it(stored, dev, parts):
    sidecar, expected = stored
    w = torch.cat([_plugin_decode_one(_module(sidecar, p), dev) for p in parts], dim=0)      # plugin:526-543
    want = torch.cat([expected[f"{PREFIX}.{p}.weight"] for p in parts], dim=0)
    assert torch.equal(w.cpu().view(torch.uint16), want.view(torch.uint16))
    x = (torch.randn(5, w.shape[1], generator=torch.Generator().manual_seed(3)) * 0.1).to(torch.bfloat16).to(dev)
    assert torch.equal(torch.matmul(x, w.t()), torch.matmul(x, want.to(dev).t()))             # plugin:657-661


def test_fused_decoder_equals_cat_of_shard_decodes(dev):
    """Decode straight into the fused qkv / gate_up layout: no torch.cat, outputs kept across calls."""
    from mpserve_b200 import sidecar as sc

    modules = sc.read_sidecar(FIXTURE / "huffman_fp8.safetensors", device=dev)
    from safetensors.torch import load_file

    expected = load_file(str(FIXTURE / "expected_bf16.safetensors"))
    groups_names = [("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), ("self_attn.o_proj",),
                    ("mlp.gate_proj", "mlp.up_proj"), ("mlp.down_proj",)]
    groups = []
    for names in groups_names:
        shards = []
        for nm in names:
            e = modules[f"{PREFIX}.{nm}"]
            shards.append((e["fp8_u8"], {k: v for k, v in e.items() if k != "fp8_u8"}))
        groups.append(shards)
    fused = sc.FusedDecoder(groups)
    ptrs = [w.data_ptr() for w in fused.weights]
    for _ in range(2):
        for w in fused.weights:
            w.zero_()
        out = fused.decode()
        torch.cuda.synchronize()
        assert [w.data_ptr() for w in out] == ptrs
        for names, w in zip(groups_names, out):
            want = torch.cat([expected[f"{PREFIX}.{nm}.weight"] for nm in names], dim=0)
            assert torch.equal(w.cpu().view(torch.uint16), want.view(torch.uint16)), names


def test_decode_into_a_row_range(stored, dev):
    """``out=``: the per-tensor entry writing one shard into its rows of a larger buffer."""
    import MPServe_cuda
    from mpserve_b200 import sidecar as sc

    sidecar, expected = stored
    e = sc.as_decode_inputs({leaf: sidecar[f"{PREFIX}.self_attn.k_proj.huff_{leaf}"].to(dev) for leaf in ORDER[1:]})
    fp8 = sidecar[f"{PREFIX}.self_attn.k_proj.huff_fp8_u8"].to(dev)
    n, m = fp8.shape
    big = torch.zeros((3 * n, m), dtype=torch.bfloat16, device=dev)
    ret = MPServe_cuda.huffman_decode_fp8(fp8, *[e[k] for k in ORDER[1:]], n, m, 7, out=big[n:2 * n])
    torch.cuda.synchronize()
    assert ret.data_ptr() == big[n:2 * n].data_ptr()
    want = expected[f"{PREFIX}.self_attn.k_proj.weight"]
    assert torch.equal(big[n:2 * n].cpu().view(torch.uint16), want.view(torch.uint16))
    assert not big[:n].any() and not big[2 * n:].any()
    with pytest.raises(ValueError):
        MPServe_cuda.huffman_decode_fp8(fp8, *[e[k] for k in ORDER[1:]], n, m, 7, out=big[:, : m // 2])


def test_own_builder_and_writer_reproduce_the_reference_shard(stored, dev, tmp_path):
    """GPU builder + write_sidecar on the fixture's inputs == the shard the reference's compressor wrote,
    key for key and byte for byte (names, dtypes after the signed casts, shapes, contents)."""
    import MPServe_cuda
    from mpserve_b200 import sidecar as sc
    from safetensors.torch import load_file
    from tests.golden import make_sidecar_fixture as mk

    sidecar, expected = stored
    mk.make_checkpoints(tmp_path / "bf16", tmp_path / "fp8")
    fp8_ckpt = load_file(str(tmp_path / "fp8" / "model.safetensors"))
    modules = {}
    for name, (n, m, _layout) in mk.MODULES.items():
        key = f"{PREFIX}.{name}"
        scales = fp8_ckpt.get(key + ".weight_scale_inv", fp8_ckpt.get(key + ".weight_scale"))
        fp8_u8 = fp8_ckpt[key + ".weight"].view(torch.uint8).reshape(n, m).contiguous()
        art = MPServe_cuda.huffman_build_fp8_decode_tables(expected[key + ".weight"].to(dev), fp8_u8.to(dev),
                                                           sc.scales_for_build(scales, n, m).to(dev), max_len=7,
                                                           threads_per_block=1024)
        modules[key] = (fp8_u8, art)
    sc.write_sidecar(tmp_path / "mine.safetensors", modules)
    mine = load_file(str(tmp_path / "mine.safetensors"))
    assert sorted(mine) == sorted(sidecar)
    for k, ref in sidecar.items():
        assert mine[k].dtype == ref.dtype and tuple(mine[k].shape) == tuple(ref.shape), k
        assert torch.equal(mine[k], ref), k
