"""The reference's UNMODIFIED vLLM plugin, driven end to end on the host.

Runs only where the reference tree is mounted (``MPSERVE_REFERENCE_ROOT``, else a ``reference`` directory beside this repository);
elsewhere it skips.  ``scripts/mpserve_vllm_fp8_huffman.py`` is imported as it is; its
``create_weights`` registers the parameters, its weight loaders take the tensors of the sidecar
fixture (written by the reference's own compressor, see tests/golden/make_sidecar_fixture.py), and its
``apply`` -- ``_decode_weight_for_layer`` -> ``_decode_one`` -> ``MPServe_cuda.huffman_decode_fp8`` ->
``torch.matmul`` -- runs on CPU tensors that merely claim to be CUDA tensors.

``MPServe_cuda`` is a test double here: it applies this library's own argument checks
(``api.validate_decode_fp8``, device test left out) to what the plugin passes and decodes with the CPU
oracle, because there is no GPU on this machine.  What the test pins is the host-side contract: names,
positional order, dtypes after the plugin's re-views, shard handling, the returned dtype and shape.
The same call sequence on the real kernels is tests/test_sidecar_contract_gpu.py.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import pytest
import torch

from tests._util import GOLDEN_DIR

REF_ROOT = Path(os.environ.get("MPSERVE_REFERENCE_ROOT") or Path(__file__).resolve().parents[2] / "reference")
PLUGIN = REF_ROOT / "scripts" / "mpserve_vllm_fp8_huffman.py"
FIXTURE = GOLDEN_DIR / "tiny_llama_sidecar"
PREFIX = "model.layers.0"

pytestmark = pytest.mark.skipif(not PLUGIN.exists(), reason="reference tree not mounted")

DECODE_LEAVES = ("fp8_u8", "bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32",
                 "bucket_col_start_i32", "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32",
                 "bucket_thread_startbit_u32", "bucket_bit_base_i64")


class ClaimsCuda(torch.Tensor):
    """A CPU tensor whose ``is_cuda`` says True: gets an activation past plugin:395."""

    is_cuda = property(lambda self: True)


@pytest.fixture(scope="module")
def plugin():
    from mpserve_b200 import api
    from oracle import oracle as orc

    pytest.importorskip("vllm")
    double = types.ModuleType("MPServe_cuda")
    double.calls = []

    def huffman_decode_fp8(*args, **kwargs):
        assert not kwargs, "the plugin calls positionally (plugin:474-489)"
        assert len(args) == 14
        n, m, max_len, B, k, tensors = api.validate_decode_fp8(*args, require_cuda=False)
        names = ("fp8", "bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_col_start_i32",
                 "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32", "bucket_thread_startbit_u32",
                 "bucket_bit_base_i64")
        art = {nm: t.detach().numpy() for nm, t in zip(names, tensors)}
        double.calls.append({"n": n, "m": m, "max_len": max_len, "k": k, "dtypes": [t.dtype for t in tensors]})
        bits = orc.decode_fp8(art.pop("fp8"), art, n, m)
        return torch.from_numpy(bits).view(torch.bfloat16)

    double.huffman_decode_fp8 = huffman_decode_fp8
    saved = sys.modules.get("MPServe_cuda")
    saved_env = os.environ.get("MPSERVE_ENABLE_FP8_HUFFMAN")
    sys.modules["MPServe_cuda"] = double
    os.environ["MPSERVE_ENABLE_FP8_HUFFMAN"] = "1"
    spec = importlib.util.spec_from_file_location("mpserve_vllm_fp8_huffman", str(PLUGIN))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mpserve_vllm_fp8_huffman"] = mod
    # one process, no tensor parallelism: what vLLM's parameter class would read from an initialised
    # tensor-parallel group of size 1 (no such group exists outside an engine)
    import vllm.model_executor.parameter as vparam

    saved_tp = (vparam.get_tensor_model_parallel_rank, vparam.get_tensor_model_parallel_world_size)
    vparam.get_tensor_model_parallel_rank = lambda: 0
    vparam.get_tensor_model_parallel_world_size = lambda: 1
    try:
        spec.loader.exec_module(mod)
        yield mod, double
    finally:
        vparam.get_tensor_model_parallel_rank, vparam.get_tensor_model_parallel_world_size = saved_tp
        sys.modules.pop("mpserve_vllm_fp8_huffman", None)
        if saved is not None:
            sys.modules["MPServe_cuda"] = saved
        else:
            sys.modules.pop("MPServe_cuda", None)
        if saved_env is None:
            os.environ.pop("MPSERVE_ENABLE_FP8_HUFFMAN", None)
        else:
            os.environ["MPSERVE_ENABLE_FP8_HUFFMAN"] = saved_env


@pytest.fixture(scope="module")
def fixture_tensors():
    from safetensors.torch import load_file

    return load_file(str(FIXTURE / "huffman_fp8.safetensors")), load_file(str(FIXTURE / "expected_bf16.safetensors"))


def _make_layer(mod, name, in_features, out_sizes):
    layer = torch.nn.Module()
    layer.prefix = name
    method = mod.FP8HuffmanLinearMethod(mod.FP8HuffmanParams(max_len=7))
    method.create_weights(layer, in_features, list(out_sizes), in_features, sum(out_sizes), torch.bfloat16)
    return layer, method


def _load(layer, sidecar, module, shard_id=None):
    """What vLLM's loader does with every checkpoint key of a module: param.weight_loader(param, tensor[, shard_id])."""
    unregistered = []
    for key, tensor in sidecar.items():
        prefix, _, leaf = key.rpartition(".")
        if prefix != module:
            continue
        param = getattr(layer, leaf, None)
        if param is None:
            unregistered.append(leaf)
            continue
        if shard_id is None:
            param.weight_loader(param, tensor)
        else:
            param.weight_loader(param, tensor, shard_id)
    return sorted(unregistered)


def test_single_layers_through_the_plugin(plugin, fixture_tensors):
    mod, double = plugin
    sidecar, expected = fixture_tensors
    for name in ("self_attn.o_proj", "mlp.down_proj"):
        w = expected[f"{PREFIX}.{name}.weight"]
        n, m = w.shape
        layer, method = _make_layer(mod, f"{PREFIX}.{name}", m, [n])
        unregistered = _load(layer, sidecar, f"{PREFIX}.{name}")
        # three keys the reference's compressor writes (compress:302-306) have no parameter in its own
        # plugin; a stock vLLM loader would raise KeyError on them.  Recorded, not patched.
        assert unregistered == ["huff_2d_nb1_i32", "huff_attn_block_col_len_i32", "huff_attn_block_col_start_i32"]
        method.process_weights_after_loading(layer)
        x = (torch.randn(3, m, generator=torch.Generator().manual_seed(1)) * 0.1).to(torch.bfloat16)
        double.calls.clear()
        out = method.apply(layer, x.as_subclass(ClaimsCuda))
        assert len(double.calls) == 1
        call = double.calls[0]
        assert (call["n"], call["m"], call["max_len"], call["k"]) == (n, m, 7, 1024)
        # the plugin re-views the signed storage dtypes before the call (plugin:457-472)
        assert call["dtypes"][1] == torch.uint64 and call["dtypes"][2] == torch.uint16 and call["dtypes"][9] == torch.uint32
        assert torch.equal(torch.Tensor(out), torch.matmul(x, w.t()))


@pytest.mark.parametrize("fused,parts,ids", [
    ("self_attn.qkv_proj", ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), ("q", "k", "v")),
    ("mlp.gate_up_proj", ("mlp.gate_proj", "mlp.up_proj"), (0, 1)),
])
def test_fused_layers_through_the_plugin(plugin, fixture_tensors, fused, parts, ids):
    mod, double = plugin
    sidecar, expected = fixture_tensors
    ws = [expected[f"{PREFIX}.{p}.weight"] for p in parts]
    m = ws[0].shape[1]
    layer, method = _make_layer(mod, f"{PREFIX}.{fused}", m, [w.shape[0] for w in ws])
    for p, sid in zip(parts, ids):
        _load(layer, sidecar, f"{PREFIX}.{p}", shard_id=sid)
    method.process_weights_after_loading(layer)
    x = (torch.randn(2, 5, m, generator=torch.Generator().manual_seed(2)) * 0.1).to(torch.bfloat16)
    double.calls.clear()
    out = method.apply(layer, x.as_subclass(ClaimsCuda))
    assert [c["n"] for c in double.calls] == [w.shape[0] for w in ws]     # one decode per shard, in shard order
    want = torch.matmul(x.reshape(-1, m), torch.cat(ws, dim=0).t()).reshape(2, 5, -1)
    assert torch.equal(torch.Tensor(out), want)


def test_the_plugin_refuses_tensor_parallelism(plugin):
    """plugin:165-168 -- recorded as a reference limitation; per-shard sidecars are this library's answer."""
    mod, _ = plugin
    layer = torch.nn.Module()
    layer.tp_size, layer.tp_rank = 2, 0
    method = mod.FP8HuffmanLinearMethod(mod.FP8HuffmanParams(max_len=7))
    with pytest.raises(NotImplementedError):
        method.create_weights(layer, 128, [128], 128, 128, torch.bfloat16)


def test_fixture_decodes_with_the_oracle(fixture_tensors):
    """The reference compressor's own output, read back through this library's sidecar reader."""
    from mpserve_b200 import sidecar as sc
    from oracle import oracle as orc

    _, expected = fixture_tensors
    modules = sc.read_sidecar(FIXTURE / "huffman_fp8.safetensors")
    assert sorted(modules) == sorted(k[: -len(".weight")] for k in expected)
    for prefix, entry in modules.items():
        w = expected[prefix + ".weight"]
        n, m = w.shape
        art = {k: v.numpy() for k, v in entry.items() if k != "fp8_u8"}
        bits = orc.decode_fp8(entry["fp8_u8"].numpy(), art, n, m)
        assert torch.equal(torch.from_numpy(bits).view(torch.bfloat16), w), prefix
