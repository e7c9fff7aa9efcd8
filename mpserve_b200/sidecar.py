"""The sidecar's on-disk contract and the decode of fused layers.

A compressed checkpoint carries, next to its FP8 weights, one safetensors shard with sixteen
``<module>.huff_*`` tensors per linear layer.  Key names, shapes and dtype casts are those of the
reference's offline compressor (scripts/compress_llm_fp8_huffman.py:284-306): safetensors has no
unsigned 16/32/64-bit types, so ``bitstream_u64`` is stored as int64, ``decode_syms_u16`` as int16
and ``bucket_thread_startbit_u32`` as int32, bit for bit; the loader side re-views them
(scripts/mpserve_vllm_fp8_huffman.py:457-472).  ``write_sidecar`` and ``read_sidecar`` interchange
with those scripts.

``FusedDecoder`` is what a serving plugin keeps per model: persistent BF16 buffers in the fused
``qkv`` / ``gate_up`` layout and one launch that decodes every shard straight into its row range, so
the per-forward ``torch.cat`` (plugin:526-543), the fresh allocation per call (decode_huffman.cu:699)
and the ``.item()`` synchronisation (plugin:419) of the reference's call site have no counterpart.
"""
from __future__ import annotations

from pathlib import Path
from typing import Mapping, Sequence

import torch

# artifact name -> dtype it is stored with (None: stored as is)
DECODE_KEYS: dict[str, torch.dtype | None] = {
    "bitstream_u64": torch.int64,
    "decode_syms_u16": torch.int16,
    "decode_lens_u8": None,
    "bucket_table_i32": None,
    "bucket_col_start_i32": None,
    "bucket_col_len_i32": None,
    "bucket_row_offsets_i32": None,
    "row_indices_i32": None,
    "bucket_thread_startbit_u32": torch.int32,
    "bucket_bit_base_i64": None,
}
_UNSIGNED = {"bitstream_u64": torch.uint64, "decode_syms_u16": torch.uint16, "bucket_thread_startbit_u32": torch.uint32}
# written by the compressor for other packing modes and left empty (compress:302-306)
_EXTRA_KEYS = {
    "huff_2d_nb1_i32": lambda: torch.tensor([1], dtype=torch.int32),
    "huff_attn_block_row_start_i32": lambda: torch.empty((0,), dtype=torch.int32),
    "huff_attn_block_row_len_i32": lambda: torch.empty((0,), dtype=torch.int32),
    "huff_attn_block_col_start_i32": lambda: torch.empty((0,), dtype=torch.int32),
    "huff_attn_block_col_len_i32": lambda: torch.empty((0,), dtype=torch.int32),
}


def scales_for_build(scales: torch.Tensor, n: int, m: int) -> torch.Tensor:
    """A checkpoint's ``weight_scale`` / ``weight_scale_inv`` tensor in the form the sidecar builder
    takes, by the rules of the reference's compressor (compress:96-140): fp32 scales are narrowed to
    fp16 and passed as their raw 16 bits (fp16 as is, bf16 as bf16); ``[n, 1]`` is squeezed, a scale
    per group of rows is repeated per row, and two-dimensional block scales ``[n/b0, m/b1]`` are
    collapsed to per-row scales by taking the first column block of every row block."""
    if scales.dtype == torch.float16:
        scales = scales.view(torch.uint16)
    elif scales.dtype == torch.float32:
        scales = scales.to(torch.float16).view(torch.uint16)
    elif scales.dtype not in (torch.uint16, torch.bfloat16):
        scales = scales.to(torch.bfloat16)
    scales = scales.contiguous()
    if scales.numel() == 1:
        return scales
    if scales.dim() == 2 and scales.size(0) == n and scales.size(1) == 1:
        scales = scales.squeeze(1)
    if scales.dim() == 1 and scales.numel() == n:
        return scales.contiguous()
    if scales.dim() == 1 and scales.numel() > 0 and n % scales.numel() == 0:
        return scales.repeat_interleave(n // scales.numel()).contiguous()
    if scales.dim() == 2 and scales.size(1) == 1 and scales.size(0) > 0 and n % scales.size(0) == 0:
        return scales.squeeze(1).repeat_interleave(n // scales.size(0)).contiguous()
    if scales.dim() == 2 and scales.size(0) > 0 and scales.size(1) > 0 and n % scales.size(0) == 0 and m % scales.size(1) == 0:
        return scales[:, 0].repeat_interleave(n // scales.size(0)).contiguous()
    return scales


def sidecar_tensors(module_prefix: str, fp8_u8: torch.Tensor, artifacts: Mapping[str, torch.Tensor],
                    store_fp8_u8: bool = True) -> dict[str, torch.Tensor]:
    """The sixteen tensors of one module as the compressor stores them (signed dtypes, CPU)."""
    out: dict[str, torch.Tensor] = {}
    out[f"{module_prefix}.huff_fp8_u8"] = (fp8_u8.detach().cpu().contiguous() if store_fp8_u8
                                           else torch.empty((0, 0), dtype=torch.uint8))
    for name, stored in DECODE_KEYS.items():
        t = artifacts[name].detach().cpu().contiguous()
        out[f"{module_prefix}.huff_{name}"] = t.view(stored) if stored is not None and t.dtype != stored else t
    for key, make in _EXTRA_KEYS.items():
        out[f"{module_prefix}.{key}"] = make()
    return out


def write_sidecar(path, modules: Mapping[str, tuple[torch.Tensor, Mapping[str, torch.Tensor]]]) -> None:
    """``modules``: module prefix (``model.layers.0.self_attn.q_proj``) -> (fp8 bytes ``[n, m]``, artifacts
    as ``huffman_build_fp8_decode_tables`` returns them)."""
    from safetensors.torch import save_file

    tensors: dict[str, torch.Tensor] = {}
    for prefix, (fp8_u8, art) in modules.items():
        tensors.update(sidecar_tensors(prefix, fp8_u8, art))
    save_file(tensors, str(path))


# ---- tensor parallelism -----------------------------------------------------------------------------
# A bitstream cannot be narrowed the way a weight loader narrows a checkpoint tensor to its rank's rows
# or columns, which is why the reference's plugin refuses tp_size > 1 (scripts/
# mpserve_vllm_fp8_huffman.py:165-168).  Here every rank gets a sidecar of its own, built from its
# shards (mpserve_b200/shard.py: column-parallel layers split rows, row-parallel layers split columns),
# and the file says which rank of which degree it is for, so that a loader running under another layout
# fails at load time instead of decoding the wrong rows.

def rank_sidecar_name(tp_rank: int, tp_size: int) -> str:
    return "model.huffman.safetensors" if tp_size == 1 else f"model.huffman.tp{tp_size}-rank{tp_rank:02d}.safetensors"


def write_rank_sidecar(directory, tp_rank: int, tp_size: int,
                       modules: Mapping[str, tuple[torch.Tensor, Mapping[str, torch.Tensor]]]) -> Path:
    """Write rank ``tp_rank``'s sidecar: ``modules`` as for ``write_sidecar``, built from this rank's shards."""
    from safetensors.torch import save_file

    if not 0 <= tp_rank < tp_size:
        raise ValueError(f"tp_rank {tp_rank} outside tensor-parallel degree {tp_size}")
    tensors: dict[str, torch.Tensor] = {}
    for prefix, (fp8_u8, art) in modules.items():
        tensors.update(sidecar_tensors(prefix, fp8_u8, art))
    path = Path(directory) / rank_sidecar_name(tp_rank, tp_size)
    save_file(tensors, str(path), metadata={"mpserve_tp_size": str(tp_size), "mpserve_tp_rank": str(tp_rank)})
    return path


def read_rank_sidecar(directory, tp_rank: int, tp_size: int, device=None) -> dict[str, dict[str, torch.Tensor]]:
    """This rank's modules (as ``read_sidecar`` returns them).  Raises when the directory has no sidecar
    for this layout or the file was written for another one."""
    from safetensors import safe_open

    path = Path(directory) / rank_sidecar_name(tp_rank, tp_size)
    if not path.exists():
        have = sorted(p.name for p in Path(directory).glob("model.huffman*.safetensors"))
        raise FileNotFoundError(f"no Huffman sidecar for rank {tp_rank} of {tp_size} in {directory} (found: {have}); "
                                "sidecars are built per tensor-parallel shard and cannot be re-split")
    with safe_open(str(path), framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
    said = (int(meta.get("mpserve_tp_size", "1")), int(meta.get("mpserve_tp_rank", "0")))
    if said != (tp_size, tp_rank):
        raise ValueError(f"{path.name} was written for rank {said[1]} of {said[0]}, not rank {tp_rank} of {tp_size}")
    return read_sidecar(path, device=device)


def as_decode_inputs(stored: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Re-view one module's stored tensors (keys without the ``huff_`` prefix) for the decode entry."""
    out = {}
    for name in DECODE_KEYS:
        t = stored[name]
        want = _UNSIGNED.get(name)
        if want is not None and t.dtype != want:
            if t.element_size() != torch.empty((), dtype=want).element_size():
                raise ValueError(f"huff_{name}: stored dtype {t.dtype} cannot be re-viewed as {want}")
            t = t.view(want)
        out[name] = t.contiguous()
    return out


def read_sidecar(path, device=None) -> dict[str, dict[str, torch.Tensor]]:
    """module prefix -> {"fp8_u8": [n, m] uint8, <the ten decode artifacts, unsigned dtypes restored>}."""
    from safetensors import safe_open

    modules: dict[str, dict[str, torch.Tensor]] = {}
    with safe_open(str(Path(path)), framework="pt", device="cpu") as f:
        for key in f.keys():
            prefix, sep, leaf = key.rpartition(".huff_")
            if not sep:
                continue
            modules.setdefault(prefix, {})[leaf] = f.get_tensor(key)
    result = {}
    for prefix, stored in modules.items():
        missing = [k for k in ("fp8_u8", *DECODE_KEYS) if k not in stored]
        if missing:
            raise KeyError(f"{prefix}: sidecar lacks {missing}")
        entry = as_decode_inputs(stored)
        entry["fp8_u8"] = stored["fp8_u8"].contiguous()
        if device is not None:
            entry = {k: v.to(device) for k, v in entry.items()}
        result[prefix] = entry
    return result


class FusedDecoder:
    """Decode groups of shards into persistent fused weights with one launch per call.

    ``groups``: for every fused weight a list of shards in row order; a shard is ``(fp8_u8 [n_i, m],
    artifacts)`` with all tensors on the device.  ``weights[g]`` is the ``[sum n_i, m]`` BF16 tensor of
    group ``g``; it is allocated once and reused by every ``decode()``, which is asynchronous on the
    current stream and involves no host synchronisation.
    """

    def __init__(self, groups: Sequence[Sequence[tuple[torch.Tensor, Mapping[str, torch.Tensor]]]]):
        from . import api

        if not groups or not all(len(g) for g in groups):
            raise ValueError("every fused weight needs at least one shard")
        device = groups[0][0][0].device
        self.weights: list[torch.Tensor] = []
        entries = []
        for shards in groups:
            m = int(shards[0][0].shape[1])
            if any(int(ctx.shape[1]) != m for ctx, _ in shards):
                raise ValueError("the shards of a fused weight must have the same number of columns")
            rows = [int(ctx.shape[0]) for ctx, _ in shards]
            w = torch.empty((sum(rows), m), dtype=torch.bfloat16, device=device)
            self.weights.append(w)
            r0 = 0
            for (ctx, art), n in zip(shards, rows):
                entries.append((ctx, art, w[r0:r0 + n]))   # a row range of a row-major tensor is contiguous
                r0 += n
        self.plan = api.BucketDecodePlan(entries, mode=0)

    def decode(self) -> list[torch.Tensor]:
        self.plan.decode()
        return self.weights
