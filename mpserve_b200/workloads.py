"""Seeded synthetic checkpoints with the shapes, value distributions and quantisers the benchmark
configurations name.  No real checkpoint or dataset is involved: weights are random-init
(N(0, 0.02) or Student-t(4) x 0.02), quantised here to FP8-E4M3 or AWQ-style INT4.

The scale dtype handling follows the offline compressor of the reference
(scripts/compress_llm_fp8_huffman.py:96-104): fp32 scales are narrowed to fp16 and handed to the
encoder as their raw 16 bits, which is all the codec ever uses of a scale (a context key).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator

import torch

FP8_MAX = 448.0

# (name, n, m) of the linears of one decoder layer; scripts/mpserve_vllm_fp8_huffman.py:174-183
# decodes q/k/v and gate/up as separate shards, so they stay separate tensors here.
LLAMA3_8B = dict(layers=32, hidden=4096, inter=14336, q_heads=32, kv_heads=8, head_dim=128, vocab=128256)
LLAMA3_70B = dict(layers=80, hidden=8192, inter=28672, q_heads=64, kv_heads=8, head_dim=128, vocab=128256)


def layer_linears(cfg: dict) -> list[tuple[str, int, int]]:
    h, i = cfg["hidden"], cfg["inter"]
    q, kv = cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
    return [
        ("self_attn.q_proj", q, h), ("self_attn.k_proj", kv, h), ("self_attn.v_proj", kv, h),
        ("self_attn.o_proj", h, q), ("mlp.gate_proj", i, h), ("mlp.up_proj", i, h), ("mlp.down_proj", h, i),
    ]


def tp_shard_shape(name: str, n: int, m: int, tp: int) -> tuple[int, int]:
    """Column-parallel linears (q,k,v,gate,up) split rows; row-parallel (o,down) split columns."""
    if name.endswith(("o_proj", "down_proj")):
        return n, m // tp
    return n // tp, m


def random_weight(n: int, m: int, seed: int, dist: str = "normal", device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    if dist == "normal":
        w = torch.randn((n, m), generator=g, device=device, dtype=torch.float32) * 0.02
    elif dist == "student_t":
        # t(nu=4) = z / sqrt(chi2_4 / 4)
        z = torch.randn((n, m), generator=g, device=device, dtype=torch.float32)
        c = torch.randn((4, n, m), generator=g, device=device, dtype=torch.float32).square_().sum(0)
        w = z / torch.sqrt(c / 4.0) * 0.02
    else:
        raise ValueError(f"unknown dist {dist!r}")
    return w.to(torch.bfloat16)


@dataclass
class Fp8Case:
    bf16: torch.Tensor        # [n,m] bfloat16
    fp8_u8: torch.Tensor      # [n,m] uint8 (E4M3 bit patterns)
    scales_u16: torch.Tensor  # uint16 raw fp16 bits: [1], [n] or [n/bs0, m/bs1]


def quantize_fp8(w: torch.Tensor, scale_mode: str = "channel", block: tuple[int, int] = (128, 128)) -> Fp8Case:
    """FP8-E4M3 with scale = amax/448 per tensor, per output channel (row) or per 2-D block."""
    wf = w.float()
    n, m = wf.shape
    if scale_mode == "tensor":
        scale = (wf.abs().amax() / FP8_MAX).clamp_min(1e-12).reshape(1)
        q = wf / scale
    elif scale_mode == "channel":
        scale = (wf.abs().amax(dim=1) / FP8_MAX).clamp_min(1e-12)
        q = wf / scale[:, None]
    elif scale_mode == "block":
        b0, b1 = block
        v = wf.reshape(n // b0, b0, m // b1, b1)
        scale = (v.abs().amax(dim=(1, 3)) / FP8_MAX).clamp_min(1e-12)
        q = (v / scale[:, None, :, None]).reshape(n, m)
    else:
        raise ValueError(f"unknown scale_mode {scale_mode!r}")
    fp8 = q.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    scales_u16 = scale.to(torch.float16).view(torch.uint16).contiguous()
    return Fp8Case(w.contiguous(), fp8, scales_u16)


@dataclass
class AwqCase:
    bf16: torch.Tensor        # [n,m] bfloat16
    int4_u8: torch.Tensor     # [n,m] uint8, one INT4 code (0..15) per byte
    scales_u16: torch.Tensor  # [n, m/group] uint16 raw fp16 bits
    zeros_u8: torch.Tensor    # [n, m/group] zero-points (generated, not consumed by the codec)
    group: int


def quantize_awq(w: torch.Tensor, group: int = 128) -> AwqCase:
    """Asymmetric INT4, groups of `group` along the input dim: scale=(max-min)/15 (fp16),
    zero=round(-min/scale), q=clamp(round(w/scale)+zero, 0, 15), stored unpacked."""
    wf = w.float()
    n, m = wf.shape
    v = wf.reshape(n, m // group, group)
    lo, hi = v.amin(dim=2), v.amax(dim=2)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8).to(torch.float16)
    sf = scale.float()
    zero = torch.round(-lo / sf).clamp(0, 15)
    q = (torch.round(v / sf[:, :, None]) + zero[:, :, None]).clamp(0, 15).to(torch.uint8).reshape(n, m)
    return AwqCase(w.contiguous(), q.contiguous(), scale.view(torch.uint16).contiguous(), zero.to(torch.uint8), group)


def model_tensors(cfg: dict, tp: int = 1, layers: int | None = None) -> Iterator[tuple[str, int, int]]:
    """(name, n, m) of every decoded linear of a rank's shard of the model."""
    nl = cfg["layers"] if layers is None else layers
    for li in range(nl):
        for name, n, m in layer_linears(cfg):
            sn, sm = tp_shard_shape(name, n, m, tp)
            yield f"model.layers.{li}.{name}", sn, sm
