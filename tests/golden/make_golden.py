"""Generates the golden fixtures in this folder with the REFERENCE's own CPU encoder.

Run where the reference tree exists (it is compiled by ``oracle/build_ref.sh`` into
``oracle/_ref``):

    oracle/build_ref.sh && python tests/golden/make_golden.py

Each ``<case>.npz`` holds the seeded inputs (BF16 bits, context bytes, scale bits), the encoder
arguments, and every artifact the reference encoder returned: stored whole when small, else as a
SHA-256 over its bytes plus shape and dtype.  The reference ships no decoder that runs on a CPU and
no golden vectors, so the expected decode of every case is its own ``in_bf16``.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from mpserve_b200 import workloads as wl  # noqa: E402
from oracle import ref_encoder as ref  # noqa: E402

OUT = Path(__file__).resolve().parent
WHOLE_LIMIT = 96 * 1024  # bytes


def _np(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def _save(name: str, kind: str, bf16, ctx, scales, params: dict, art: dict) -> None:
    rec = {"in_bf16": _np(bf16), "in_ctx": _np(ctx), "in_scales": _np(scales)}
    meta = {"kind": kind, "params": params, "artifacts": {}}
    for k, v in art.items():
        a = np.ascontiguousarray(_np(v))
        meta["artifacts"][k] = {"shape": list(a.shape), "dtype": str(a.dtype),
                                "sha256": hashlib.sha256(a.tobytes()).hexdigest()}
        if a.nbytes <= WHOLE_LIMIT:
            rec["art_" + k] = a
    rec["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(OUT / f"{name}.npz", **rec)
    print(f"{name}: {sum(v.nbytes for v in rec.values())} raw bytes")


def fp8(name, n, m, seed, dist, mode, k, block=(128, 128), L=7, mutate=None):
    w = wl.random_weight(n, m, seed, dist)
    if mutate is not None:
        w = mutate(w)
    c = wl.quantize_fp8(w, mode, block)
    art = ref.build_fp8(c.bf16, c.fp8_u8, c.scales_u16, L, k)
    _save(name, "fp8", c.bf16, c.fp8_u8, c.scales_u16, {"max_len": L, "threads_per_block": k}, art)


def awq(name, n, m, seed, group, k, scale_kind="group", L=11, cap=1024, const_q=None, dist="normal"):
    w = wl.random_weight(n, m, seed, dist)
    c = wl.quantize_awq(w, group)
    sc, q = c.scales_u16, c.int4_u8
    if scale_kind == "row":
        sc = sc[:, 0].contiguous()
    elif scale_kind == "scalar":
        sc = sc[:1, 0].contiguous().reshape(1)
    if const_q is not None:
        q = torch.full_like(q, const_q)
    _save(name + "_bucket", "awq_bucket", c.bf16, q, sc, {"max_len": L, "threads_per_block": k},
          ref.build_awq_bucket(c.bf16, q, sc, L, k))
    _save(name + "_byscale", "awq_by_scale", c.bf16, q, sc, {"max_len": L, "threads": k, "group_cap": cap},
          ref.build_awq_by_scale(c.bf16, q, sc, L, k, cap))
    _save(name + "_shared", "awq_shared", c.bf16, q, sc, {"max_len": L}, ref.build_awq_shared(c.bf16, q, sc, L))


def _outlier(w: torch.Tensor) -> torch.Tensor:
    # one huge element => per-tensor scale so coarse that nearly everything quantises to fp8 codes
    # 0x00/0x80, whose contexts then hold far more than 128 distinct BF16 values (ESC tables)
    w = w.clone()
    w[0, 0] = 1.0e4
    return w


def main() -> None:
    fp8("fp8_tensor_64x256_k256", 64, 256, 11, "normal", "tensor", 256)
    fp8("fp8_channel_48x320_k1024", 48, 320, 12, "normal", "channel", 1024)       # col_len < k
    fp8("fp8_block_128x256_k256", 128, 256, 13, "student_t", "block", 256, (64, 128))  # 2-D block scales
    fp8("fp8_esc_96x256_k128", 96, 256, 14, "normal", "tensor", 128, mutate=_outlier)   # ESC contexts
    fp8("fp8_tiny_3x5_k32", 3, 5, 15, "normal", "tensor", 32)                     # total_elems < k
    awq("awq_group_16x256_k256", 16, 256, 21, 128, 256)
    awq("awq_row_32x128_k64", 32, 128, 22, 128, 64, scale_kind="row")
    awq("awq_esc_96x256_k256", 96, 256, 23, 128, 256, scale_kind="scalar", const_q=3, cap=7,
        dist="student_t")  # one context with > 2048 distinct symbols


if __name__ == "__main__":
    main()
