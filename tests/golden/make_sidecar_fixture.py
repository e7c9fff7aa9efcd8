"""Generates ``tests/golden/tiny_llama_sidecar/`` by running the REFERENCE's own offline compressor.

Run where the reference tree exists (``oracle/build_ref.sh`` must have compiled its CPU encoder):

    python tests/golden/make_sidecar_fixture.py [reference_root]

What it does: writes a one-layer Llama-shaped checkpoint twice (BF16, and FP8-E4M3 with per-tensor,
per-channel and 2-D block scales) into a temporary folder, then executes the reference's unmodified
``scripts/compress_llm_fp8_huffman.py`` on it with ``MPServe_cuda.huffman_build_fp8_decode_tables``
bound to the reference's unmodified CPU encoder (kernel/build_huffman.cu).  The sidecar shard that
script writes -- key names, signed-dtype casts, index and config edits, all of it the reference's --
is copied here together with the BF16 weights it must decode to.  Weights are seeded synthetic
N(0, 0.02); no real checkpoint is involved.
"""
from __future__ import annotations

import json
import os
import runpy
import shutil
import sys
import tempfile
import types
from pathlib import Path

import torch
from safetensors.torch import save_file

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from mpserve_b200 import workloads as wl  # noqa: E402
from oracle import ref_encoder as ref  # noqa: E402

OUT = Path(__file__).resolve().parent / "tiny_llama_sidecar"
HIDDEN, INTER, Q, KV = 128, 256, 128, 64
PREFIX = "model.layers.0"
# module -> (n, m, scale layout)
MODULES = {
    "self_attn.q_proj": (Q, HIDDEN, "tensor"),
    "self_attn.k_proj": (KV, HIDDEN, "channel_col"),   # per-channel scales stored [n, 1]
    "self_attn.v_proj": (KV, HIDDEN, "channel"),       # per-channel scales stored [n]
    "self_attn.o_proj": (HIDDEN, Q, "tensor"),
    "mlp.gate_proj": (INTER, HIDDEN, "block"),         # 2-D block scales [n/128, m/128], stored as weight_scale_inv
    "mlp.up_proj": (INTER, HIDDEN, "tensor"),
    "mlp.down_proj": (HIDDEN, INTER, "tensor"),
}


def pow2_channel_scales(w: torch.Tensor) -> torch.Tensor:
    """Per-row scales rounded up to a power of two: rows share scales, so the sidecar stays small."""
    amax = w.float().abs().amax(dim=1).clamp_min(1e-12)
    return torch.exp2(torch.ceil(torch.log2(amax / wl.FP8_MAX)))


def make_checkpoints(bf16_dir: Path, fp8_dir: Path) -> dict[str, torch.Tensor]:
    bf16, fp8 = {}, {}
    for i, (name, (n, m, layout)) in enumerate(MODULES.items()):
        w = wl.random_weight(n, m, 4242 + i, "normal")
        key = f"{PREFIX}.{name}.weight"
        bf16[key] = w
        wf = w.float()
        if layout == "tensor":
            scale = (wf.abs().amax() / wl.FP8_MAX).reshape(())
            q = wf / scale
            fp8[f"{PREFIX}.{name}.weight_scale"] = scale.to(torch.float32)
        elif layout in ("channel", "channel_col"):
            scale = pow2_channel_scales(w)
            q = wf / scale[:, None]
            fp8[f"{PREFIX}.{name}.weight_scale"] = (scale[:, None] if layout == "channel_col" else scale).to(torch.float32).contiguous()
        else:
            b0, b1 = 128, 128
            v = wf.reshape(n // b0, b0, m // b1, b1)
            scale = v.abs().amax(dim=(1, 3)) / wl.FP8_MAX
            q = (v / scale[:, None, :, None]).reshape(n, m)
            fp8[f"{PREFIX}.{name}.weight_scale_inv"] = scale.to(torch.float32).contiguous()
        fp8[key] = q.clamp(-wl.FP8_MAX, wl.FP8_MAX).to(torch.float8_e4m3fn).contiguous()
    # tensors the compressor must leave alone: no FP8 twin / not 2-D
    bf16["model.embed_tokens.weight"] = wl.random_weight(32, HIDDEN, 7, "normal")
    bf16["model.norm.weight"] = torch.ones(HIDDEN, dtype=torch.bfloat16)
    fp8["model.embed_tokens.weight"] = bf16["model.embed_tokens.weight"]
    fp8["model.norm.weight"] = bf16["model.norm.weight"]
    for d, tensors in ((bf16_dir, bf16), (fp8_dir, fp8)):
        d.mkdir(parents=True)
        save_file(tensors, str(d / "model.safetensors"))
        (d / "model.safetensors.index.json").write_text(json.dumps(
            {"metadata": {}, "weight_map": {k: "model.safetensors" for k in tensors}}))
        (d / "config.json").write_text(json.dumps({"model_type": "llama", "hidden_size": HIDDEN}))
    return bf16


def main() -> None:
    beside = Path(__file__).resolve().parents[3] / "reference"
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MPSERVE_REFERENCE_ROOT") or beside)
    script = ref_root / "scripts" / "compress_llm_fp8_huffman.py"
    if not script.exists():
        raise SystemExit(f"reference compressor not found: {script}")
    if not ref.available():
        raise SystemExit("oracle/_ref is not built: run oracle/build_ref.sh first")
    stub = types.ModuleType("MPServe_cuda")
    stub.huffman_build_fp8_decode_tables = ref.build_fp8   # the reference's own encoder, same keyword names
    sys.modules["MPServe_cuda"] = stub
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        bf16 = make_checkpoints(tmp / "bf16", tmp / "fp8")
        argv = sys.argv
        sys.argv = [str(script), "--bf16_model", str(tmp / "bf16"), "--fp8_model", str(tmp / "fp8"), "--out_dir", str(tmp / "out")]
        try:
            runpy.run_path(str(script), run_name="__main__")
        finally:
            sys.argv = argv
        if OUT.exists():
            shutil.rmtree(OUT)
        OUT.mkdir(parents=True)
        for name in ("huffman_fp8.safetensors", "model.safetensors.index.json", "config.json"):
            shutil.copy2(tmp / "out" / name, OUT / name)
        save_file({k: v for k, v in bf16.items() if k.startswith(PREFIX)}, str(OUT / "expected_bf16.safetensors"))
    total = sum(p.stat().st_size for p in OUT.iterdir())
    print(f"wrote {OUT} ({total} bytes)")


if __name__ == "__main__":
    main()
