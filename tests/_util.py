"""Shared helpers of the test-suite: golden fixture loading and artifact comparison."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


class Golden:
    def __init__(self, path: Path):
        z = np.load(path)
        self.name = path.stem
        self.meta = json.loads(bytes(z["meta"]).decode())
        self.kind = self.meta["kind"]
        self.params = self.meta["params"]
        self.bf16 = z["in_bf16"]
        self.ctx = z["in_ctx"]
        self.scales = z["in_scales"]
        self.whole = {k[4:]: z[k] for k in z.files if k.startswith("art_")}
        self.info = self.meta["artifacts"]

    def check_artifacts(self, art: dict) -> None:
        """Every artifact equals the reference encoder's, whole or by SHA-256."""
        assert set(art) == set(self.info), (sorted(art), sorted(self.info))
        for k, inf in self.info.items():
            a = np.ascontiguousarray(art[k])
            assert list(a.shape) == inf["shape"], (self.name, k, a.shape, inf["shape"])
            assert str(a.dtype) == inf["dtype"], (self.name, k, a.dtype, inf["dtype"])
            if k in self.whole:
                np.testing.assert_array_equal(a, self.whole[k], err_msg=f"{self.name}:{k}")
            assert hashlib.sha256(a.tobytes()).hexdigest() == inf["sha256"], (self.name, k)


def load_all_golden() -> dict[str, Golden]:
    return {p.stem: Golden(p) for p in sorted(GOLDEN_DIR.glob("*.npz"))}


def golden_names(kind: str | None = None) -> list[str]:
    out = []
    for p in sorted(GOLDEN_DIR.glob("*.npz")):
        if kind is None or p.stem.startswith(kind):
            out.append(p.stem)
    return out


def has_esc_fp8(art: dict) -> bool:
    lens = art["decode_lens_u8"]
    return bool((((lens & 0x08) != 0) | ((lens & 0x80) != 0)).any())


def has_esc_awq(art: dict) -> bool:
    lens = art["decode_lens_u8"]
    return bool((((lens & 0x0F) == 15) | ((lens >> 4) == 15)).any())
