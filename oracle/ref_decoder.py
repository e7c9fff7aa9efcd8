"""Loader for the reference's own CUDA FP8 decoder compiled by ``oracle/build_ref_decode.sh``.

TEST INFRASTRUCTURE ONLY: a second checker of this library's decoder on a GPU, and a timing of the
reference kernel for context.  ``available()`` is False where ``oracle/_ref`` holds no such build.

The shipped kernel (kernel/decode_huffman.cu:188-372) is correct only on part of the input space, so
``refusal(...)`` says why a sidecar must not be given to it, and ``decode_fp8`` refuses such a sidecar
on the host, before anything is launched:

* tables with an ESC entry: the kernel masks the flag off (:349-353) and loses its place in the stream;
* bitstreams of 3072 < W < 10240 words: the kernel copies the whole bitstream into shared memory when
  W < 10240 (:229-237) but the launch reserves room for 3072 words (:731-732);
* buckets narrower than their sub-stream count (col_len < k_eff): the element walk wraps at most one
  row per step (:358-369).
"""
from __future__ import annotations

import importlib.util
from pathlib import Path

_REF_DIR = Path(__file__).resolve().parent / "_ref"
_mod = None

ORDER = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_col_start_i32",
         "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32", "bucket_thread_startbit_u32",
         "bucket_bit_base_i64")


def _find():
    if not _REF_DIR.is_dir():
        return None
    for p in sorted(_REF_DIR.glob("mpserve_ref_decode*.so")):
        return p
    return None


def available() -> bool:
    return _find() is not None


def module():
    global _mod
    if _mod is None:
        import torch  # noqa: F401  (the extension links against libtorch)

        path = _find()
        if path is None:
            raise RuntimeError("oracle/_ref holds no reference decoder; run oracle/build_ref_decode.sh where the reference tree exists")
        spec = importlib.util.spec_from_file_location("mpserve_ref_decode", str(path))
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod


def refusal(art, n: int, m: int) -> str | None:
    """Why the shipped reference kernel must not be run on this sidecar (None: it may)."""
    import torch

    lens = art["decode_lens_u8"]
    if bool(((lens & 0x08) | (lens & 0x80)).any()):
        return "a table holds an ESC entry"
    words = int(art["bitstream_u64"].numel())
    if 3072 < words < 10240:
        return f"bitstream of {words} words would overrun the kernel's shared-memory copy"
    k = int(art["bucket_thread_startbit_u32"].shape[1]) - 1
    if not 1 <= k <= 1024:
        return "invalid sub-stream count"
    ofs = art["bucket_row_offsets_i32"].to(torch.int64)
    rows = ofs[1:] - ofs[:-1]
    col_len = art["bucket_col_len_i32"].to(torch.int64)
    col_start = art["bucket_col_start_i32"].to(torch.int64)
    k_eff = torch.clamp(rows * col_len, max=k)
    if bool((col_len < k_eff).any()):
        return "a bucket is narrower than its sub-stream count"
    if bool((rows <= 0).any()) or bool((col_start < 0).any()) or bool((col_start + col_len > m).any()):
        return "bucket geometry outside the tensor"
    idx = art["row_indices_i32"]
    if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= n):
        return "row index outside the tensor"
    table = art["bucket_table_i32"]
    if int(table.max()) >= int(art["decode_syms_u16"].shape[0]):
        return "table id outside the tables"
    return None


def decode_fp8(fp8_u8, art, n: int, m: int):
    """The reference kernel's output ``[n, m]`` BF16 for a sidecar it handles (raises otherwise).
    The reference launches on the legacy default stream; callers synchronise around the call."""
    why = refusal(art, n, m)
    if why is not None:
        raise ValueError(f"not given to the reference kernel: {why}")
    return module().huffman_decode_fp8(fp8_u8, *[art[k] for k in ORDER], int(n), int(m), 7)
