"""Decode throughput of single tensors by size, value distribution and sidecar format.

    python -m mpserve_b200.sweep single          # one 4096x4096 weight, per-tensor FP8 scale
    python -m mpserve_b200.sweep sizes           # 64 KB ... 1 GB of BF16 output, N(0,0.02) and Student-t(4)
    python -m mpserve_b200.sweep awq             # Llama-3-8B-shaped linears as INT4 (group 128), the three sidecar layouts

Every case is generated, quantised and encoded on the GPU by this library's own builder, decoded
through the per-tensor entry point the reference's plugin calls (``huffman_decode_fp8`` and the AWQ
siblings), checked bit for bit against the source weights, and then timed with CUDA events.  L2 is
flushed (a 256 MB write) before every timed call, so small tensors are read from HBM as they would be
during a model load.  One JSON line per case on stdout.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from . import workloads as wl


def _flush_buffer(dev):
    return torch.empty(256 << 20, dtype=torch.uint8, device=dev)


def _time_calls(fn, flush, reps: int) -> tuple[float, float]:
    """(median, best) milliseconds of fn() with a cold L2."""
    for _ in range(3):
        fn()
    times = []
    for _ in range(reps):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2], times[0]


def _art_bytes(art: dict, keys) -> int:
    return sum(art[k].numel() * art[k].element_size() for k in keys)


_FP8_KEYS = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_col_start_i32",
             "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32", "bucket_thread_startbit_u32",
             "bucket_bit_base_i64")
_SHARED_KEYS = ("bitstream_u64", "decode_syms_i16", "decode_nbits_u8", "scale_bit_base_i64", "chunk_startbit_rel_u32",
                "chunk_out_base_u32", "chunk_meta_u32", "chunk_scale_id_i32", "out_idx_i32", "stream_chunk_ofs_i64",
                "stream_chunk_ids_i32")
_BYSCALE_KEYS = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_group_offsets_i32",
                 "group_rows_i32", "group_col_start_i32", "bucket_thread_startbit_u32", "bucket_bit_base_i64")


def fp8_case(n: int, m: int, dist: str, scale_mode: str, k: int, seed: int, dev, flush, reps: int) -> dict:
    import MPServe_cuda

    w = wl.random_weight(n, m, seed, dist, device=dev)
    c = wl.quantize_fp8(w, scale_mode)
    art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=k)
    a = [art[key] for key in _FP8_KEYS]

    def run():
        return MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *a, n, m, 7)

    out = run()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16)), "decode mismatch"
    med, best = _time_calls(run, flush, reps)
    elems = n * m
    alg = elems + _art_bytes(art, _FP8_KEYS) + 2 * elems
    return {"case": f"fp8 {scale_mode} {dist} {n}x{m} k={k}", "out_bytes": 2 * elems, "ms_median": med, "ms_best": best,
            "bf16_gbps": 2 * elems / med / 1e6, "algorithmic_gbps": alg / med / 1e6,
            "algorithmic_bytes_per_element": alg / elems,
            "code_bits_per_element": 64.0 * art["bitstream_u64"].numel() / elems,
            "buckets": int(art["bucket_table_i32"].size(0)), "tables": int(art["decode_syms_u16"].size(0))}


def awq_case(name: str, n: int, m: int, layout: str, k: int, seed: int, dev, flush, reps: int) -> dict:
    import MPServe_cuda

    w = wl.random_weight(n, m, seed, "normal", device=dev)
    c = wl.quantize_awq(w, 128)
    if layout == "bucket":
        art = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables(c.bf16, c.int4_u8, c.scales_u16, max_len=11,
                                                                       threads_per_block=k)
        keys = _FP8_KEYS
        a = [art[key] for key in keys]

        def run():
            return MPServe_cuda.huffman_decode_awq_int4_bucket(c.int4_u8, *a, n, m, 11)
    elif layout == "shared":
        art = MPServe_cuda.huffman_build_awq_decode_tables(c.bf16, c.int4_u8, c.scales_u16, max_len=11)
        keys = _SHARED_KEYS
        a = [art[key] for key in keys]

        def run():
            return MPServe_cuda.huffman_decode_awq_shared_table(*a, n * m, 11).view(torch.bfloat16).view(n, m)
    else:
        art = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables_by_scale(c.bf16, c.int4_u8, c.scales_u16, max_len=11,
                                                                                threads=k, group_cap=1024)
        keys = _BYSCALE_KEYS
        a = [art[key] for key in keys]
        gs = int(art["shape_nmkg_i64"][3])

        def run():
            return MPServe_cuda.huffman_decode_awq_int4_bucket_by_scale(c.int4_u8, *a, n, m, 11, gs)

    out = run()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16)), "decode mismatch"
    med, best = _time_calls(run, flush, reps)
    elems = n * m
    alg = (0 if layout == "shared" else elems) + _art_bytes(art, keys) + 2 * elems   # the shared layout reads no int4 codes
    return {"case": f"awq g128 {layout} {name} {n}x{m} k={k}", "out_bytes": 2 * elems, "ms_median": med, "ms_best": best,
            "bf16_gbps": 2 * elems / med / 1e6, "algorithmic_gbps": alg / med / 1e6,
            "algorithmic_bytes_per_element": alg / elems,
            "code_bits_per_element": 64.0 * art["bitstream_u64"].numel() / elems,
            "buckets": int(art["bucket_table_i32"].size(0)) if layout != "shared" else int(art["chunk_meta_u32"].numel()),
            "tables": int(art["decode_syms_u16" if layout != "shared" else "decode_syms_i16"].size(0))}


SIZES = [(128, 256), (256, 512), (512, 1024), (1024, 2048), (2048, 4096), (4096, 4096), (8192, 8192), (16384, 8192),
         (16384, 16384), (32768, 16384)]     # 64 KB ... 1 GB of BF16


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["single", "sizes", "awq"])
    ap.add_argument("--reps", type=int, default=15)
    ap.add_argument("--k", type=int, default=None, help="sub-streams per bucket (threads_per_block of the builder)")
    ap.add_argument("--max-bytes", type=int, default=1 << 30, help="largest BF16 output of the size sweep")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("a CUDA device is required", file=sys.stderr)
        return 2
    dev = torch.device("cuda", 0)
    flush = _flush_buffer(dev)
    rows = []
    if args.what == "single":
        for k in ([args.k] if args.k else [256, 1024]):
            rows.append(fp8_case(4096, 4096, "normal", "tensor", k, 7, dev, flush, args.reps))
            print(json.dumps(rows[-1]), flush=True)
    elif args.what == "sizes":
        k = args.k or 1024
        for dist in ("normal", "student_t"):
            for n, m in SIZES:
                if 2 * n * m > args.max_bytes:
                    continue
                rows.append(fp8_case(n, m, dist, "channel", k, 11, dev, flush, args.reps))
                print(json.dumps(rows[-1]), flush=True)
                torch.cuda.empty_cache()
    else:
        k = args.k or 256
        for layout in ("byscale", "bucket", "shared"):
            for i, (name, n, m) in enumerate(wl.layer_linears(wl.LLAMA3_8B)):
                if layout == "shared" and i not in (0, 1):
                    continue   # one square and one small tensor: the format's metadata is ~20 B per element
                rows.append(awq_case(name, n, m, layout, k, 100 + i, dev, flush, max(3, args.reps // 3)))
                print(json.dumps(rows[-1]), flush=True)
                torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
