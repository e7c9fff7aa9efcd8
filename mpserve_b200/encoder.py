"""Sidecar builders (the ``huffman_build_*`` entry points) on the GPU.

Argument checks, scale broadcasting rules and returned dict keys/dtypes follow the reference's CPU
builders (kernel/build_huffman.cu:292-969 for FP8, :1582-2126 for AWQ rectangular buckets;
bindings kernel/wrapper.cpp:258-288, 419-454).  Like the reference, inputs are CPU tensors and the
result is a dict of CPU tensors; the per-element work (histogram, codebooks, bit counting, bit
emission) runs on the current CUDA device through the C ABI, only the bucket row lists (a few
thousand integers derived from the scale tensor) are made on the host.  CUDA tensors are accepted
too and then nothing but the small metadata crosses PCIe.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib

V_FP8, V_AWQ_BUCKET = 0, 1


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("the sidecar builder needs a CUDA device (there is no CPU fallback)")
    return torch.device("cuda", torch.cuda.current_device())


def _scale_mode(scales: torch.Tensor, n: int, m: int, fp8_rules: bool):
    """(mode, nb0, nb1, sb0, sb1): 0 scalar, 1 per row, 2 two-dimensional blocks."""
    numel = scales.numel()
    if numel == 1:
        return 0, 1, 1, n, m
    if fp8_rules:
        if numel == n * m:
            raise ValueError("bucket packing requires scales to be scalar, per-row (n,), or 2D block-wise")
        if numel == n:
            return 1, n, 1, 1, m
        if scales.dim() == 2:
            nb0, nb1 = int(scales.size(0)), int(scales.size(1))
            if nb0 > 0 and nb1 > 0 and n % nb0 == 0 and m % nb1 == 0:
                return 2, nb0, nb1, n // nb0, m // nb1
        raise ValueError("unsupported scales shape: use scalar, per-row (n,), per-element (numel), or 2D block-wise "
                         "[n/bs0,m/bs1]")
    if scales.dim() == 1 and numel == n:
        return 1, n, 1, 1, m
    if scales.dim() == 2:
        nb0, nb1 = int(scales.size(0)), int(scales.size(1))
        if nb0 > 0 and nb1 > 0 and n % nb0 == 0 and m % nb1 == 0:
            return 2, nb0, nb1, n // nb0, m // nb1
    raise ValueError("unsupported scales_u16 shape: use scalar, per-row (n,), or 2D block-wise [n/bs0,m/bs1]")


def rect_buckets(scales_u16: np.ndarray, mode: int, n: int, m: int, nb0: int, nb1: int, sb0: int, sb1: int):
    """Buckets of <= 128 rows (build_huffman.cu:611-696): per distinct scale in ascending order for
    scalar / per-row scales, per (row block, column block) for 2-D block scales."""
    s = scales_u16.reshape(-1)
    if mode in (0, 1):
        row_scale = np.full(n, s[0], dtype=np.uint16) if mode == 0 else s.astype(np.uint16)
        order = np.lexsort((np.arange(n), row_scale))          # by scale, then row
        sorted_scale = row_scale[order]
        starts = np.flatnonzero(np.r_[True, sorted_scale[1:] != sorted_scale[:-1]])
        ends = np.r_[starts[1:], n]
        b_scale, b_ofs = [], [0]
        for a, e in zip(starts, ends):
            for off in range(a, e, 128):
                b_scale.append(sorted_scale[a])
                b_ofs.append(min(off + 128, e))
        B = len(b_scale)
        return (np.asarray(b_scale, dtype=np.uint16), np.asarray(b_ofs, dtype=np.int32), order.astype(np.int32),
                np.zeros(B, dtype=np.int32), np.full(B, m, dtype=np.int32))
    chunks = [(off, min(off + 128, sb0)) for off in range(0, sb0, 128)]
    b_scale, b_ofs, rows, cs, cl = [], [0], [], [], []
    grid = s.reshape(nb0, nb1)
    for br in range(nb0):
        for bc in range(nb1):
            for a, e in chunks:
                rows.append(np.arange(br * sb0 + a, br * sb0 + e, dtype=np.int32))
                b_scale.append(grid[br, bc])
                b_ofs.append(b_ofs[-1] + (e - a))
                cs.append(bc * sb1)
                cl.append(sb1)
    return (np.asarray(b_scale, dtype=np.uint16), np.asarray(b_ofs, dtype=np.int32),
            np.concatenate(rows).astype(np.int32) if rows else np.zeros(0, np.int32),
            np.asarray(cs, dtype=np.int32), np.asarray(cl, dtype=np.int32))


def _build_rect(variant: int, bf16, ctx_u8, scales, max_len: int, k: int, ctx_name: str) -> dict:
    lib = _lib.load()
    dev = _device()
    n, m = int(bf16.size(0)), int(bf16.size(1))
    if n <= 0 or m <= 0:
        raise ValueError("bf16_params shape must be non-empty")
    s16 = scales.contiguous()
    if s16.dtype == torch.bfloat16:
        s16 = s16.view(torch.uint16)
    mode, nb0, nb1, sb0, sb1 = _scale_mode(s16, n, m, variant == V_FP8)
    nctx = 256 if variant == V_FP8 else 16
    L = int(max_len)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        sym_d = bf16.contiguous().view(torch.uint16).to(dev)
        ctx_d = ctx_u8.contiguous().reshape(n, m).to(dev)
        sc_d = s16.to(dev)
        b_scale, b_ofs, rows, cs, cl = rect_buckets(s16.cpu().numpy(), mode, n, m, nb0, nb1, sb0, sb1)
        B = int(b_scale.size)
        ws_bytes = int(lib.mps_build_workspace_bytes(n * m, max(n * m, B * k)))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        state = (C.c_ubyte * 256)()
        G, N = C.c_int64(0), C.c_int64(0)
        _lib.check(lib.mps_build_analyze(state, sym_d.data_ptr(), ctx_d.data_ptr(), sc_d.data_ptr(), mode, nb1, sb0, sb1,
                                         n, m, variant, L, ws.data_ptr(), ws_bytes, stream, C.byref(G), C.byref(N)))
        G = int(G.value)
        TS = 1 << L
        syms = torch.empty((G, TS), dtype=torch.uint16, device=dev)
        lens = torch.empty((G, TS // 2), dtype=torch.uint8, device=dev)
        tscale = torch.empty((G,), dtype=torch.uint16, device=dev)
        tctx = torch.empty((G,), dtype=torch.uint16, device=dev)
        _lib.check(lib.mps_build_codebooks(state, syms.data_ptr(), lens.data_ptr(), tscale.data_ptr(), tctx.data_ptr(),
                                           stream))
        b_scale_d = torch.from_numpy(b_scale).to(dev)
        b_ofs_d = torch.from_numpy(b_ofs).to(dev)
        rows_d = torch.from_numpy(rows).to(dev)
        cs_d = torch.from_numpy(cs).to(dev)
        cl_d = torch.from_numpy(cl).to(dev)
        btab = torch.empty((B, nctx), dtype=torch.int32, device=dev)
        _lib.check(lib.mps_build_bucket_table(state, b_scale_d.data_ptr(), B, btab.data_ptr(), stream))
        tsb = torch.empty((B, k + 1), dtype=torch.uint32, device=dev)
        bbase = torch.empty((B + 1,), dtype=torch.int64, device=dev)
        total = C.c_int64(0)
        _lib.check(lib.mps_build_rect_layout(state, sym_d.data_ptr(), ctx_d.data_ptr(), btab.data_ptr(), cs_d.data_ptr(),
                                             cl_d.data_ptr(), b_ofs_d.data_ptr(), rows_d.data_ptr(), B, k, tsb.data_ptr(),
                                             bbase.data_ptr(), stream, C.byref(total)))
        words = (int(total.value) + 63) >> 6
        bits = torch.empty((words,), dtype=torch.uint64, device=dev)
        _lib.check(lib.mps_build_rect_emit(state, sym_d.data_ptr(), ctx_d.data_ptr(), btab.data_ptr(), cs_d.data_ptr(),
                                           cl_d.data_ptr(), b_ofs_d.data_ptr(), rows_d.data_ptr(), B, k, tsb.data_ptr(),
                                           bbase.data_ptr(), bits.data_ptr(), words, stream))
        out = {
            "decode_syms_u16": syms, "decode_lens_u8": lens, "table_scale_u16": tscale,
            ("table_fp8_u16" if variant == V_FP8 else "table_qv_u16"): tctx,
            "bucket_scale_u16": b_scale_d, "bucket_row_offsets_i32": b_ofs_d, "row_indices_i32": rows_d,
            "bucket_table_i32": btab, "bucket_col_start_i32": cs_d, "bucket_col_len_i32": cl_d,
            "bucket_thread_startbit_u32": tsb, "bucket_bit_base_i64": bbase, "bitstream_u64": bits,
            "shape_nmk_i64": torch.tensor([n, m, k], dtype=torch.int64),
        }
        if variant == V_FP8:
            U = torch.empty((B,), dtype=torch.int32, device=dev)
            uniq = torch.empty((B, 256), dtype=torch.int32, device=dev)
            uidx = torch.empty((B, 256), dtype=torch.int16, device=dev)
            _lib.check(lib.mps_build_bucket_unique(btab.data_ptr(), B, U.data_ptr(), uniq.data_ptr(), uidx.data_ptr(),
                                                   stream))
            out["bucket_U_i32"], out["bucket_unique_gid_i32"], out["bucket_fp8_uidx_i16"] = U, uniq, uidx
        torch.cuda.synchronize(dev)
        keep_on_device = bf16.is_cuda
        return {k_: (v if keep_on_device and v.is_cuda else v.cpu()) for k_, v in out.items()}


def build_fp8(bf16_params, fp8_params, scales, max_len, threads_per_block, limit=1024):
    """huffman_build_fp8_decode_tables (kernel/wrapper.cpp:419-454, build_huffman.cu:292-969).  ``limit``:
    most sub-streams per bucket accepted; 1024 is the reference's, with the reference's message."""
    for t in (bf16_params, fp8_params, scales):
        if not isinstance(t, torch.Tensor):
            raise ValueError("inputs must be defined")
    if bf16_params.dtype != torch.bfloat16:
        raise ValueError("bf16_params must be torch.bfloat16")
    if fp8_params.dtype != torch.uint8:
        raise ValueError("fp8_params must be torch.uint8")
    if max_len <= 0 or max_len > 15:
        raise ValueError("max_len must be in [1, 15]")
    if threads_per_block <= 0 or threads_per_block > limit:
        raise ValueError(f"threads_per_block must be in [1, {limit}]")
    if fp8_params.numel() != bf16_params.numel():
        raise ValueError("bf16_params and fp8_params must have same numel")
    if scales.dtype not in (torch.uint16, torch.bfloat16):
        raise ValueError("scales must be torch.uint16 or torch.bfloat16")
    if bf16_params.dim() != 2:
        raise ValueError("bucket packing requires bf16_params to be 2D [n,m]")
    return _build_rect(V_FP8, bf16_params, fp8_params, scales, max_len, int(threads_per_block), "fp8_params")


def build_awq_bucket(bf16_params, int4_values_u8, scales_u16, max_len, threads_per_block):
    """huffman_build_awq_int4_bucket_decode_tables (wrapper.cpp:258-288, build_huffman.cu:1582-2126)."""
    for t in (bf16_params, int4_values_u8, scales_u16):
        if not isinstance(t, torch.Tensor):
            raise ValueError("inputs must be defined")
    if bf16_params.dtype != torch.bfloat16:
        raise ValueError("bf16_params must be torch.bfloat16")
    if int4_values_u8.dtype != torch.uint8:
        raise ValueError("int4_values_u8 must be torch.uint8")
    if scales_u16.dtype != torch.uint16:
        raise ValueError("scales_u16 must be torch.uint16 (bf16 raw bits)")
    if max_len <= 0 or max_len > 15:
        raise ValueError("max_len must be in (0,15]")
    if threads_per_block <= 0 or threads_per_block > 1024:
        raise ValueError("threads_per_block must be in [1,1024]")
    if bf16_params.dim() != 2:
        raise ValueError("bf16_params must be 2D [n,m]")
    if tuple(int4_values_u8.shape) != tuple(bf16_params.shape):
        raise ValueError("int4_values_u8 shape must match bf16_params")
    return _build_rect(V_AWQ_BUCKET, bf16_params, int4_values_u8, scales_u16, max_len, int(threads_per_block),
                       "int4_values_u8")


def ragged_buckets(scales_u16: np.ndarray, mode: int, n: int, m: int, nb1: int, sb0: int, sb1: int, group_cap: int):
    """Groups (row, col_start) sorted by (scale, row, col) and cut into buckets of <= group_cap groups of
    one scale (build_huffman.cu:1353-1392)."""
    s = scales_u16.reshape(-1)
    if mode == 2:
        gpr, gsize = nb1, sb1
        rows = np.repeat(np.arange(n, dtype=np.int64), gpr)
        bcs = np.tile(np.arange(gpr, dtype=np.int64), n)
        sc = s.reshape(-1, nb1)[rows // sb0, bcs]
        c0 = bcs * sb1
    else:
        gpr, gsize = 1, m
        rows = np.arange(n, dtype=np.int64)
        c0 = np.zeros(n, dtype=np.int64)
        sc = np.full(n, s[0], dtype=np.uint16) if mode == 0 else s.astype(np.uint16)
    order = np.lexsort((c0, rows, sc))
    sc, rows, c0 = sc[order], rows[order], c0[order]
    starts = np.flatnonzero(np.r_[True, sc[1:] != sc[:-1]])
    ends = np.r_[starts[1:], sc.size]
    b_scale, b_ofs = [], [0]
    for a, e in zip(starts, ends):
        for off in range(a, e, group_cap):
            b_scale.append(sc[a])
            b_ofs.append(min(off + group_cap, e))
    return (np.asarray(b_scale, dtype=np.uint16), np.asarray(b_ofs, dtype=np.int32), rows.astype(np.int32),
            c0.astype(np.int32), int(gsize))


def build_awq_by_scale(bf16_values, int4_values, scales_u16, max_len, threads, group_cap):
    """huffman_build_awq_int4_bucket_decode_tables_by_scale (wrapper.cpp:290-321, build_huffman.cu:1074-1580)."""
    for t in (bf16_values, int4_values, scales_u16):
        if not isinstance(t, torch.Tensor):
            raise ValueError("inputs must be defined")
    if bf16_values.dtype != torch.bfloat16:
        raise ValueError("bf16_params must be torch.bfloat16")
    if int4_values.dtype != torch.uint8:
        raise ValueError("int4_values_u8 must be torch.uint8")
    if scales_u16.dtype != torch.uint16:
        raise ValueError("scales_u16 must be torch.uint16 (bf16 raw bits)")
    if max_len <= 0 or max_len > 15:
        raise ValueError("max_len must be in (0,15]")
    if threads <= 0 or threads > 1024:
        raise ValueError("threads_per_block must be in [1,1024]")
    if group_cap <= 0:
        raise ValueError("group_cap must be > 0")
    if bf16_values.dim() != 2:
        raise ValueError("bf16_params must be 2D [n,m]")
    if tuple(int4_values.shape) != tuple(bf16_values.shape):
        raise ValueError("int4_values_u8 shape must match bf16_params")
    lib = _lib.load()
    dev = _device()
    n, m = int(bf16_values.size(0)), int(bf16_values.size(1))
    if n <= 0 or m <= 0:
        raise ValueError("bf16_params shape must be non-empty")
    s16 = scales_u16.contiguous()
    mode, nb0, nb1, sb0, sb1 = _scale_mode(s16, n, m, False)
    L, k = int(max_len), int(threads)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        sym_d = bf16_values.contiguous().view(torch.uint16).to(dev)
        ctx_d = int4_values.contiguous().to(dev)
        sc_d = s16.to(dev)
        b_scale, b_ofs, g_rows, g_cols, gsize = ragged_buckets(s16.cpu().numpy(), mode, n, m, nb1, sb0, sb1,
                                                               int(group_cap))
        B = int(b_scale.size)
        ws_bytes = int(lib.mps_build_workspace_bytes(n * m, max(n * m, B * k)))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        state = (C.c_ubyte * 256)()
        G, N = C.c_int64(0), C.c_int64(0)
        _lib.check(lib.mps_build_analyze(state, sym_d.data_ptr(), ctx_d.data_ptr(), sc_d.data_ptr(), mode, nb1, sb0, sb1,
                                         n, m, 2, L, ws.data_ptr(), ws_bytes, stream, C.byref(G), C.byref(N)))
        G = int(G.value)
        TS = 1 << L
        syms = torch.empty((G, TS), dtype=torch.uint16, device=dev)
        lens = torch.empty((G, TS // 2), dtype=torch.uint8, device=dev)
        tscale = torch.empty((G,), dtype=torch.uint16, device=dev)
        tctx = torch.empty((G,), dtype=torch.uint16, device=dev)
        _lib.check(lib.mps_build_codebooks(state, syms.data_ptr(), lens.data_ptr(), tscale.data_ptr(), tctx.data_ptr(),
                                           stream))
        b_scale_d = torch.from_numpy(b_scale).to(dev)
        b_ofs_d = torch.from_numpy(b_ofs).to(dev)
        rows_d = torch.from_numpy(g_rows).to(dev)
        cols_d = torch.from_numpy(g_cols).to(dev)
        btab = torch.empty((B, 16), dtype=torch.int32, device=dev)
        _lib.check(lib.mps_build_bucket_table(state, b_scale_d.data_ptr(), B, btab.data_ptr(), stream))
        tsb = torch.empty((B, k + 1), dtype=torch.uint32, device=dev)
        bbase = torch.empty((B + 1,), dtype=torch.int64, device=dev)
        total = C.c_int64(0)
        _lib.check(lib.mps_build_rect_layout(state, sym_d.data_ptr(), ctx_d.data_ptr(), btab.data_ptr(),
                                             cols_d.data_ptr(), None, b_ofs_d.data_ptr(), rows_d.data_ptr(), B, k,
                                             tsb.data_ptr(), bbase.data_ptr(), stream, C.byref(total)))
        words = (int(total.value) + 63) >> 6
        bits = torch.empty((words,), dtype=torch.uint64, device=dev)
        _lib.check(lib.mps_build_rect_emit(state, sym_d.data_ptr(), ctx_d.data_ptr(), btab.data_ptr(), cols_d.data_ptr(),
                                           None, b_ofs_d.data_ptr(), rows_d.data_ptr(), B, k, tsb.data_ptr(),
                                           bbase.data_ptr(), bits.data_ptr(), words, stream))
        out = {
            "decode_syms_u16": syms, "decode_lens_u8": lens, "table_scale_u16": tscale, "table_qv_u16": tctx,
            "bucket_scale_u16": b_scale_d, "bucket_group_offsets_i32": b_ofs_d, "group_rows_i32": rows_d,
            "group_col_start_i32": cols_d, "bucket_table_i32": btab, "bucket_thread_startbit_u32": tsb,
            "bucket_bit_base_i64": bbase, "bitstream_u64": bits,
            "shape_nmkg_i64": torch.tensor([n, m, k, gsize], dtype=torch.int64),
        }
        torch.cuda.synchronize(dev)
        keep_on_device = bf16_values.is_cuda
        return {k_: (v if keep_on_device and v.is_cuda else v.cpu()) for k_, v in out.items()}


def build_awq_shared(bf16_params, int4_values_u8, scales_u16, max_len):
    """huffman_build_awq_decode_tables (wrapper.cpp:182-209, build_huffman.cu:2157-2633): one table per
    (scale id, int4 code) stream, one bitstream per scale, chunks of <= 255 same-stream elements."""
    for t in (bf16_params, int4_values_u8, scales_u16):
        if not isinstance(t, torch.Tensor):
            raise ValueError("inputs must be defined")
    if bf16_params.dtype != torch.bfloat16:
        raise ValueError("bf16_params must be torch.bfloat16")
    if int4_values_u8.dtype != torch.uint8:
        raise ValueError("int4_values_u8 must be torch.uint8")
    if scales_u16.dtype != torch.uint16:
        raise ValueError("scales_u16 must be torch.uint16 (bf16 raw bits)")
    if max_len <= 0 or max_len > 20:
        raise ValueError("max_len must be in (0,20]")
    if max_len > 15:
        raise NotImplementedError("the GPU builder holds code lengths up to 15 bits")
    if bf16_params.dim() != 2:
        raise ValueError("bf16_params must be 2D [n,m]")
    if tuple(int4_values_u8.shape) != tuple(bf16_params.shape):
        raise ValueError("int4_values_u8 shape must match bf16_params")
    lib = _lib.load()
    dev = _device()
    n, m = int(bf16_params.size(0)), int(bf16_params.size(1))
    if n <= 0 or m <= 0:
        raise ValueError("bf16_params shape must be non-empty")
    s16 = scales_u16.contiguous()
    mode, nb0, nb1, sb0, sb1 = _scale_mode(s16, n, m, False)
    L = int(max_len)
    numel = n * m
    # dense ids of the scale values that occur, ascending by value (build_huffman.cu:2221-2256)
    sv = np.unique(s16.cpu().numpy().reshape(-1))
    S = int(sv.size)
    lut = np.full(65536, -1, dtype=np.int32)
    lut[sv] = np.arange(S, dtype=np.int32)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        sym_d = bf16_params.contiguous().view(torch.uint16).to(dev)
        q_d = int4_values_u8.contiguous().to(dev)
        sc_d = s16.to(dev)
        lut_d = torch.from_numpy(lut).to(dev)
        ws_bytes = int(lib.mps_build_workspace_bytes(numel, 8 * numel))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        state = (C.c_ubyte * 256)()
        G, N = C.c_int64(0), C.c_int64(0)
        _lib.check(lib.mps_build_analyze(state, sym_d.data_ptr(), q_d.data_ptr(), sc_d.data_ptr(), mode, nb1, sb0, sb1,
                                         n, m, 3, L, ws.data_ptr(), ws_bytes, stream, C.byref(G), C.byref(N)))
        TS = 1 << L
        syms = torch.empty((S * 16, TS), dtype=torch.int16, device=dev)
        nbits = torch.empty((S * 16, TS), dtype=torch.uint8, device=dev)
        _lib.check(lib.mps_build_shared_codebooks(state, lut_d.data_ptr(), S, syms.data_ptr(), nbits.data_ptr(), stream))
        sbase = torch.empty((S + 1,), dtype=torch.int64, device=dev)
        nchunks, total_bits = C.c_int64(0), C.c_int64(0)
        _lib.check(lib.mps_build_shared_layout(state, sym_d.data_ptr(), q_d.data_ptr(), sc_d.data_ptr(), mode, nb1, sb0,
                                               sb1, lut_d.data_ptr(), sbase.data_ptr(), stream, C.byref(nchunks),
                                               C.byref(total_bits)))
        NC, words = int(nchunks.value), int(total_bits.value) >> 6
        bits = torch.empty((words,), dtype=torch.uint64, device=dev)
        c_start = torch.empty((NC,), dtype=torch.uint32, device=dev)
        c_base = torch.empty((NC,), dtype=torch.uint32, device=dev)
        c_meta = torch.empty((NC,), dtype=torch.uint32, device=dev)
        c_sid = torch.empty((NC,), dtype=torch.int32, device=dev)
        out_idx = torch.empty((numel,), dtype=torch.int32, device=dev)
        s_ofs = torch.empty((S * 16 + 1,), dtype=torch.int64, device=dev)
        s_ids = torch.empty((NC,), dtype=torch.int32, device=dev)
        _lib.check(lib.mps_build_shared_emit(state, sym_d.data_ptr(), sbase.data_ptr(), bits.data_ptr(), words,
                                             c_start.data_ptr(), c_base.data_ptr(), c_meta.data_ptr(), c_sid.data_ptr(),
                                             out_idx.data_ptr(), s_ofs.data_ptr(), s_ids.data_ptr(), stream))
        out = {
            "decode_syms_i16": syms, "decode_nbits_u8": nbits, "scale_values_u16": torch.from_numpy(sv.astype(np.uint16)),
            "scale_bit_base_i64": sbase, "chunk_startbit_rel_u32": c_start, "chunk_out_base_u32": c_base,
            "chunk_meta_u32": c_meta, "chunk_scale_id_i32": c_sid, "out_idx_i32": out_idx,
            "stream_chunk_ofs_i64": s_ofs, "stream_chunk_ids_i32": s_ids, "bitstream_u64": bits,
        }
        torch.cuda.synchronize(dev)
        keep_on_device = bf16_params.is_cuda
        return {k_: (v if keep_on_device and v.is_cuda else v.cpu()) for k_, v in out.items()}
