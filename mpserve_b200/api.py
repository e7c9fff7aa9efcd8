"""Python mirror of the reference's ``MPServe_cuda`` extension module for the Huffman-sidecar path.

Same function names, argument order, keyword names, defaults, returned dtypes and exception
classes as the pybind module in kernel/wrapper.cpp:132-504 of the reference
(``std::invalid_argument`` -> ``ValueError``, ``std::runtime_error`` -> ``RuntimeError``), so that
scripts/mpserve_vllm_fp8_huffman.py and scripts/compress_llm_fp8_huffman.py can import this module
under the name ``MPServe_cuda`` unchanged.  Underneath, every call goes through the C ABI of
``libmpserve_b200.so``; PyTorch only supplies device memory and the current stream.  There is no
CPU fallback: without the built library (or without a CUDA device) the calls raise.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib

__all__ = [
    "cuda_clock_rate_khz", "huffman_decode_fp8", "huffman_decode_awq_int4_bucket",
    "huffman_decode_awq_int4_bucket_by_scale", "huffman_decode_awq_shared_table",
    "huffman_build_fp8_decode_tables", "huffman_build_awq_int4_bucket_decode_tables",
    "huffman_build_awq_int4_bucket_decode_tables_by_scale", "huffman_build_awq_decode_tables",
    "build_fp8_fine_substreams", "MAX_SUBSTREAMS", "MAX_SUBSTREAMS_REFERENCE",
    "BucketDecodePlan", "checksum_u16", "decode_timed_out", "noalloc_decode_timed_out", "selftest_stalled_decode",
]

# Sub-streams per bucket: the reference builds and decodes at most 1024 (one thread of one block each,
# kernel/build_huffman.cu:313, kernel/decode_huffman.cu:695); this library up to MAX_SUBSTREAMS
# (include/mpserve_b200.h).  The decode calls for rectangular buckets (FP8, AWQ) accept both, the by-scale
# call keeps the reference's limit (no builder here writes more); the builders under the reference's
# names keep the reference's limit too, build_fp8_fine_substreams is the way to more.
MAX_SUBSTREAMS_REFERENCE = 1024
MAX_SUBSTREAMS = 8192

_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, stream=None) -> torch.Tensor:
    """Zeroed queue counters, one per (device, stream); kernels hand them back zeroed."""
    if stream is None:
        stream = torch.cuda.current_stream(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream.cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        nbytes = int(_lib.load().mps_workspace_bytes())
        ws = torch.zeros(nbytes // 4, dtype=torch.int32, device=device)
        _workspaces[key] = ws
    return ws


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def _check_cuda_contig(t, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be defined")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _same_device(tensors: Sequence[torch.Tensor]) -> torch.device:
    dev = tensors[0].device
    for t in tensors[1:]:
        if t.device != dev:
            raise ValueError("all tensors must be on the same CUDA device")
    return dev


def decode_timed_out(device: torch.device | None = None) -> bool:
    """Waits for the current stream and tells whether a decode launched on it since the last call gave
    up on one of its bounded waits (its outputs are then incomplete).  Always False in normal operation."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        ws = _workspace(dev)
        flag = C.c_int32(0)
        _lib.check(_lib.load().mps_decode_status(ws.data_ptr(), ws.numel() * 4, _stream_ptr(dev), C.byref(flag)))
    return bool(flag.value)


def noalloc_decode_timed_out(device: torch.device | None = None) -> bool:
    """Same question for the decodes made through ``mps_decode_fp8_noalloc``, whose queue counters (and
    give-up record) live in the library's own device scratch instead of a caller's workspace."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        flag = C.c_int32(0)
        _lib.check(_lib.load().mps_decode_status(None, 0, _stream_ptr(dev), C.byref(flag)))
    return bool(flag.value)


def selftest_stalled_decode(ctx_u8: torch.Tensor, art: dict, out: torch.Tensor, stall_block: int = 1,
                            polls: int = 20000) -> None:
    """Bring-up check of the bounded waits (``mps_selftest_stalled_decode``): decodes one FP8 tensor with the
    context bytes of one block of steps never copied, so that the decoding warps' wait runs out after
    ``polls`` polls and the kernel returns early.  ``decode_timed_out()`` is True afterwards; ``out`` is
    incomplete.  Nothing hangs or faults."""
    dev = ctx_u8.device
    d = _lib.BucketTensor()
    n, m = int(ctx_u8.shape[0]), int(ctx_u8.shape[1])
    d.ctx_bytes = ctx_u8.data_ptr()
    d.bitstream = art["bitstream_u64"].data_ptr(); d.bitstream_words = art["bitstream_u64"].numel()
    d.decode_syms = art["decode_syms_u16"].data_ptr(); d.decode_lens = art["decode_lens_u8"].data_ptr()
    d.num_tables = art["decode_syms_u16"].size(0)
    d.bucket_table = art["bucket_table_i32"].data_ptr()
    d.bucket_col_start = art["bucket_col_start_i32"].data_ptr(); d.bucket_col_len = art["bucket_col_len_i32"].data_ptr()
    d.bucket_row_offsets = art["bucket_row_offsets_i32"].data_ptr(); d.row_indices = art["row_indices_i32"].data_ptr()
    d.num_rows = art["row_indices_i32"].numel()
    d.thread_startbit = art["bucket_thread_startbit_u32"].data_ptr(); d.bucket_bit_base = art["bucket_bit_base_i64"].data_ptr()
    d.num_buckets = art["bucket_table_i32"].size(0)
    d.k = int(art["bucket_thread_startbit_u32"].size(1)) - 1
    d.mode, d.n, d.m, d.out = 0, n, m, out.data_ptr()
    with torch.cuda.device(dev):
        ws = _workspace(dev)
        _lib.check(_lib.load().mps_selftest_stalled_decode(C.byref(d), int(stall_block), int(polls), ws.data_ptr(),
                                                          ws.numel() * 4, _stream_ptr(dev)))


def cuda_clock_rate_khz() -> int:
    """SM clock of the current device in kHz (kernel/wrapper.cpp:133-141)."""
    v = int(_lib.load().mps_cuda_clock_rate_khz())
    if v <= 0:
        _lib.check(v if v < 0 else 1)
    return v


# ----------------------------------------------------------------------------------------------
# decode
# ----------------------------------------------------------------------------------------------

def _check_bucket_common(ctx, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
                         bucket_thread_startbit_u32, bucket_bit_base_i64, ctx_name: str, nctx: int) -> None:
    if ctx.dtype != torch.uint8:
        raise ValueError(f"{ctx_name} must be uint8 CUDA")
    if bitstream_u64.dtype != torch.uint64 or bitstream_u64.dim() != 1:
        raise ValueError("bitstream_u64 must be uint64 1D CUDA")
    if decode_syms_u16.dtype != torch.uint16 or decode_syms_u16.dim() != 2:
        raise ValueError("decode_syms_u16 must be uint16 2D CUDA [G, 2^L]")
    if decode_lens_u8.dtype != torch.uint8 or decode_lens_u8.dim() != 2:
        raise ValueError("decode_lens_u8 must be uint8 2D CUDA [G, 2^(L-1)]")
    if bucket_table_i32.dtype != torch.int32 or bucket_table_i32.dim() != 2 or bucket_table_i32.size(1) != nctx:
        raise ValueError(f"bucket_table_i32 must be int32 CUDA [B,{nctx}]")
    if bucket_thread_startbit_u32.dtype != torch.uint32 or bucket_thread_startbit_u32.dim() != 2:
        raise ValueError("bucket_thread_startbit_u32 must be uint32 2D CUDA [B,k+1]")
    if bucket_bit_base_i64.dtype != torch.int64 or bucket_bit_base_i64.dim() != 1:
        raise ValueError("bucket_bit_base_i64 must be int64 1D CUDA [B+1]")


def _check_tables(decode_syms_u16, decode_lens_u8, L: int) -> None:
    if decode_syms_u16.size(1) != (1 << L):
        raise ValueError("decode_syms_u16 second dim must be 2^max_len")
    if decode_lens_u8.size(1) != (1 << (L - 1)):
        raise ValueError("decode_lens_u8 second dim must be 2^(max_len-1)")
    if decode_syms_u16.size(0) != decode_lens_u8.size(0):
        raise ValueError("decode_syms_u16 and decode_lens_u8 first dim must match")


def _check_rect(bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
                bucket_thread_startbit_u32, bucket_bit_base_i64, B: int) -> int:
    for t, nm, shape in ((bucket_col_start_i32, "bucket_col_start_i32", "[B]"),
                         (bucket_col_len_i32, "bucket_col_len_i32", "[B]"),
                         (bucket_row_offsets_i32, "bucket_row_offsets_i32", "[B+1]"),
                         (row_indices_i32, "row_indices_i32", "")):
        if t.dtype != torch.int32 or t.dim() != 1:
            raise ValueError(f"{nm} must be int32 1D CUDA {shape}".rstrip())
    if bucket_col_start_i32.numel() != B:
        raise ValueError("bucket_col_start_i32 length must be B")
    if bucket_col_len_i32.numel() != B:
        raise ValueError("bucket_col_len_i32 length must be B")
    if bucket_row_offsets_i32.numel() != B + 1:
        raise ValueError("bucket_row_offsets_i32 length must be B+1")
    if bucket_thread_startbit_u32.size(0) != B:
        raise ValueError("bucket_thread_startbit_u32 first dim must be B")
    if bucket_bit_base_i64.numel() != B + 1:
        raise ValueError("bucket_bit_base_i64 length must be B+1")
    k = int(bucket_thread_startbit_u32.size(1)) - 1
    if k <= 0 or k > MAX_SUBSTREAMS:
        raise ValueError(f"bucket_thread_startbit_u32 has invalid k (must be 1..{MAX_SUBSTREAMS})")
    return k


def validate_decode_fp8(fp8_params_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
                        bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
                        bucket_thread_startbit_u32, bucket_bit_base_i64, n, m, max_len, require_cuda: bool = True):
    """Argument checks of ``huffman_decode_fp8`` in the order, and with the messages, of the reference
    entry (decode_huffman.cu:606-697).  Returns ``(n, m, max_len, B, k, tensors)``.  ``require_cuda=False``
    leaves out the device test only, so that the host-side contract can be exercised without a GPU."""
    names = ("fp8_params_u8", "bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32",
             "bucket_col_start_i32", "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32",
             "bucket_thread_startbit_u32", "bucket_bit_base_i64")
    tensors = (fp8_params_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
               bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
               bucket_thread_startbit_u32, bucket_bit_base_i64)
    for t, nm in zip(tensors, names):
        if require_cuda:
            _check_cuda_contig(t, nm)
        else:
            if not isinstance(t, torch.Tensor):
                raise ValueError(f"{nm} must be defined")
            if not t.is_contiguous():
                raise ValueError(f"{nm} must be contiguous")
    _check_bucket_common(fp8_params_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
                         bucket_thread_startbit_u32, bucket_bit_base_i64, "fp8_params_u8", 256)
    n, m, max_len = int(n), int(m), int(max_len)
    if max_len <= 0 or max_len > 15:
        raise ValueError("max_len must be in [1,15]")
    if max_len != 7:
        raise ValueError("decode kernel is specialized: max_len must be 7")
    if n <= 0 or m <= 0:
        raise ValueError("n,m must be > 0")
    if fp8_params_u8.numel() != n * m:
        raise ValueError("fp8_params_u8 numel must equal n*m")
    B = int(bucket_table_i32.size(0))
    k = _check_rect(bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
                    bucket_thread_startbit_u32, bucket_bit_base_i64, B)
    _check_tables(decode_syms_u16, decode_lens_u8, 7)
    return n, m, max_len, B, k, tensors


def huffman_decode_fp8(fp8_params_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
                       bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
                       bucket_thread_startbit_u32, bucket_bit_base_i64, n, m, max_len=12, *, out=None):
    """FP8 + sidecar -> BF16 ``[n, m]`` (kernel/wrapper.cpp:457-503, decode_huffman.cu:591-758).

    Launches asynchronously on the current CUDA stream of the inputs' device and returns a newly
    allocated tensor, as the reference does.  ``out`` (keyword only, not part of the reference's
    signature) names a contiguous BF16 ``[n, m]`` tensor to decode into instead: a row range of a fused
    ``qkv`` / ``gate_up`` weight, or a buffer kept across forwards.
    """
    tensors = (fp8_params_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32, bucket_col_start_i32,
               bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32, bucket_thread_startbit_u32,
               bucket_bit_base_i64)
    try:
        key = (*map(id, tensors), n, m, max_len)
        memo = _fp8_checked.get(key)
    except TypeError:   # an argument that cannot be hashed takes the full checks, which name it
        key = memo = None
    if memo is None or not memo.still_holds(tensors):
        memo = _CheckedFp8(*validate_decode_fp8(*tensors, n, m, max_len))
        if key is not None:
            if len(_fp8_checked) >= _CHECKED_CAP:
                _fp8_checked.clear()
            _fp8_checked[key] = memo
    dev = memo.device
    if out is None:
        out = torch.empty((memo.n, memo.m), dtype=torch.bfloat16, device=dev)
    else:
        _check_cuda_contig(out, "out")
        if out.dtype != torch.bfloat16 or out.numel() != memo.n * memo.m or out.device != dev:
            raise ValueError("out must be a contiguous bfloat16 CUDA tensor of n*m elements on the inputs' device")
    desc = _lib.BucketTensor.from_buffer_copy(memo.desc)   # a private copy: concurrent callers share the memo
    desc.out = out.data_ptr()
    if torch.cuda.current_device() == memo.device_index:
        stream = torch.cuda.current_stream(dev)
        ws = _workspace(dev, stream)
        rc = _lib.load().mps_decode_bucket_tensor(C.byref(desc), ws.data_ptr(), ws.numel() * 4, stream.cuda_stream)
    else:
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev)
            ws = _workspace(dev, stream)
            rc = _lib.load().mps_decode_bucket_tensor(C.byref(desc), ws.data_ptr(), ws.numel() * 4, stream.cuda_stream)
    _lib.check(rc)
    return out


class _CheckedFp8:
    """What one full argument check of ``huffman_decode_fp8`` established, kept so that the next call with
    the same tensor objects only has to confirm that nothing about them changed: a serving loop decodes
    the same weights on every forward, and the checks cost more host time than the launch.  Holds weak
    references only, so it keeps no device memory alive."""

    __slots__ = ("refs", "facts", "desc", "n", "m", "device", "device_index")

    def __init__(self, n, m, max_len, B, k, tensors):
        import weakref

        (fp8_params_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32, bucket_col_start_i32,
         bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32, bucket_thread_startbit_u32,
         bucket_bit_base_i64) = tensors
        self.device = _same_device(tensors)
        self.device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.refs = tuple(weakref.ref(t) for t in tensors)
        self.facts = tuple((t.data_ptr(), t.shape, t.dtype) for t in tensors)
        self.n, self.m = n, m
        d = _lib.BucketTensor()
        d.ctx_bytes = fp8_params_u8.data_ptr()
        d.bitstream = bitstream_u64.data_ptr(); d.bitstream_words = bitstream_u64.numel()
        d.decode_syms = decode_syms_u16.data_ptr(); d.decode_lens = decode_lens_u8.data_ptr()
        d.num_tables = decode_syms_u16.size(0)
        d.bucket_table = bucket_table_i32.data_ptr()
        d.bucket_col_start = bucket_col_start_i32.data_ptr(); d.bucket_col_len = bucket_col_len_i32.data_ptr()
        d.bucket_row_offsets = bucket_row_offsets_i32.data_ptr(); d.row_indices = row_indices_i32.data_ptr()
        d.num_rows = row_indices_i32.numel()
        d.thread_startbit = bucket_thread_startbit_u32.data_ptr(); d.bucket_bit_base = bucket_bit_base_i64.data_ptr()
        d.num_buckets = B
        d.k = k
        d.mode, d.n, d.m = 0, n, m
        self.desc = d

    def still_holds(self, tensors) -> bool:
        for t, ref, (ptr, shape, dtype) in zip(tensors, self.refs, self.facts):
            if ref() is not t or t.data_ptr() != ptr or t.shape != shape or t.dtype is not dtype or not t.is_contiguous():
                return False
        return True


_fp8_checked: dict[tuple, _CheckedFp8] = {}
_CHECKED_CAP = 4096


def huffman_decode_awq_int4_bucket(int4_values_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
                                   bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
                                   bucket_thread_startbit_u32, bucket_bit_base_i64, n, m, max_len=11):
    """AWQ-INT4 rectangular buckets -> BF16 ``[n, m]`` (wrapper.cpp:324-369, decode_huffman.cu:877-1017)."""
    names = ("int4_values_u8", "bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32",
             "bucket_col_start_i32", "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32",
             "bucket_thread_startbit_u32", "bucket_bit_base_i64")
    tensors = (int4_values_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
               bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
               bucket_thread_startbit_u32, bucket_bit_base_i64)
    for t, nm in zip(tensors, names):
        _check_cuda_contig(t, nm)
    _check_bucket_common(int4_values_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
                         bucket_thread_startbit_u32, bucket_bit_base_i64, "int4_values_u8", 16)
    n, m, max_len = int(n), int(m), int(max_len)
    if max_len <= 0 or max_len > 15:
        raise ValueError("max_len must be in [1,15]")
    if max_len != 11:
        raise ValueError("AWQ bucket decode kernel is specialized: max_len must be 11")
    if n <= 0 or m <= 0:
        raise ValueError("n,m must be > 0")
    if int4_values_u8.numel() != n * m:
        raise ValueError("int4_values_u8 numel must equal n*m")
    B = int(bucket_table_i32.size(0))
    k = _check_rect(bucket_col_start_i32, bucket_col_len_i32, bucket_row_offsets_i32, row_indices_i32,
                    bucket_thread_startbit_u32, bucket_bit_base_i64, B)
    _check_tables(decode_syms_u16, decode_lens_u8, 11)
    dev = _same_device(tensors)
    out = torch.empty((n, m), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        ws = _workspace(dev)
        rc = _lib.load().mps_decode_awq_int4_bucket(
            int4_values_u8.data_ptr(), bitstream_u64.data_ptr(), bitstream_u64.numel(), decode_syms_u16.data_ptr(),
            decode_lens_u8.data_ptr(), decode_syms_u16.size(0), bucket_table_i32.data_ptr(),
            bucket_col_start_i32.data_ptr(), bucket_col_len_i32.data_ptr(), bucket_row_offsets_i32.data_ptr(),
            row_indices_i32.data_ptr(), row_indices_i32.numel(), bucket_thread_startbit_u32.data_ptr(),
            bucket_bit_base_i64.data_ptr(), B, k, n, m, max_len, out.data_ptr(), ws.data_ptr(),
            ws.numel() * 4, _stream_ptr(dev))
    _lib.check(rc)
    return out


def huffman_decode_awq_int4_bucket_by_scale(int4_values_u8, bitstream_u64, decode_syms_u16, decode_lens_u8,
                                            bucket_table_i32, bucket_group_offsets_i32, group_rows_i32,
                                            group_col_start_i32, bucket_thread_startbit_u32, bucket_bit_base_i64,
                                            n, m, max_len, group_size):
    """AWQ-INT4 ragged buckets -> BF16 ``[n, m]`` (wrapper.cpp:371-416, decode_huffman.cu:760-875)."""
    names = ("int4_values_u8", "bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32",
             "bucket_group_offsets_i32", "group_rows_i32", "group_col_start_i32", "bucket_thread_startbit_u32",
             "bucket_bit_base_i64")
    tensors = (int4_values_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
               bucket_group_offsets_i32, group_rows_i32, group_col_start_i32, bucket_thread_startbit_u32,
               bucket_bit_base_i64)
    for t, nm in zip(tensors, names):
        _check_cuda_contig(t, nm)
    if int4_values_u8.dim() != 2:
        raise ValueError("int4_values_u8 must be uint8 2D CUDA [n,m]")
    _check_bucket_common(int4_values_u8, bitstream_u64, decode_syms_u16, decode_lens_u8, bucket_table_i32,
                         bucket_thread_startbit_u32, bucket_bit_base_i64, "int4_values_u8", 16)
    for t, nm in ((bucket_group_offsets_i32, "bucket_group_offsets_i32"), (group_rows_i32, "group_rows_i32"),
                  (group_col_start_i32, "group_col_start_i32")):
        if t.dtype != torch.int32 or t.dim() != 1:
            raise ValueError(f"{nm} must be int32 1D CUDA")
    n, m, max_len, group_size = int(n), int(m), int(max_len), int(group_size)
    if max_len <= 0 or max_len > 15:
        raise ValueError("max_len must be in [1,15]")
    if max_len != 11:
        raise ValueError("AWQ ragged bucket decode kernel is specialized: max_len must be 11")
    if n <= 0 or m <= 0:
        raise ValueError("n,m must be > 0")
    if group_size <= 0 or group_size > m:
        raise ValueError("group_size must be in (0,m]")
    if int4_values_u8.numel() != n * m:
        raise ValueError("int4_values_u8 numel must equal n*m")
    B = int(bucket_table_i32.size(0))
    if bucket_group_offsets_i32.numel() != B + 1:
        raise ValueError("bucket_group_offsets_i32 length must be B+1")
    if bucket_thread_startbit_u32.size(0) != B:
        raise ValueError("bucket_thread_startbit_u32 first dim must be B")
    if bucket_bit_base_i64.numel() != B + 1:
        raise ValueError("bucket_bit_base_i64 length must be B+1")
    if group_rows_i32.numel() != group_col_start_i32.numel():
        raise ValueError("group_rows_i32 and group_col_start_i32 length must match")
    _check_tables(decode_syms_u16, decode_lens_u8, 11)
    k = int(bucket_thread_startbit_u32.size(1)) - 1
    if k <= 0 or k > 1024:
        raise ValueError("bucket_thread_startbit_u32 has invalid k (must be 1..1024)")
    dev = _same_device(tensors)
    out = torch.empty((n, m), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        ws = _workspace(dev)
        rc = _lib.load().mps_decode_awq_int4_bucket_by_scale(
            int4_values_u8.data_ptr(), bitstream_u64.data_ptr(), bitstream_u64.numel(), decode_syms_u16.data_ptr(),
            decode_lens_u8.data_ptr(), decode_syms_u16.size(0), bucket_table_i32.data_ptr(),
            bucket_group_offsets_i32.data_ptr(), group_rows_i32.data_ptr(), group_col_start_i32.data_ptr(),
            group_rows_i32.numel(), bucket_thread_startbit_u32.data_ptr(), bucket_bit_base_i64.data_ptr(), B, k, n, m,
            max_len, group_size, out.data_ptr(), ws.data_ptr(), ws.numel() * 4, _stream_ptr(dev))
    _lib.check(rc)
    return out


def huffman_decode_awq_shared_table(bitstream_u64, decode_syms_i16, decode_nbits_u8, scale_bit_base_i64,
                                    chunk_startbit_rel_u32, chunk_out_base_u32, chunk_meta_u32, chunk_scale_id_i32,
                                    out_idx_i32, stream_chunk_ofs_i64, stream_chunk_ids_i32, out_len, max_len=11):
    """AWQ shared-table chunks -> int16 ``[out_len]`` BF16 bit patterns
    (wrapper.cpp:212-255, decode_huffman_encode_only.cu:279-383)."""
    names = ("bitstream_u64", "decode_syms_i16", "decode_nbits_u8", "scale_bit_base_i64", "chunk_startbit_rel_u32",
             "chunk_out_base_u32", "chunk_meta_u32", "chunk_scale_id_i32", "out_idx_i32", "stream_chunk_ofs_i64",
             "stream_chunk_ids_i32")
    tensors = (bitstream_u64, decode_syms_i16, decode_nbits_u8, scale_bit_base_i64, chunk_startbit_rel_u32,
               chunk_out_base_u32, chunk_meta_u32, chunk_scale_id_i32, out_idx_i32, stream_chunk_ofs_i64,
               stream_chunk_ids_i32)
    for t, nm in zip(tensors, names):
        _check_cuda_contig(t, nm)
    if stream_chunk_ofs_i64.dtype != torch.int64 or stream_chunk_ofs_i64.dim() != 1:
        raise ValueError("stream_chunk_ofs_i64 must be int64 1D (CUDA)")
    if stream_chunk_ids_i32.dtype != torch.int32 or stream_chunk_ids_i32.dim() != 1:
        raise ValueError("stream_chunk_ids_i32 must be int32 1D (CUDA)")
    expect = ((bitstream_u64, torch.uint64), (decode_syms_i16, torch.int16), (decode_nbits_u8, torch.uint8),
              (scale_bit_base_i64, torch.int64), (chunk_startbit_rel_u32, torch.uint32),
              (chunk_out_base_u32, torch.uint32), (chunk_meta_u32, torch.uint32), (chunk_scale_id_i32, torch.int32),
              (out_idx_i32, torch.int32))
    for (t, dt), nm in zip(expect, names):
        if t.dtype != dt:
            raise ValueError(f"{nm} must be {dt}")
    L, out_len = int(max_len), int(out_len)
    if L <= 0 or L > 20:
        raise ValueError("max_len must be in (0,20]")
    if decode_syms_i16.dim() != 2 or decode_syms_i16.size(1) != (1 << L):
        raise ValueError("decode table second dim must be 2^max_len")
    num_streams = int(decode_syms_i16.size(0))
    if stream_chunk_ofs_i64.numel() != num_streams + 1:
        raise ValueError("stream_chunk_ofs_i64 must have length num_streams+1")
    if stream_chunk_ids_i32.numel() != chunk_meta_u32.numel():
        raise ValueError("stream_chunk_ids_i32 must have length num_chunks")
    dev = _same_device(tensors)
    out = torch.empty((max(out_len, 0),), dtype=torch.int16, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().mps_decode_awq_shared_table(
            bitstream_u64.data_ptr(), bitstream_u64.numel(), decode_syms_i16.data_ptr(), decode_nbits_u8.data_ptr(),
            num_streams, scale_bit_base_i64.data_ptr(), scale_bit_base_i64.numel(), chunk_startbit_rel_u32.data_ptr(),
            chunk_out_base_u32.data_ptr(), chunk_meta_u32.data_ptr(), chunk_scale_id_i32.data_ptr(),
            chunk_meta_u32.numel(), out_idx_i32.data_ptr(), stream_chunk_ofs_i64.data_ptr(),
            stream_chunk_ids_i32.data_ptr(), out_len, L, out.data_ptr(), _stream_ptr(dev))
    _lib.check(rc)
    return out


# ----------------------------------------------------------------------------------------------
# build (encode)
# ----------------------------------------------------------------------------------------------

def huffman_build_fp8_decode_tables(bf16_params, fp8_params, scales, max_len=12, threads_per_block=256):
    """Builds the FP8 sidecar (wrapper.cpp:419-454, build_huffman.cu:292-969)."""
    from . import encoder

    return encoder.build_fp8(bf16_params, fp8_params, scales, int(max_len), int(threads_per_block))


def build_fp8_fine_substreams(bf16_params, fp8_params, scales, max_len=7, substreams=4096):
    """The FP8 sidecar with up to MAX_SUBSTREAMS sub-streams per bucket: the same seventeen artifacts as
    ``huffman_build_fp8_decode_tables``, byte for byte what that call would write if the reference's
    limit of 1024 (build_huffman.cu:313) were lifted, with ``bucket_thread_startbit_u32`` of shape
    ``[B, substreams + 1]``.  No counterpart in the reference, whose decoder refuses such a sidecar
    (decode_huffman.cu:695); ``huffman_decode_fp8`` and ``BucketDecodePlan`` of this module read it.

    What it is for: a weight of few buckets (a per-tensor scale gives 128-row buckets: 32 for a
    4096 x 4096 weight) has only ``B * k`` independent chains of symbols; at k = 1024 they fill a
    quarter of a B200's decode slots and the call is bound by the latency of one chain.  Four times the
    sub-streams cost 4 KB of start offsets per bucket more and cut that call from 54 to 34 microseconds.
    A weight with per-channel scales has chains enough at 1024 and only pays for the longer rows."""
    from . import encoder

    return encoder.build_fp8(bf16_params, fp8_params, scales, int(max_len), int(substreams), limit=MAX_SUBSTREAMS)


def huffman_build_awq_int4_bucket_decode_tables(bf16_params, int4_values_u8, scales_u16, max_len=11,
                                                threads_per_block=256):
    """Builds the AWQ rectangular-bucket sidecar (wrapper.cpp:258-288, build_huffman.cu:1582-2126)."""
    from . import encoder

    return encoder.build_awq_bucket(bf16_params, int4_values_u8, scales_u16, int(max_len), int(threads_per_block))


def huffman_build_awq_int4_bucket_decode_tables_by_scale(bf16_values, int4_values, scales_u16, max_len=11,
                                                         threads=256, group_cap=1024):
    """Builds the AWQ ragged-bucket sidecar (wrapper.cpp:290-321, build_huffman.cu:1074-1580)."""
    from . import encoder

    return encoder.build_awq_by_scale(bf16_values, int4_values, scales_u16, int(max_len), int(threads),
                                      int(group_cap))


def huffman_build_awq_decode_tables(bf16_params, int4_values_u8, scales_u16, max_len=11):
    """Builds the AWQ shared-table sidecar (wrapper.cpp:182-209, build_huffman.cu:2157-2633)."""
    from . import encoder

    return encoder.build_awq_shared(bf16_params, int4_values_u8, scales_u16, int(max_len))


# ----------------------------------------------------------------------------------------------
# whole-model decode in one launch
# ----------------------------------------------------------------------------------------------

_DECODE_KEYS = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_col_start_i32",
                "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32", "bucket_thread_startbit_u32",
                "bucket_bit_base_i64")


class BucketDecodePlan:
    """Decode many FP8-compressed tensors with ONE persistent-kernel launch.

    The reference decodes weight by weight (scripts/mpserve_vllm_fp8_huffman.py:526-543); a model
    has hundreds of small and large weights, so a single launch that feeds every SM from one work
    queue removes the per-launch tails.  ``entries`` is a list of ``(ctx_u8 [n,m], artifacts dict,
    out bf16 [n,m] or None)`` with all tensors already on the device; outputs are allocated when
    None.  ``decode()`` is asynchronous on the current stream.
    """

    def __init__(self, entries, mode: int = 0):
        lib = _lib.load()
        if not entries:
            raise ValueError("no tensors to decode")
        self.mode = int(mode)
        self.device = entries[0][0].device
        self.outputs: list[torch.Tensor] = []
        self._keep = []
        descs = (_lib.BucketTensor * len(entries))()
        outs: list = [None] * len(entries)
        # widest buckets first: the work queue hands out items in descriptor order, and finishing with
        # the small items keeps the tail of the launch short
        order = sorted(range(len(entries)), key=lambda j: (-int(entries[j][0].shape[1]), -int(entries[j][0].shape[0])))
        for i, j in enumerate(order):
            ctx, art, out = entries[j]
            n, m = int(ctx.shape[0]), int(ctx.shape[1])
            if out is None:
                out = torch.empty((n, m), dtype=torch.bfloat16, device=self.device)
            elif (not out.is_cuda or out.device != self.device or not out.is_contiguous() or out.element_size() != 2
                  or out.numel() != n * m):
                raise ValueError("an output must be a contiguous 16-bit CUDA tensor of n*m elements on the plan's device "
                                 "(a row range of a larger row-major tensor qualifies)")
            outs[j] = out
            self._keep.append((ctx, art))
            d = descs[i]
            d.ctx_bytes = ctx.data_ptr()
            d.bitstream = art["bitstream_u64"].data_ptr()
            d.bitstream_words = art["bitstream_u64"].numel()
            d.decode_syms = art["decode_syms_u16"].data_ptr()
            d.decode_lens = art["decode_lens_u8"].data_ptr()
            d.num_tables = art["decode_syms_u16"].size(0)
            d.bucket_table = art["bucket_table_i32"].data_ptr()
            if self.mode == 2:
                d.bucket_row_offsets = art["bucket_group_offsets_i32"].data_ptr()
                d.row_indices = art["group_rows_i32"].data_ptr()
                d.group_col_start = art["group_col_start_i32"].data_ptr()
                d.num_rows = art["group_rows_i32"].numel()
                d.group_size = int(art["group_size"])
            else:
                d.bucket_col_start = art["bucket_col_start_i32"].data_ptr()
                d.bucket_col_len = art["bucket_col_len_i32"].data_ptr()
                d.bucket_row_offsets = art["bucket_row_offsets_i32"].data_ptr()
                d.row_indices = art["row_indices_i32"].data_ptr()
                d.num_rows = art["row_indices_i32"].numel()
            d.thread_startbit = art["bucket_thread_startbit_u32"].data_ptr()
            d.bucket_bit_base = art["bucket_bit_base_i64"].data_ptr()
            d.num_buckets = art["bucket_table_i32"].size(0)
            d.k = int(art["bucket_thread_startbit_u32"].size(1)) - 1
            d.mode = self.mode
            d.n, d.m = n, m
            d.out = out.data_ptr()
        self.outputs = outs  # in the caller's order
        count = len(entries)
        prefix = (C.c_int64 * (count + 1))()
        threads, chains = C.c_int32(0), C.c_int32(0)
        _lib.check(lib.mps_bucket_batch_plan(descs, count, prefix, C.byref(threads), C.byref(chains)))
        self.count, self.threads, self.chains = count, int(threads.value), int(chains.value)
        self.total_items = int(prefix[count])
        # tensors of tiny buckets get no work items in the shared launch: each is decoded on its own
        self._descs_host = descs
        self._direct = [i for i in range(count) if prefix[i + 1] == prefix[i] and descs[i].num_buckets > 0]
        raw = torch.frombuffer(bytearray(bytes(descs)), dtype=torch.uint8)
        self._descs_dev = raw.to(self.device)
        self._prefix_dev = torch.tensor(list(prefix), dtype=torch.int64).to(self.device)

    def decode(self) -> list[torch.Tensor]:
        with torch.cuda.device(self.device):
            ws = _workspace(self.device)
            lib = _lib.load()
            stream = _stream_ptr(self.device)
            if self.total_items > 0:
                _lib.check(lib.mps_decode_bucket_batch(
                    self._descs_dev.data_ptr(), self._prefix_dev.data_ptr(), self.count, self.total_items, self.threads,
                    self.chains, self.mode, ws.data_ptr(), ws.numel() * 4, stream))
            for i in self._direct:
                _lib.check(lib.mps_decode_bucket_tensor(C.byref(self._descs_host[i]), ws.data_ptr(), ws.numel() * 4, stream))
        return self.outputs


def checksum_u16(t: torch.Tensor, acc: torch.Tensor | None = None) -> torch.Tensor:
    """Device checksum of a decoded tensor's 16-bit patterns: ``int64[2]`` = (sum mod 2^64, xor fold).
    Accumulates into ``acc`` when given (the sum adds and the fold xors across tensors)."""
    if not t.is_cuda or not t.is_contiguous() or t.element_size() != 2:
        raise ValueError("checksum_u16 needs a contiguous CUDA tensor of 16-bit elements")
    if acc is None:
        acc = torch.zeros(2, dtype=torch.int64, device=t.device)
    with torch.cuda.device(t.device):
        rc = _lib.load().mps_checksum_u16(t.data_ptr(), t.numel(), acc.data_ptr(), _stream_ptr(t.device))
    _lib.check(rc)
    return acc
