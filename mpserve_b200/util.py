"""Small host-side helpers shared by the benchmark, the smoke entry and the tests."""
from __future__ import annotations

import numpy as np
import torch


def to_torch(a) -> torch.Tensor:
    """numpy array (any of the sidecar dtypes, unsigned included) or tensor -> CPU tensor."""
    if isinstance(a, torch.Tensor):
        return a
    return torch.from_numpy(np.ascontiguousarray(a))


def artifacts_to_device(art: dict, device, pin: bool = False) -> dict:
    """Move every array of a sidecar dict to `device`, keeping dtypes (uint16/uint32/uint64 as is)."""
    out = {}
    for k, v in art.items():
        if isinstance(v, (np.ndarray, torch.Tensor)):
            t = to_torch(v)
            if pin and t.device.type == "cpu":
                t = t.pin_memory()
            out[k] = t.to(device, non_blocking=pin)
        else:
            out[k] = v
    return out


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    """BF16 tensor -> numpy uint16 bit patterns (CPU copy)."""
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


def decode_fp8_args(ctx_dev: torch.Tensor, art: dict, n: int, m: int, max_len: int = 7):
    """Positional argument tuple of huffman_decode_fp8 from a device-resident sidecar dict."""
    return (ctx_dev, art["bitstream_u64"], art["decode_syms_u16"], art["decode_lens_u8"], art["bucket_table_i32"],
            art["bucket_col_start_i32"], art["bucket_col_len_i32"], art["bucket_row_offsets_i32"],
            art["row_indices_i32"], art["bucket_thread_startbit_u32"], art["bucket_bit_base_i64"], n, m, max_len)
