"""Partitioning of a model's compressed weights across the GPUs of one box, and the checksum that
ranks all-reduce after decoding.

The hot path has no collective: every weight (or tensor-parallel shard of a weight) is an
independent unit that is encoded on its own, so rank r decodes only its own list.  The reference
refuses tensor parallelism (scripts/mpserve_vllm_fp8_huffman.py:165-168); the split used here is the
one vLLM's linears use: column-parallel layers (q, k, v, gate, up) split rows, row-parallel layers
(o, down) split columns, each shard made contiguous before it is encoded.
"""
from __future__ import annotations

import numpy as np
import torch

from . import workloads as wl

MASK64 = (1 << 64) - 1


def shard_of(name: str, w: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """This rank's contiguous tensor-parallel shard of weight `w` ([n, m])."""
    n, m = w.shape
    if name.endswith(("o_proj", "down_proj")):
        step = m // tp
        return w[:, rank * step:(rank + 1) * step].contiguous()
    step = n // tp
    return w[rank * step:(rank + 1) * step].contiguous()


def rank_tensors(cfg: dict, tp: int, layers: int | None = None) -> list[tuple[str, int, int]]:
    """(name, n, m) of every shard a rank decodes under tensor parallelism of degree `tp`."""
    return list(wl.model_tensors(cfg, tp, layers))


def layers_of_rank(n_layers: int, world: int, rank: int) -> range:
    """Alternative split for models that fit one GPU: whole layers, contiguous blocks per rank."""
    per, extra = divmod(n_layers, world)
    start = rank * per + min(rank, extra)
    return range(start, start + per + (1 if rank < extra else 0))


def checksum_host(bits: np.ndarray) -> tuple[int, int]:
    """Same checksum as the device kernel (mps_checksum_u16): (sum of the 16-bit patterns mod 2^64,
    xor over i of pattern[i] * (i + 1) mod 2^64)."""
    a = np.ascontiguousarray(bits).reshape(-1).astype(np.uint64)
    s = int(a.sum(dtype=np.uint64))
    x = int(np.bitwise_xor.reduce(a * (np.arange(a.size, dtype=np.uint64) + np.uint64(1)))) if a.size else 0
    return s & MASK64, x & MASK64


def combine(acc: tuple[int, int], other: tuple[int, int]) -> tuple[int, int]:
    return (acc[0] + other[0]) & MASK64, acc[1] ^ other[1]


def all_reduce_checksum(local: tuple[int, int], device=None) -> tuple[int, int]:
    """Reduce per-rank checksums over the default process group (NCCL on GPUs, gloo on CPU).
    The sum travels as four 16-bit limbs in int64 (exact for any realistic world size); the xor
    fold is gathered (there is no XOR reduction) and folded locally."""
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    limbs = torch.tensor([(local[0] >> (16 * i)) & 0xFFFF for i in range(4)], dtype=torch.int64, device=device)
    dist.all_reduce(limbs, op=dist.ReduceOp.SUM)
    total = sum(int(limbs[i]) << (16 * i) for i in range(4)) & MASK64
    mine = torch.tensor([local[1] & 0xFFFFFFFF, local[1] >> 32], dtype=torch.int64, device=device)
    gathered = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(gathered, mine)
    x = 0
    for g in gathered:
        x ^= int(g[0]) | (int(g[1]) << 32)
    return total, x & MASK64
