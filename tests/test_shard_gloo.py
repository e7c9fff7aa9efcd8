"""Multi-rank host logic on CPU (gloo, world_size 2): the shard partition covers the model exactly
once and the all-reduced checksum of per-rank decodes equals the single-process one."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from mpserve_b200 import shard
from mpserve_b200 import workloads as wl
from oracle import oracle as orc

TINY = dict(layers=2, hidden=64, inter=128, q_heads=4, kv_heads=2, head_dim=16, vocab=100)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _full_weight(name, n, m, li):
    return wl.random_weight(n, m, 7000 + 13 * li + sum(name.encode()) % 97, "normal")  # no str hash: it differs per process


def _rank_checksum(cfg, tp, rank):
    acc = (0, 0)
    for li in range(cfg["layers"]):
        for name, n, m in wl.layer_linears(cfg):
            w = shard.shard_of(name, _full_weight(name, n, m, li), tp, rank)
            c = wl.quantize_fp8(w, "channel")
            bits = c.bf16.view(torch.uint16).numpy()
            art = orc.build_fp8(bits, c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 64)
            dec = orc.decode_fp8(c.fp8_u8.numpy(), art, *bits.shape)
            assert np.array_equal(dec, bits)
            acc = shard.combine(acc, shard.checksum_host(dec))
    return acc


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        local = _rank_checksum(TINY, world, rank)
        total = shard.all_reduce_checksum(local)
        q.put((rank, local, total))
    finally:
        dist.destroy_process_group()


def test_tp_shards_tile_each_weight():
    for name, n, m in wl.layer_linears(TINY):
        w = _full_weight(name, n, m, 0)
        parts = [shard.shard_of(name, w, 2, r) for r in range(2)]
        dim = 1 if name.endswith(("o_proj", "down_proj")) else 0
        assert torch.equal(torch.cat(parts, dim=dim), w)
        assert tuple(parts[0].shape) == wl.tp_shard_shape(name, n, m, 2)


def test_layer_partition_is_exact():
    for world in (1, 2, 3, 8):
        seen = [li for r in range(world) for li in shard.layers_of_rank(32, world, r)]
        assert seen == list(range(32))


def test_checksum_all_reduce_two_ranks_gloo():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    locals_ = {r: loc for r, loc, _ in results}
    want = shard.combine(locals_[0], locals_[1])
    for _, _, total in results:
        assert total == want
    # the sum part is independent of how the weights were sharded: whole weights give the same sum
    whole = (0, 0)
    for li in range(TINY["layers"]):
        for name, n, m in wl.layer_linears(TINY):
            bits = _full_weight(name, n, m, li).view(torch.uint16).numpy()
            whole = shard.combine(whole, shard.checksum_host(bits))
    assert whole[0] == want[0]


# ---- per-rank sidecars: written and read back by two ranks, the shards re-assembled by the parent ------

def _sidecar_worker(rank, world, port, directory, q):
    import torch.distributed as dist

    from mpserve_b200 import sidecar

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        modules, sources = {}, {}
        for name, n, m in wl.layer_linears(TINY):
            w = shard.shard_of(name, _full_weight(name, n, m, 0), world, rank)
            c = wl.quantize_fp8(w, "channel")
            bits = c.bf16.view(torch.uint16).numpy()
            art = orc.build_fp8(bits, c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 64)
            prefix = f"model.layers.0.{name}"
            modules[prefix] = (c.fp8_u8, {k: torch.from_numpy(v) for k, v in art.items() if isinstance(v, np.ndarray)})
            sources[prefix] = bits
        sidecar.write_rank_sidecar(directory, rank, world, modules)
        dist.barrier()
        back = sidecar.read_rank_sidecar(directory, rank, world)
        assert set(back) == set(modules)
        decoded = {}
        for prefix, entry in back.items():
            n, m = entry["fp8_u8"].shape
            art = {k: v.numpy() for k, v in entry.items() if k != "fp8_u8"}
            decoded[prefix] = orc.decode_fp8(entry["fp8_u8"].numpy(), art, n, m)
            assert np.array_equal(decoded[prefix], sources[prefix])
        refusals = []
        for wrong_rank, wrong_size in ((1 - rank, world), (rank, world + 2)):
            try:
                if (wrong_rank, wrong_size) == (1 - rank, world):   # the other rank's file under this rank's name
                    other = sidecar.read_sidecar(os.path.join(directory, sidecar.rank_sidecar_name(1 - rank, world)))
                    assert set(other) == set(modules)
                    os.makedirs(os.path.join(directory, f"swap{rank}"), exist_ok=True)
                    src = os.path.join(directory, sidecar.rank_sidecar_name(1 - rank, world))
                    dst = os.path.join(directory, f"swap{rank}", sidecar.rank_sidecar_name(rank, world))
                    with open(src, "rb") as a, open(dst, "wb") as b:
                        b.write(a.read())
                    sidecar.read_rank_sidecar(os.path.join(directory, f"swap{rank}"), rank, world)
                else:
                    sidecar.read_rank_sidecar(directory, wrong_rank, wrong_size)
                refusals.append(None)
            except (ValueError, FileNotFoundError) as e:
                refusals.append(type(e).__name__)
        q.put((rank, decoded, refusals))
    finally:
        dist.destroy_process_group()


def test_rank_sidecars_two_ranks_gloo(tmp_path):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_sidecar_worker, args=(r, world, port, str(tmp_path), q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict((r, (d, ref)) for r, d, ref in (q.get(timeout=180) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        # a file written for the other rank, and a layout nobody wrote, are both refused at load time
        assert results[r][1] == ["ValueError", "FileNotFoundError"]
    for name, n, m in wl.layer_linears(TINY):
        prefix = f"model.layers.0.{name}"
        dim = 1 if name.endswith(("o_proj", "down_proj")) else 0
        whole = np.concatenate([results[r][0][prefix] for r in range(world)], axis=dim)
        assert np.array_equal(whole, _full_weight(name, n, m, 0).view(torch.uint16).numpy())
