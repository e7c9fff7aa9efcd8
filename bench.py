#!/usr/bin/env python
"""Benchmark of the hot path: FP8 checkpoint + Huffman sidecar -> BF16 weights on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload model|single|sizes|awq] [--layers L]

``--workload model`` (the default, what the round-end driver runs).  One "step" decompresses every
linear weight of the workload once (one persistent-kernel launch per rank).  N=1: Llama-3-8B-shaped
random-init weights, per-channel FP8-E4M3 scales (all 32 layers, 224 tensors, 6.98 G elements).  N>1
(launched by torchrun, one rank per GPU): Llama-3-70B-shaped weights, all 80 layers, tensor-parallel
sharded N ways, each rank decoding only its own shards (the total work is fixed, so ``scaling`` is
"strong"; ``--layers`` shortens the model for quick runs).  There is no collective in the timed
region; NCCL only reduces the timings and, afterwards, the checksum of all ranks' outputs.

``--workload single | sizes | awq`` (N=1) time one tensor per call through the per-tensor entry
points the reference's plugin calls: a lone 4096x4096 weight with a per-tensor scale; single tensors
from 64 KB to 1 GB of output, N(0, 0.02) and Student-t(4); the Llama-3-8B linears as INT4 (group 128)
in the three AWQ sidecar layouts.  L2 is flushed before every timed call.

Rank 0 prints ONE JSON line.  ``value`` is decompressed BF16 GB/s (2*n*m bytes per tensor) with
compressed inputs resident in HBM; ``e2e`` includes the host->device copy of the compressed inputs
from pinned memory and the read-back of the checksum; ``dropin`` is the same step made of one
``MPServe_cuda.huffman_decode_fp8`` call per weight, each returning a fresh tensor, as the
reference's plugin does.  ``--impl reference`` times the CPU decode of the same format on all host
cores of rank 0 (the other ranks exit).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from mpserve_b200 import workloads as wl  # noqa: E402

METRIC = "decompressed_bf16_gbps"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch divided by its elements, from the ncu
# capture summarised in profiles/ (traffic grows in proportion to the elements of a launch)
NCU_TRAFFIC_BYTES_PER_ELEMENT = 3.942
E2E_MAX_PINNED_BYTES = 24 << 30   # pinned host memory one rank may take for the end-to-end leg, at most
E2E_PINNED_SHARE = 0.35           # ... and all ranks of the box together this share of the memory that is free

DECODE_KEYS = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_col_start_i32",
               "bucket_col_len_i32", "bucket_row_offsets_i32", "row_indices_i32", "bucket_thread_startbit_u32",
               "bucket_bit_base_i64")
SHARED_KEYS = ("bitstream_u64", "decode_syms_i16", "decode_nbits_u8", "scale_bit_base_i64", "chunk_startbit_rel_u32",
               "chunk_out_base_u32", "chunk_meta_u32", "chunk_scale_id_i32", "out_idx_i32", "stream_chunk_ofs_i64",
               "stream_chunk_ids_i32")
BYSCALE_KEYS = ("bitstream_u64", "decode_syms_u16", "decode_lens_u8", "bucket_table_i32", "bucket_group_offsets_i32",
                "group_rows_i32", "group_col_start_i32", "bucket_thread_startbit_u32", "bucket_bit_base_i64")
SIZES = [(128, 256), (256, 512), (512, 1024), (1024, 2048), (2048, 4096), (4096, 4096), (8192, 8192), (16384, 8192),
         (16384, 16384), (32768, 16384)]     # 64 KB ... 1 GB of BF16


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def pinned_allowance(local_world: int) -> int:
    """Bytes of pinned host memory one rank may take: a share of what the box has free, split over its ranks."""
    free = None
    try:
        for ln in open("/proc/meminfo"):
            if ln.startswith("MemAvailable:"):
                free = int(ln.split()[1]) * 1024
                break
    except OSError:
        pass
    if free is None:
        return 4 << 30
    return int(min(E2E_MAX_PINNED_BYTES, E2E_PINNED_SHARE * free / max(1, local_world)))


def bind_near_gpu(local_rank: int):
    """Keep this rank's threads on the CPUs of its GPU's NUMA node (pinned copies and launches then stay off the
    inter-socket link).  Returns what was done, for the JSON line; does nothing on a single-node host."""
    try:
        props = torch.cuda.get_device_properties(local_rank)
        base = Path(f"/sys/bus/pci/devices/{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0")
        node = int((base / "numa_node").read_text())
        nodes = [p for p in Path("/sys/devices/system/node").glob("node[0-9]*")]
        if node < 0 or len(nodes) < 2:
            return {"numa_node": node, "numa_nodes": len(nodes), "bound": False}
        cpus = set()
        for part in (base / "local_cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return {"numa_node": node, "numa_nodes": len(nodes), "bound": False}
        os.sched_setaffinity(0, cpus)
        return {"numa_node": node, "numa_nodes": len(nodes), "bound": True, "cpus": len(cpus)}
    except Exception as e:  # noqa: BLE001 - best effort: a box without sysfs entries runs unbound
        return {"bound": False, "why": type(e).__name__}


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback"


def cpu_model() -> str:
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


# ------------------------------------------------------------------------------------------------
# workload
# ------------------------------------------------------------------------------------------------

def workload_for(n_gpus: int, layers_override: int | None):
    if n_gpus == 1:
        cfg, tp, name = wl.LLAMA3_8B, 1, "llama3-8b-shaped"
    else:
        cfg, tp, name = wl.LLAMA3_70B, n_gpus, "llama3-70b-shaped"
    layers = cfg["layers"]
    if layers_override:
        layers = min(layers, layers_override)
    return cfg, tp, name, layers


def workload_text(wname, tp, layers) -> str:
    return f"{wname} fp8-e4m3 per-channel + huffman sidecar (L=7,k=1024), tp={tp}, layers={layers}"


def encode_layer_cpu(cfg, tp, rank, seed_base):
    """One decoder layer's shards of this rank, quantised and encoded on the host by the CPU
    restatement of the reference encoder (setup only, never timed as part of the GPU arm)."""
    from oracle import oracle as orc

    out = []
    for i, (name, n, m) in enumerate(wl.layer_linears(cfg)):
        sn, sm = wl.tp_shard_shape(name, n, m, tp)
        w = wl.random_weight(sn, sm, seed_base + 1000 * rank + i, "normal")
        c = wl.quantize_fp8(w, "channel")
        art = orc.build_fp8(c.bf16.view(torch.uint16).numpy(), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, 1024)
        out.append((name, sn, sm, c, art))
    return out


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------

class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception as e:  # nvidia-smi absent: report no clocks rather than fail the bench
            log("clock sampling unavailable:", e)

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU legs: decode by the C port of the decode kernel (the reference has no CPU decoder), encode by the
# reference's own CPU encoder where it was compiled
# ------------------------------------------------------------------------------------------------

def cpu_decode_sample(layer, repeats: int):
    """Decode one layer's tensors `repeats` times with the CPU port; returns (GB/s of BF16, seconds)."""
    from oracle import oracle as orc

    outs = [np.zeros((n, m), dtype=np.uint16) for _, n, m, _, _ in layer]
    t0 = time.perf_counter()
    for _ in range(repeats):
        for (_, n, m, c, art), o in zip(layer, outs):
            orc.decode_fp8(c.fp8_u8.numpy(), art, n, m, out=o)
    dt = time.perf_counter() - t0
    nbytes = repeats * sum(2 * n * m for _, n, m, _, _ in layer)
    for (_, n, m, c, _), o in zip(layer, outs):
        assert np.array_equal(o, c.bf16.view(torch.uint16).numpy()), "CPU port decode mismatch"
    return nbytes / dt / 1e9, dt


def _ref_encode_worker(job):
    """(child process) encode one tensor with the reference's CPU encoder; returns (elements, seconds)."""
    n, m, seed = job
    torch.set_num_threads(1)
    from oracle import ref_encoder as ref

    c = wl.quantize_fp8(wl.random_weight(n, m, seed, "normal"), "channel")
    t0 = time.perf_counter()
    ref.build_fp8(c.bf16, c.fp8_u8, c.scales_u16, 7, 1024)
    return n * m, time.perf_counter() - t0


def cpu_encode_baseline(cfg, seed: int) -> dict | None:
    """The reference's own encoder (kernel/build_huffman.cu:292-969, single-threaded by construction): one
    thread on two tensors of a layer, then one process per tensor of a whole layer."""
    from oracle import ref_encoder as ref

    if not ref.available():
        return None
    import multiprocessing as mp

    linears = wl.layer_linears(cfg)
    small = [(n, m, seed + i) for i, (_, n, m) in enumerate(linears[:2])]      # q and k projections
    e1 = t1 = 0.0
    for job in small:
        e, t = _ref_encode_worker(job)
        e1 += e; t1 += t
    jobs = [(n, m, seed + i) for i, (_, n, m) in enumerate(linears)]
    procs = min(len(jobs), os.cpu_count() or 1)
    t0 = time.perf_counter()
    with mp.get_context("spawn").Pool(procs) as pool:
        res = pool.map(_ref_encode_worker, jobs)
    wall = time.perf_counter() - t0
    return {"kind": "reference", "what": "kernel/build_huffman.cu huffman_build_fp8_decode_tables_entry, per-channel scales, "
                                         "max_len=7, threads_per_block=1024",
            "one_thread": {"value": e1 / t1 / 1e6, "unit": "M elements/s", "cores": 1,
                           "sample": f"{len(small)} tensors ({e1 / 1e6:.0f} M elements) in {t1:.1f}s"},
            "processes": {"value": sum(e for e, _ in res) / wall / 1e6, "unit": "M elements/s", "cores": procs,
                          "sample": f"one decoder layer, {len(jobs)} tensors ({sum(e for e, _ in res) / 1e6:.0f} M elements), one "
                                    f"process each, {wall:.1f}s wall (process start-up included)"}}


def run_reference(args, rank, world):
    from oracle import oracle as orc

    if rank != 0:
        return
    cores = os.cpu_count() or 1
    orc.set_num_threads(cores)   # not what a launcher exported: torchrun sets OMP_NUM_THREADS=1
    cores = orc.num_threads()
    if args.workload == "build":
        enc = cpu_encode_baseline(wl.LLAMA3_8B, args.seed)
        if enc is None:
            print(json.dumps({"impl": "reference", "unavailable": "the reference's encoder is not built here (oracle/build_ref.sh)"}))
            return
        print(json.dumps({"impl": "reference", "metric": "sidecar_build_melem_per_s", "value": enc["processes"]["value"],
                          "unit": "M elements/s", "n_gpus": args.gpus, "higher_is_better": True, "dtype": "u16",
                          "data": "synthetic", "config": {"workload": enc["what"], "cpu": cpu_model()},
                          "cpu_baseline": {"value": enc["processes"]["value"], "unit": "M elements/s", "kind": "reference",
                                           "cores": enc["processes"]["cores"], "sample": enc["processes"]["sample"]},
                          "one_thread": enc["one_thread"],
                          "e2e": {"value": enc["processes"]["value"], "unit": "M elements/s", "h2d_bytes_per_step": 0,
                                  "d2h_bytes_per_step": 0}, "gpu_launches": 0}), flush=True)
        return
    if args.workload == "layer":
        print(json.dumps({"impl": "reference", "unavailable": "the layer workload times GEMMs on the GPU; the reference's CPU side "
                                                               "has no counterpart (its call sequence is leg (a) of our arm)"}), flush=True)
        return
    if args.workload != "model":
        return run_reference_cases(args, cores)
    cfg, tp, wname, layers = workload_for(args.gpus, args.layers)
    layer = encode_layer_cpu(cfg, tp, 0, args.seed)
    for _ in range(args.warmup):
        cpu_decode_sample(layer, 1)
    times, nbytes = [], sum(2 * n * m for _, n, m, _, _ in layer)
    for _ in range(args.steps):
        _, dt = cpu_decode_sample(layer, 1)
        times.append(dt)
    ms = 1e3 * float(np.mean(times))
    value = nbytes / (ms / 1e3) / 1e9
    sample = (f"one decoder layer of rank 0 ({len(layer)} tensors, {nbytes / 2 / 1e6:.0f} M elements) per step, all host "
              f"threads of this process; a rate, independent of the GPU count")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": workload_text(wname, tp, layers),
                   "note": "the reference has no CPU decoder; this is the CPU port of its decode kernel "
                           "(ESC honoured), OpenMP over buckets x sub-streams; bounded sample per step",
                   "cpu": cpu_model()},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm, whole model
# ------------------------------------------------------------------------------------------------

def encode_layer_gpu(cfg, tp, rank, seed_base, layer, dev):
    """One decoder layer's shards of this rank: random-init weights, FP8 quantisation and the sidecar,
    all made on the GPU with this library's own builder (setup, outside every timed region)."""
    import MPServe_cuda

    out = []
    for i, (name, n, m) in enumerate(wl.layer_linears(cfg)):
        sn, sm = wl.tp_shard_shape(name, n, m, tp)
        w = wl.random_weight(sn, sm, seed_base + 100003 * layer + 1000 * rank + i, "normal", device=dev)
        c = wl.quantize_fp8(w, "channel")
        art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7,
                                                           threads_per_block=1024)
        out.append((name, sn, sm, c, art))
    return out


def run_ours(args, rank, world, local_rank):
    import MPServe_cuda
    from mpserve_b200 import _lib, api, shard

    _lib.load()  # no fallback: a missing extension is an error
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    # (a lone rank stays unbound: its CPU baseline is meant to use every core of the box)
    host_binding = bind_near_gpu(local_rank) if world > 1 else {"bound": False, "why": "single rank"}
    pinned_cap = pinned_allowance(int(os.environ.get("LOCAL_WORLD_SIZE", world)))
    cfg, tp, wname, layers = workload_for(args.gpus, args.layers)
    # what a rank holds: compressed inputs (~1.75 B/element) and BF16 outputs; shorten the model rather than
    # run out of device memory, and say so in config.workload
    per_layer = sum(wl.tp_shard_shape(nm, n, m, tp)[0] * wl.tp_shard_shape(nm, n, m, tp)[1] for nm, n, m in wl.layer_linears(cfg))
    budget = 0.85 * torch.cuda.get_device_properties(dev).total_memory - (14 << 30)
    fit = int(budget // (per_layer * 3.8))
    if fit < layers:
        log(f"[rank {rank}] {layers} layers need more than this GPU's memory; running {fit}")
        layers = max(1, fit)

    # Layer by layer: generate, quantise, encode, pack the compressed inputs into one device buffer (with a
    # pinned host twin for the end-to-end leg, as a loader would hold them), decode, compare with the source
    # bit for bit, drop the source.
    t_setup = time.perf_counter()
    entries, layer_entries, layer_bufs, shapes = [], [], [], []
    alg_bytes = n_elem = h2d_bytes = 0
    want = torch.zeros(2, dtype=torch.int64, device=dev)     # checksum of the source tensors
    layer0_host = None
    pinned = 0
    for li in range(layers):
        layer = encode_layer_gpu(cfg, tp, rank, args.seed, li, dev)
        if li == 0 and rank == 0 and world == 1:
            layer0_host = [(name, n, m, wl.Fp8Case(c.bf16.cpu(), c.fp8_u8.cpu(), c.scales_u16.cpu()),
                            {k: v.cpu().numpy() for k, v in art.items()}) for name, n, m, c, art in layer]
        arrays = []
        for name, n, m, c, art in layer:
            arrays.append(c.fp8_u8)
            arrays.extend(art[k] for k in DECODE_KEYS)
        offs, total = [], 0
        for a in arrays:
            offs.append(total)
            total += (a.numel() * a.element_size() + 255) // 256 * 256
        flat = torch.empty(total, dtype=torch.uint8, device=dev)
        views = []
        for a, o in zip(arrays, offs):
            v = flat[o:o + a.numel() * a.element_size()].view(a.dtype).view(a.shape)
            v.copy_(a)
            views.append(v)
        it = iter(views)
        these = []
        out_flat = torch.empty(sum(n * m for _, n, m, _, _ in layer), dtype=torch.bfloat16, device=dev)   # the layer's outputs
        o0 = 0
        for name, n, m, c, art in layer:
            ctx = next(it)
            d = {k: next(it) for k in DECODE_KEYS}
            these.append((ctx, d, out_flat[o0:o0 + n * m].view(n, m)))
            o0 += n * m
            alg_bytes += n * m + sum(v.numel() * v.element_size() for v in d.values()) + 2 * n * m
            n_elem += n * m
            shapes.append((n, m))
        lp = api.BucketDecodePlan(these, mode=0)
        lp.decode()
        for (name, n, m, c, art), (_, _, out) in zip(layer, these):
            assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16)), f"decode mismatch in layer {li} {name}"
            api.checksum_u16(c.bf16, want)
        host = None
        if pinned + total <= pinned_cap:
            host = torch.empty(total, dtype=torch.uint8, pin_memory=True)
            host.copy_(flat)
            pinned += total
            h2d_bytes += total
        entries.extend(these)
        layer_entries.append((these, lp, out_flat))
        layer_bufs.append((flat, host))
        del layer, arrays, views
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    enc_s = time.perf_counter() - t_setup
    log(f"[rank {rank}] generated, quantised, encoded and verified {layers} layers ({n_elem / 1e9:.2f} G elements) in {enc_s:.1f}s")

    plan = api.BucketDecodePlan(entries, mode=0)     # the whole model in one launch, same buffers and outputs
    out_bytes = 2 * n_elem
    plan.decode()
    torch.cuda.synchronize()
    assert not api.decode_timed_out(dev), "a bounded wait ran out in the verification decode"

    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist

    def barrier():
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ------------------------------------------------------------
    for _ in range(args.warmup):
        plan.decode()
    # clocks are sampled from before an untimed pre-roll of the same launches (so that the sampler,
    # whose period is ~100 ms, sees the load of the short timed region) until after a post-roll
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()

    def roll(seconds):
        t_stop = time.perf_counter() + seconds
        while time.perf_counter() < t_stop:
            for _ in range(4):
                plan.decode()
            torch.cuda.synchronize()

    roll(0.6)
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for a, b in evs:
        a.record()
        plan.decode()
        b.record()
    t_end.record()
    torch.cuda.synchronize()
    roll(0.3)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    assert not api.decode_timed_out(dev), "a bounded wait ran out in the timed region"
    total_ms = t_begin.elapsed_time(t_end)
    kernel_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))
    t = torch.tensor([total_ms, kernel_ms], dtype=torch.float64, device=dev)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kernel_ms_max = float(t[0]), float(t[1])
    ms_per_step = total_ms / args.steps

    # ---- the same step through the drop-in per-tensor entry: one call per weight, a fresh tensor each -------
    dropin = None
    if not args.no_dropin:
        calls = [(ctx, [d[k] for k in DECODE_KEYS], n, m) for (ctx, d, _), (n, m) in zip(entries, shapes)]

        def dropin_step():
            outs = None
            for ctx, a, n, m in calls:
                outs = MPServe_cuda.huffman_decode_fp8(ctx, *a, n, m, 7)   # the previous result is released, as in a forward
            return outs

        for _ in range(2):
            dropin_step()
        barrier()
        d_steps = max(1, min(args.steps, 5))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        e0.record()
        for _ in range(d_steps):
            dropin_step()
        e1.record()
        host_issue_ms = 1e3 * (time.perf_counter() - w0) / d_steps
        barrier()
        d_ms = e0.elapsed_time(e1) / d_steps
        t = torch.tensor([d_ms], dtype=torch.float64, device=dev)
        if use_dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        d_ms = float(t[0])
        dropin = {"value": world * out_bytes / (d_ms / 1e3) / 1e9, "unit": UNIT, "ms_per_step": d_ms,
                  "calls_per_step": len(calls), "host_issue_ms_per_step": host_issue_ms, "steps": d_steps,
                  "how": "MPServe_cuda.huffman_decode_fp8 once per weight, inputs resident, a newly allocated output per "
                         "call (kernel/wrapper.cpp:457-503 semantics), device time of the whole step"}

    # ---- end to end: pinned host -> device copy of the compressed inputs, decode, checksum back ------
    # Layer i is decoded (and check-summed) on the compute stream while layer i+1 crosses PCIe on the copy
    # stream.  Layers whose inputs did not fit the pinned-memory allowance are left out of this leg.
    e2e_layers = [(flat, host, lp, out_flat) for (flat, host), (these, lp, out_flat) in zip(layer_bufs, layer_entries)
                  if host is not None]
    e2e_out_bytes = sum(2 * out_flat.numel() for _, _, _, out_flat in e2e_layers)
    e2e_want = torch.zeros(2, dtype=torch.int64, device=dev)   # what a step must read back: from the verified outputs
    for _, _, _, out_flat in e2e_layers:
        api.checksum_u16(out_flat, e2e_want)
    e2e_want = e2e_want.cpu()
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    acc = torch.zeros(2, dtype=torch.int64, device=dev)
    e2e_steps = max(1, min(args.steps, 3))

    def e2e_step():
        acc.zero_()
        copy_stream.wait_stream(main_stream)   # the previous step's decodes have read the buffers
        for flat_dev, flat_host, lp, out_flat in e2e_layers:
            with torch.cuda.stream(copy_stream):
                flat_dev.copy_(flat_host, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            main_stream.wait_event(ev)
            lp.decode()
            api.checksum_u16(out_flat, acc)     # the layer's outputs are one buffer: one launch
        return acc.cpu()

    assert torch.equal(e2e_step(), e2e_want), "the end-to-end step read back another checksum than the verified outputs give"
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_got = e2e_step()
    e1.record()
    barrier()
    assert not api.decode_timed_out(dev), "a bounded wait ran out in the end-to-end leg"
    assert torch.equal(e2e_got, e2e_want), "the end-to-end step read back another checksum than the verified outputs give"
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0])
    e2e_launches = e2e_steps * 2 * len(e2e_layers)

    # ---- checksum of all ranks' outputs (outside every timed region; NCCL when there are several ranks) ----
    got = torch.zeros(2, dtype=torch.int64, device=dev)
    for _, _, o in entries:
        api.checksum_u16(o, got)
    got_host, want_host = got.cpu(), want.cpu()
    mine = (int(got_host[0]) & shard.MASK64, int(got_host[1]) & shard.MASK64)
    expect = (int(want_host[0]) & shard.MASK64, int(want_host[1]) & shard.MASK64)
    assert mine == expect, f"checksum mismatch on rank {rank}: {mine} != {expect}"
    all_got = shard.all_reduce_checksum(mine, device=dev)
    all_want = shard.all_reduce_checksum(expect, device=dev)
    assert all_got == all_want, "all-reduced checksum mismatch"

    if rank != 0:
        return
    peak, peak_src = hbm_peak()
    achieved = alg_bytes / (kernel_ms_max / 1e3) / 1e9
    value = world * out_bytes / (ms_per_step / 1e3) / 1e9
    e2e_value = world * e2e_out_bytes / (e2e_ms / 1e3) / 1e9

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as orc

        orc.set_num_threads(os.cpu_count() or 1)
        cores = orc.num_threads()
        cpu_decode_sample(layer0_host, 1)
        one, dt1 = cpu_decode_sample(layer0_host, 1)
        reps = int(max(1, min(200, 12.0 / max(dt1, 1e-3))))   # about 12 s of CPU work
        gbs, dt = cpu_decode_sample(layer0_host, reps)
        cpu_baseline = {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "cpu": cpu_model(),
                        "sample": f"one decoder layer ({len(layer0_host)} tensors) decoded {reps}x in {dt:.1f}s by the CPU "
                                  f"port of the reference decode kernel, OpenMP, {cores} threads",
                        "encode": cpu_encode_baseline(cfg, args.seed),
                        "encode_gpu": {"value": n_elem / enc_s / 1e6, "unit": "M elements/s",
                                       "what": "this library's builder on the GPU, weight generation, quantisation, packing "
                                               "and verification included"}}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
        "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {
            "workload": workload_text(wname, tp, layers),
            "tensors_per_rank": len(entries), "elements_per_rank": n_elem,
            "l2": "inputs+outputs per step far exceed L2 (no flush needed)",
            "inputs": "every layer random-init with its own seed, quantised and encoded on the GPU by this library's builder",
            "decode": f"one launch per step, threads={plan.threads}, chains={plan.chains}",
        },
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_nominal_8000_gbs": achieved / 8000.0,
                     "traffic": NCU_TRAFFIC_BYTES_PER_ELEMENT * n_elem,
                     "traffic_source": "ncu capture of a smaller launch, scaled by elements", "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": kernel_ms_max},
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 16,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "gpu_launches": e2e_launches, "layers": len(e2e_layers),
                "how": "per layer: one pinned-host -> device copy of its packed compressed inputs on a copy stream, "
                       "then one decode launch and one checksum launch on the compute stream; 16 bytes read back per step "
                       "and compared with the checksum of the verified outputs"
                       + ("" if len(e2e_layers) == layers else
                          f"; {len(e2e_layers)} of {layers} layers (pinned-memory allowance), a rate over those")},
        "dropin": dropin,
        "gpu_launches": args.steps,
        "clocks": clocks,
        "host": {"cpus": os.cpu_count(), "binding": host_binding, "pinned_allowance_bytes": pinned_cap},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# single tensors through the per-tensor entry points (configs 1, 3, 4)
# ------------------------------------------------------------------------------------------------

def _time_calls(fn, flush, reps: int):
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


def _e2e_call(inputs_dev, run, out_of, reps: int):
    """Milliseconds of: copy every compressed input from pinned host memory, decode, checksum, read 16 bytes back."""
    from mpserve_b200 import api

    hosts = [t.cpu().pin_memory() for t in inputs_dev]
    acc = torch.zeros(2, dtype=torch.int64, device=inputs_dev[0].device)

    def step():
        acc.zero_()
        for d, h in zip(inputs_dev, hosts):
            d.copy_(h, non_blocking=True)
        api.checksum_u16(out_of(run()), acc)
        return acc.cpu()

    step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        step()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps, sum(h.numel() * h.element_size() for h in hosts)


def _case_result(label, n, m, art, keys, ctx_bytes, med, best, e2e_ms, h2d, host_us):
    elems = n * m
    alg = ctx_bytes + sum(art[k].numel() * art[k].element_size() for k in keys) + 2 * elems
    return {"case": label, "elements": elems, "ms_median": med, "ms_best": best, "bf16_gbps": 2 * elems / med / 1e6,
            "algorithmic_bytes": alg, "algorithmic_gbps": alg / med / 1e6, "e2e_ms": e2e_ms, "h2d_bytes": h2d,
            "host_us_per_call": host_us, "code_bits_per_element": 64.0 * art["bitstream_u64"].numel() / elems}


def _host_us(fn, reps=50):
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    dt = time.perf_counter() - t0
    torch.cuda.synchronize()
    return 1e6 * dt / reps


def fp8_case(n, m, dist, scale_mode, k, seed, dev, flush, reps):
    import MPServe_cuda

    c = wl.quantize_fp8(wl.random_weight(n, m, seed, dist, device=dev), scale_mode)
    if k <= 1024:
        art = MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=k)
    else:   # more sub-streams per bucket than the reference builds or decodes: this library's extension of the format
        from mpserve_b200 import api

        art = api.build_fp8_fine_substreams(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, substreams=k)
    a = [art[key] for key in DECODE_KEYS]

    def run():
        return MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *a, n, m, 7)

    out = run()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16)), "decode mismatch"
    med, best = _time_calls(run, flush, reps)
    e2e_ms, h2d = _e2e_call([c.fp8_u8] + a, run, lambda o: o, max(3, reps // 3))
    note = "" if k <= 1024 else " (fine sub-streams: not a reference sidecar)"
    r = _case_result(f"fp8 {scale_mode} {dist} {n}x{m} k={k}{note}", n, m, art, DECODE_KEYS, n * m, med, best, e2e_ms, h2d,
                     _host_us(run))
    r.update(buckets=int(art["bucket_table_i32"].size(0)), tables=int(art["decode_syms_u16"].size(0)))
    return r, (c, art)


def awq_case(name, n, m, layout, k, seed, dev, flush, reps):
    import MPServe_cuda

    c = wl.quantize_awq(wl.random_weight(n, m, seed, "normal", device=dev), 128)
    if layout == "bucket":
        art = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables(c.bf16, c.int4_u8, c.scales_u16, max_len=11,
                                                                       threads_per_block=k)
        keys = DECODE_KEYS
        a = [art[key] for key in keys]

        def run():
            return MPServe_cuda.huffman_decode_awq_int4_bucket(c.int4_u8, *a, n, m, 11)
    elif layout == "shared":
        art = MPServe_cuda.huffman_build_awq_decode_tables(c.bf16, c.int4_u8, c.scales_u16, max_len=11)
        keys = SHARED_KEYS
        a = [art[key] for key in keys]

        def run():
            return MPServe_cuda.huffman_decode_awq_shared_table(*a, n * m, 11).view(torch.bfloat16).view(n, m)
    else:
        art = MPServe_cuda.huffman_build_awq_int4_bucket_decode_tables_by_scale(c.bf16, c.int4_u8, c.scales_u16, max_len=11,
                                                                                threads=k, group_cap=1024)
        keys = BYSCALE_KEYS
        a = [art[key] for key in keys]
        gs = int(art["shape_nmkg_i64"][3])

        def run():
            return MPServe_cuda.huffman_decode_awq_int4_bucket_by_scale(c.int4_u8, *a, n, m, 11, gs)

    out = run()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16)), "decode mismatch"
    med, best = _time_calls(run, flush, reps)
    inputs = a if layout == "shared" else [c.int4_u8] + a      # the shared layout reads no int4 codes
    e2e_ms, h2d = _e2e_call(inputs, run, lambda o: o, max(2, reps // 5))
    r = _case_result(f"awq g128 {layout} {name} {n}x{m} k={k}", n, m, art, keys, 0 if layout == "shared" else n * m, med,
                     best, e2e_ms, h2d, _host_us(run, 20))
    return r, None


def case_list(args):
    """(label of the workload, list of case constructors) for --workload single | sizes | awq."""
    k = args.k
    if args.workload == "single":
        ks = [k] if k else [1024, 256, 4096]   # 4096: finer sub-streams than the reference's format allows
        return ("single linear weight 4096x4096, N(0,0.02), per-tensor FP8-E4M3 scale, huffman sidecar (L=7), one "
                "MPServe_cuda.huffman_decode_fp8 call",
                [("fp8", dict(n=4096, m=4096, dist="normal", scale_mode="tensor", k=kk, seed=7)) for kk in ks])
    if args.workload == "sizes":
        cases = []
        for dist in ("normal", "student_t"):
            for n, m in SIZES:
                if 2 * n * m <= args.max_bytes:
                    cases.append(("fp8", dict(n=n, m=m, dist=dist, scale_mode="channel", k=k or 1024, seed=11)))
        return ("single tensors of 64 KB ... 1 GB of BF16, N(0,0.02) and Student-t(4)x0.02, per-channel FP8-E4M3 scales, "
                "huffman sidecar (L=7,k=1024), one call per tensor", cases)
    cases = []
    for layout in ("byscale", "bucket", "shared"):
        for i, (name, n, m) in enumerate(wl.layer_linears(wl.LLAMA3_8B)):
            if layout == "shared" and i not in (0, 1):
                continue   # one square and one small tensor: the format's metadata is ~20 B per element
            cases.append(("awq", dict(name=name, n=n, m=m, layout=layout, k=k or 256, seed=100 + i)))
    return ("llama3-8b-shaped linears as INT4 AWQ (group 128, fp16 scales), huffman sidecar (L=11) in the by-scale, "
            "rectangular and shared-table layouts, one call per tensor", cases)


def run_cases(args, local_rank):
    from mpserve_b200 import _lib, api

    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    label, cases = case_list(args)
    reps = max(5, args.steps)
    sampler = ClockSampler(local_rank)
    sampler.start()
    rows, first = [], None
    for kind, kw in cases:
        r, keep = (fp8_case if kind == "fp8" else awq_case)(dev=dev, flush=flush, reps=reps, **kw)
        rows.append(r)
        if first is None:
            first = keep
        log(json.dumps(r))
        torch.cuda.empty_cache()
    clocks = sampler.stop()
    assert not api.decode_timed_out(dev), "a bounded wait ran out"
    peak, peak_src = hbm_peak()
    head = rows[0]     # the line's headline is its first case; every case is listed under "cases"
    cpu_baseline = None
    if not args.no_cpu_baseline and first is not None:
        from oracle import oracle as orc

        orc.set_num_threads(os.cpu_count() or 1)
        c, art = first
        n, m = int(c.fp8_u8.shape[0]), int(c.fp8_u8.shape[1])
        host = [("t", n, m, wl.Fp8Case(c.bf16.cpu(), c.fp8_u8.cpu(), c.scales_u16.cpu()),
                 {key: v.cpu().numpy() for key, v in art.items()})]
        cpu_decode_sample(host, 1)
        _, dt1 = cpu_decode_sample(host, 1)
        reps_cpu = int(max(1, min(500, 10.0 / max(dt1, 1e-3))))
        gbs, dt = cpu_decode_sample(host, reps_cpu)
        cpu_baseline = {"value": gbs, "unit": UNIT, "cores": orc.num_threads(), "kind": "port", "cpu": cpu_model(),
                        "sample": f"{head['case']} decoded {reps_cpu}x in {dt:.1f}s by the CPU port of the reference decode "
                                  "kernel, OpenMP"}
    line = {
        "metric": METRIC, "value": head["bf16_gbps"], "unit": UNIT, "n_gpus": 1, "steps": reps, "warmup": 3,
        "ms_per_step": head["ms_median"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u16", "data": "synthetic",
        "config": {"workload": label, "headline_case": head["case"],
                   "l2": "a 256 MB buffer is written before every timed call"},
        "roofline": {"bound": "hbm", "achieved": head["algorithmic_gbps"], "peak": peak, "unit": "GB/s",
                     "frac": head["algorithmic_gbps"] / peak, "frac_of_nominal_8000_gbs": head["algorithmic_gbps"] / 8000.0,
                     "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": head["algorithmic_bytes"], "kernel_ms": head["ms_median"]},
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": 2 * head["elements"] / head["e2e_ms"] / 1e6, "unit": UNIT, "h2d_bytes_per_step": head["h2d_bytes"],
                "d2h_bytes_per_step": 16, "ms_per_step": head["e2e_ms"],
                "how": "per call: every compressed input copied from pinned host memory, one decode call, checksum, 16 "
                       "bytes read back"},
        "gpu_launches": reps,
        "cases": rows,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# the sidecar builder on its own (the offline half of the path)
# ------------------------------------------------------------------------------------------------

def run_build(args, local_rank):
    """One gate/up-sized weight of the 8B-shaped model (14336 x 4096, per-channel scales) through
    MPServe_cuda.huffman_build_fp8_decode_tables, inputs resident, artifacts left on the device."""
    import MPServe_cuda
    from mpserve_b200 import _lib

    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    n, m = 14336, 4096
    c = wl.quantize_fp8(wl.random_weight(n, m, args.seed, "normal", device=dev), "channel")

    def step():
        return MPServe_cuda.huffman_build_fp8_decode_tables(c.bf16, c.fp8_u8, c.scales_u16, max_len=7, threads_per_block=1024)

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        art = step()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        art = step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    clocks = sampler.stop()
    out = MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *[art[k] for k in DECODE_KEYS], n, m, 7)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint16), c.bf16.view(torch.uint16)), "the built sidecar does not decode to the source"
    ms = float(np.median(times))
    art_bytes = sum(v.numel() * v.element_size() for v in art.values() if isinstance(v, torch.Tensor))
    alg = 3 * n * m + 2 * c.scales_u16.numel() + art_bytes      # read BF16 + FP8 + scales once, write the artifacts once
    peak, peak_src = hbm_peak()
    cpu_baseline = None
    if not args.no_cpu_baseline:
        cpu_baseline = cpu_encode_baseline(wl.LLAMA3_8B, args.seed)
    line = {
        "metric": "sidecar_build_melem_per_s", "value": n * m / ms / 1e3, "unit": "M elements/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u16", "data": "synthetic",
        "config": {"workload": f"sidecar build of one {n}x{m} weight, N(0,0.02), per-channel FP8-E4M3 scales, L=7, k=1024",
                   "l2": "inputs and scratch of one build (hundreds of MB) exceed L2"},
        "roofline": {"bound": "hbm", "achieved": alg / (ms / 1e3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": alg / (ms / 1e3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": alg, "kernel_ms": ms,
                     "note": "a build is some forty launches and three host synchronisations; the time is that of the whole call"},
        "cpu_baseline": cpu_baseline,
        "artifact_bytes": art_bytes, "tables": int(art["decode_syms_u16"].shape[0]), "buckets": int(art["bucket_table_i32"].shape[0]),
        "gpu_launches": None,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# one decoder layer as a serving plugin uses it: decode the weights, multiply
# ------------------------------------------------------------------------------------------------

def run_layer(args, local_rank):
    """One 8B-shaped decoder layer, weights decoded for every forward and fed to the layer's four GEMMs (16 tokens).
    (a) the reference plugin's call sequence (scripts/mpserve_vllm_fp8_huffman.py:419, 474-489, 526-543, 657-661): one
    ``huffman_decode_fp8`` per shard into a fresh tensor, ``torch.cat`` of q/k/v and of gate/up, ``torch.matmul``;
    (b) the same through ``mpserve_b200.sidecar.FusedDecoder``: one launch into persistent fused weights, no cat."""
    import MPServe_cuda
    from mpserve_b200 import _lib
    from mpserve_b200.sidecar import FusedDecoder

    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    cfg = wl.LLAMA3_8B
    layer = {name: (n, m, c, art) for name, n, m, c, art in encode_layer_gpu(cfg, 1, 0, args.seed, 0, dev)}
    tokens = 16
    x_h = torch.randn(tokens, cfg["hidden"], device=dev, dtype=torch.bfloat16)
    x_q = torch.randn(tokens, cfg["q_heads"] * cfg["head_dim"], device=dev, dtype=torch.bfloat16)
    x_i = torch.randn(tokens, cfg["inter"], device=dev, dtype=torch.bfloat16)
    fused = [["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], ["self_attn.o_proj"],
             ["mlp.gate_proj", "mlp.up_proj"], ["mlp.down_proj"]]
    acts = [x_h, x_q, x_h, x_i]

    def one(name):
        n, m, c, art = layer[name]
        return MPServe_cuda.huffman_decode_fp8(c.fp8_u8, *[art[k] for k in DECODE_KEYS], n, m, 7)

    def plugin_step():
        outs = []
        for names, x in zip(fused, acts):
            parts = [one(nm) for nm in names]
            w = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
            outs.append(torch.matmul(x, w.t()))
        return outs

    dec = FusedDecoder([[(layer[nm][2].fp8_u8, {k: layer[nm][3][k] for k in DECODE_KEYS}) for nm in names] for names in fused])

    def fused_step():
        ws = dec.decode()
        return [torch.matmul(x, w.t()) for x, w in zip(acts, ws)]

    a, b = plugin_step(), fused_step()
    torch.cuda.synchronize()
    for u, v in zip(a, b):
        assert torch.equal(u, v), "the fused layer's outputs differ from the plugin sequence's"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    reps = max(10, args.steps)
    res = {}
    for label, fn in (("plugin_sequence", plugin_step), ("fused_decoder", fused_step)):
        med, best = _time_calls(fn, flush, reps)
        res[label] = {"ms_median": med, "ms_best": best, "host_us": _host_us(fn, 20)}
    clocks = sampler.stop()
    elems = sum(n * m for n, m, _, _ in layer.values())
    med = res["fused_decoder"]["ms_median"]
    print(json.dumps({
        "metric": METRIC, "value": 2 * elems / med / 1e6, "unit": UNIT, "n_gpus": 1, "steps": reps, "warmup": 3,
        "ms_per_step": med, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16",
        "data": "synthetic",
        "config": {"workload": f"one llama3-8b-shaped decoder layer: decode 7 weights ({elems / 1e6:.0f} M elements) + 4 GEMMs of "
                               f"{tokens} tokens, per forward", "l2": "a 256 MB buffer is written before every timed forward"},
        "layer": res, "gpu_launches": None, "clocks": clocks}), flush=True)


def run_reference_cases(args, cores):
    """CPU port on the first case of the workload (FP8 workloads), a bounded number of repetitions per step."""
    from oracle import oracle as orc

    label, cases = case_list(args)
    kind, kw = cases[0]
    if kind != "fp8":
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm times the FP8 decode port only"}), flush=True)
        return
    n, m = kw["n"], kw["m"]
    c = wl.quantize_fp8(wl.random_weight(n, m, kw["seed"], kw["dist"]), kw["scale_mode"])
    art = orc.build_fp8(c.bf16.view(torch.uint16).numpy(), c.fp8_u8.numpy(), c.scales_u16.numpy(), 7, kw["k"])
    layer = [("t", n, m, c, art)]
    for _ in range(args.warmup):
        cpu_decode_sample(layer, 1)
    times = [cpu_decode_sample(layer, 1)[1] for _ in range(args.steps)]
    ms = 1e3 * float(np.mean(times))
    value = 2 * n * m / (ms / 1e3) / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u16", "data": "synthetic",
            "config": {"workload": label, "headline_case": f"fp8 {kw['scale_mode']} {kw['dist']} {n}x{m} k={kw['k']}",
                       "cpu": cpu_model()},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": "the headline case once per step, all host threads"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    line["reference_cuda_kernel"] = reference_cuda_timing(c, art, n, m, max(5, args.steps))
    print(json.dumps(line), flush=True)


def reference_cuda_timing(c, art_host, n, m, reps):
    """The reference's own CUDA decode kernel (kernel/decode_huffman.cu, unmodified, built under oracle/_ref)
    on the same sidecar, where a GPU is present and the kernel handles the sidecar (no ESC tables, no bitstream
    of 3072..10240 words, no bucket narrower than its sub-stream count): for context beside the CPU number."""
    from oracle import ref_decoder as refdec

    if not torch.cuda.is_available():
        return {"unavailable": "no GPU"}
    if not refdec.available():
        return {"unavailable": "oracle/_ref holds no build of the reference decoder (oracle/build_ref_decode.sh)"}
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    art = {k: torch.from_numpy(v).to(dev) for k, v in art_host.items() if isinstance(v, np.ndarray)}
    why = refdec.refusal(art, n, m)
    if why is not None:
        return {"unavailable": f"not given to the reference kernel: {why}"}
    ctx = c.fp8_u8.to(dev)
    args_ = [art[k] for k in refdec.ORDER]
    mod = refdec.module()
    out = mod.huffman_decode_fp8(ctx, *args_, n, m, 7)
    torch.cuda.synchronize()
    if not torch.equal(out.view(torch.uint16), c.bf16.to(dev).view(torch.uint16)):
        return {"unavailable": "the reference kernel's output differs from the source tensor"}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    med, best = _time_calls(lambda: mod.huffman_decode_fp8(ctx, *args_, n, m, 7), flush, reps)
    return {"ms_median": med, "ms_best": best, "bf16_gbps": 2 * n * m / med / 1e6,
            "what": "huffman_decode_fp8_entry of kernel/decode_huffman.cu:591-758 built for sm_100a, one call per step, "
                    "L2 flushed before every call, CUDA events"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="model", choices=["model", "single", "sizes", "awq", "build", "layer"])
    ap.add_argument("--layers", type=int, default=None, help="shorten the model to this many layers (quicker)")
    ap.add_argument("--k", type=int, default=None, help="sub-streams per bucket for the single-tensor workloads")
    ap.add_argument("--max-bytes", type=int, default=1 << 30, help="largest BF16 output of --workload sizes")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-dropin", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)  # timing hygiene: never fewer than three warm-up steps

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "build":
        if rank == 0:
            run_build(args, local_rank)
        return
    if args.workload == "layer":
        if rank == 0:
            run_layer(args, local_rank)
        return
    if args.workload != "model":
        if rank == 0:
            run_cases(args, local_rank)
        return
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
