#!/usr/bin/env python
"""Benchmark of the hot path: the uneven collectives and the synthesized SPMD training step.

    python bench.py --gpus 1 --steps K --warmup W            # 8 virtual ranks on one GPU (HBM bound)
    torchrun --nproc-per-node N ... bench.py --gpus N ...    # one rank per GPU over NVLink (N = 2, 4, 8)
    python bench.py --impl reference ...                     # the CPU port of the reference on gloo ranks

The default run prints ONE JSON line on rank 0 with three parts:

* the collective micro-benchmark (the line's ``metric`` / ``value``): a step = one uneven all_gather +
  one reduce_scatter + one all_reduce of a (256, C) fp32 tensor of ``--size-mib`` MiB split on dim 0 by
  the ratios [.22,.18,.15,.13,.11,.09,.07,.05]; ``value`` is the nccl-tests style bus bandwidth of the
  step (bus bytes = S(W-1)/W + S(W-1)/W + 2S(W-1)/W), summed over the GPUs of the job;
* ``parity``: outside every timed region, the drop-in ``hap_b200.collectives`` functions (and the list
  API on one GPU) on small seeded tensors, both ordinary torch tensors (staged) and heap-resident
  ones, checked against the CPU oracle;
* ``spmd_step``: samples/s of the Transformer-LM training step (plan dp_zero, the whole iteration
  replayed from a CUDA graph), with its tensor roofline and its own end-to-end figure.

``--workload gemm|lm|ops`` and ``--sweep`` run the individual studies.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# a collective that gets stuck in a benchmark should fail in seconds, not after the library's ten minutes
os.environ.setdefault("HAPX_TIMEOUT_MS", "30000")

R8 = [.22, .18, .15, .13, .11, .09, .07, .05]
ROWS = 256
NVLINK_NOMINAL_GBS = 900.0      # per direction per GPU


def ratios_for(world):
    r = R8[:world]
    s = sum(r)
    return [x / s for x in r]


def bus_bytes(S, W):
    return 4.0 * S * (W - 1) / W


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


# ----------------------------------------------------------------------------------------------
# CPU arm: the gloo port of the reference's collectives on the host cores
# ----------------------------------------------------------------------------------------------
def _cpu_worker(rank, world, store, size_bytes, steps, warmup, threads, out_path):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import gloo_port as gp
    from oracle.sharding_round import sharding_round
    torch.set_num_threads(max(1, threads))
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}")
    cols = size_bytes // (ROWS * 4)
    L = sharding_round(ROWS, ratios_for(world))
    g = torch.Generator().manual_seed(1000 + rank)
    shard = torch.randn(L[rank], cols, generator=g)
    full = torch.randn(ROWS, cols, generator=g)
    times = []
    for it in range(warmup + steps):
        dist.barrier()
        t0 = time.perf_counter()
        gp.all_gather(shard, 0, L, rank)
        gp.reduce_scatter(full, 0, L, rank)
        gp.all_reduce(full)
        dist.barrier()
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(times, f)
    dist.destroy_process_group()


def run_cpu_arm(world, size_bytes, steps, warmup):
    import torch.multiprocessing as mp
    cores = os.cpu_count() or 1
    threads = max(1, cores // world)
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "times.json")
        mp.spawn(_cpu_worker, args=(world, os.path.join(d, "store"), size_bytes, steps, warmup, threads, out),
                 nprocs=world, join=True)
        times = json.load(open(out))
    mean = sum(times) / len(times)
    return {"value": bus_bytes(size_bytes, world) / mean / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{world} gloo ranks x {threads} threads, fp32 tensor of {size_bytes >> 20} MiB, "
                      f"{steps} steps after {warmup} warm-ups (padding-mode all_gather + reduce_scatter + all_reduce)",
            "ms_per_step": mean * 1e3}


# ----------------------------------------------------------------------------------------------
# clocks during the timed region (read-only NVML)
# ----------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        while not self._stop_evt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(0.02)

    def finish(self):
        self._stop_evt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def collective_config(W, size_mib, emulated):
    """The `config` of the collective micro-benchmark; the reference arm prints the same object."""
    import hap_b200
    cols = (size_mib << 20) // (ROWS * 4)
    return {"workload": f"uneven collective micro-benchmark: all_gather + reduce_scatter + all_reduce of a "
                        f"({ROWS}, {cols}) fp32 tensor ({size_mib} MiB) split on dim 0",
            "world": W, "sharding_lengths": hap_b200.sharding_round(ROWS, ratios_for(W)), "ratios": "r8 (first W renormalised)",
            "ranks": ("8 virtual ranks on ONE GPU (an emulation of the 8-GPU exchange, one cooperative launch per collective, HBM bound): "
                      "not a point of a scaling curve") if emulated else "one process per GPU, peer loads over NVLink",
            "inputs": "resident in the peer-visible heap (so is the all_reduce output)", "l2": "inputs larger than L2 (126 MB)",
            "cpu_arm": "the reference arm and cpu_baseline time a bounded sample of this workload (a smaller tensor, see cpu_baseline.sample)"}


class Job:
    """Process-wide state of one bench run: rank, device, torch.distributed (N > 1 only)."""

    def __init__(self, n_gpus):
        import torch
        self.n_gpus = n_gpus
        self.rank = int(os.environ.get("RANK", 0))
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        world_env = int(os.environ.get("WORLD_SIZE", 1))
        if n_gpus > 1 and world_env != n_gpus:
            raise SystemExit(f"--gpus {n_gpus} needs a launcher with WORLD_SIZE={n_gpus} (torchrun); got {world_env}")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if n_gpus > 1:
            import torch.distributed as dist
            dist.init_process_group("cpu:gloo,cuda:nccl", rank=self.rank, world_size=n_gpus)
            self.dist = dist

    def barrier(self):
        import torch
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, *xs):
        import torch
        if self.dist is None:
            return xs if len(xs) > 1 else xs[0]
        t = torch.tensor(list(xs), dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        out = [float(v) for v in t]
        return out if len(out) > 1 else out[0]

    def everyone(self, obj):
        """All ranks' `obj` in rank order (host transport)."""
        if self.dist is None:
            return [obj]
        got = [None] * self.n_gpus
        self.dist.all_gather_object(got, obj)
        return got

    def finish(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def run_collective_bench(args, job):
    """The collective micro-benchmark: the JSON line's metric / value / roofline / e2e."""
    import torch
    import hap_b200
    from hap_b200 import _native as N

    n_gpus, rank, dev, dist = job.n_gpus, job.rank, job.dev, job.dist
    S = args.size_mib << 20
    dtype = torch.float32
    es = 4
    cols = S // (ROWS * es)
    emulated = n_gpus == 1
    W = 8 if emulated else n_gpus
    L = hap_b200.sharding_round(ROWS, ratios_for(W))
    stage = (S + S // W + (64 << 20) + 255) // 256 * 256     # staged input + the reduced slice of all_reduce
    heap = stage + 2 * S + (max(L) * cols * es) + (64 << 20)

    if emulated:
        comm = hap_b200.local_comm(W, dev, heap_bytes=heap, stage_bytes=stage)
    else:
        comm = hap_b200.init_process_comm(heap_bytes=heap, stage_bytes=stage)
        hap_b200.collectives.set_default_comm(comm)
    ranks = comm.ranks()
    nl = comm.n_local

    # inputs resident in the peer-visible heap (read in place by the kernels)
    shards, fulls = [], []
    for i, r in enumerate(ranks):
        g = torch.Generator(dev).manual_seed(1000 + r)
        sh = comm.symm_empty((L[r], cols), dtype, i)
        sh.copy_(torch.randn(L[r], cols, device=dev, generator=g))
        fu = comm.symm_empty((ROWS, cols), dtype, i)
        fu.copy_(torch.randn(ROWS, cols, device=dev, generator=g))
        shards.append(sh)
        fulls.append(fu)
    ag_out = [torch.empty(ROWS, cols, dtype=dtype, device=dev) for _ in ranks]
    # the all_reduce result goes to a second heap tensor: with every output peer-visible the slice owners write
    # their sums straight into all outputs (torch.distributed's all_reduce, which the reference calls, is in place)
    ar_out = [comm.symm_empty((ROWS, cols), dtype, i) for i in range(nl)]
    barrier = job.barrier
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step(events=None):
        marks = [ev() for _ in range(4)] if events is not None else None
        if marks: marks[0].record()
        comm.all_gather(shards, 0, L, out=ag_out)
        if marks: marks[1].record()
        rs = comm.reduce_scatter(fulls, 0, L)
        if marks: marks[2].record()
        ar = comm.all_reduce(fulls, scale=1.0 / W, out=ar_out)
        if marks:
            marks[3].record()
            events.append(marks)
        return rs, ar

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    comm.check()
    sampler = ClockSampler(job.local_rank)
    sampler.start()
    launches0 = N.lib.hapx_launch_count()
    events = []
    t_begin, t_end = ev(), ev()
    barrier()
    t_begin.record()
    for _ in range(args.steps):
        step(events)
    t_end.record()
    barrier()
    launches = N.lib.hapx_launch_count() - launches0
    clocks = sampler.finish()
    comm.check()
    total_ms = t_begin.elapsed_time(t_end)
    op_ms = [sum(m[k].elapsed_time(m[k + 1]) for m in events) / len(events) for k in range(3)]
    total_ms = job.max_over_ranks(total_ms)
    op_ms = list(job.max_over_ranks(*op_ms))
    ms_per_step = total_ms / args.steps
    busbw = bus_bytes(S, W) / (ms_per_step * 1e-3) / 1e9

    # ---- the link's own rate: rank 0 reads rank 1's copy of the 'fulls' tensor with the copy kernel ----
    peer_copy = None
    if dist is not None:
        dst = ag_out[0]
        ts = []
        for _ in range(4):
            barrier()
            if rank == 0:
                a, b = ev(), ev()
                a.record()
                comm.get(1, fulls[0], out=dst)
                b.record()
                b.synchronize()
                ts.append(a.elapsed_time(b))
        barrier()
        peer_copy = job.max_over_ranks(S / (min(ts[1:]) * 1e-3) / 1e9 if rank == 0 else 0.0)

    # ---- end to end through the public API with host buffers --------------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    host_shards = [torch.randn(L[r], cols).pin_memory() for r in ranks]
    host_full = torch.randn(ROWS, cols).pin_memory()
    host_out = [torch.empty(L[r], cols).pin_memory() for r in ranks]
    lc = hap_b200.LocalCollectives(comm) if emulated else None

    # Every step uploads its inputs from pinned host memory and brings the reduce_scatter result back.  The copies run
    # on streams of their own: the upload of step k + 1 and the download of step k - 1 overlap with the collectives of
    # step k (PCIe is full duplex), as a caller that feeds the library from the host would arrange it.
    up_s, down_s, cur_s = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    slots = [{"sh": [torch.empty(L[r], cols, device=dev) for r in ranks], "fu": [torch.empty(ROWS, cols, device=dev) for _ in ranks],
              "up": torch.cuda.Event(), "free": torch.cuda.Event()} for _ in range(2)]

    def upload(k):
        slot = slots[k % 2]
        with torch.cuda.stream(up_s):
            up_s.wait_event(slot["free"])                 # the collectives that last read this slot are done
            for d, h in zip(slot["sh"], host_shards):
                d.copy_(h, non_blocking=True)
            for d in slot["fu"]:
                d.copy_(host_full, non_blocking=True)
            slot["up"].record(up_s)

    def e2e_step(k, last):
        slot = slots[k % 2]
        if not last:
            upload(k + 1)
        cur_s.wait_event(slot["up"])
        if emulated:
            lc.all_gather(slot["sh"], 0, L)
            rs = lc.reduce_scatter(slot["fu"], 0, L)
            lc.all_reduce(slot["fu"])
        else:
            col = hap_b200.collectives
            col.all_gather(slot["sh"][0], 0, L, rank)
            rs = [col.reduce_scatter(slot["fu"][0], 0, L, rank)]
            col.all_reduce(slot["fu"][0])
        slot["free"].record(cur_s)
        done = torch.cuda.Event()
        done.record(cur_s)
        with torch.cuda.stream(down_s):
            down_s.wait_event(done)
            for o, h in zip(rs, host_out):
                o.record_stream(down_s)
                h.copy_(o, non_blocking=True)

    def e2e_run(n):
        for sl in slots:
            sl["free"].record(cur_s)
        upload(0)
        for k in range(n):
            e2e_step(k, k == n - 1)
        cur_s.wait_stream(down_s)                         # the last result has reached the host
        cur_s.wait_stream(up_s)

    e2e_run(1)
    torch.cuda.synchronize()
    barrier()
    b0, b1 = ev(), ev()
    b0.record()
    e2e_run(e2e_steps)
    b1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = job.max_over_ranks(b0.elapsed_time(b1)) / e2e_steps
    comm.check()
    h2d = sum(h.numel() * 4 for h in host_shards) + nl * host_full.numel() * 4
    d2h = sum(h.numel() * 4 for h in host_out)
    if dist is not None:
        h2d, d2h = h2d * n_gpus, d2h * n_gpus   # whole job (every rank copies its own)
    e2e = {"value": bus_bytes(S, W) / (e2e_ms * 1e-3) / 1e9 * n_gpus, "unit": "GB/s", "h2d_bytes_per_step": int(h2d),
           "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "steps": e2e_steps,
           "api": "hap_b200.LocalCollectives" if emulated else "hap_b200.collectives (drop-in)",
           "note": "ordinary torch tensors: every call also pays the copy into the staging area",
           "pipeline": "uploads and downloads on their own streams: the next step's upload and the previous step's download overlap with this step's collectives"}

    # ---- roofline of the dominant kernel -----------------------------------------------------------
    peaks, peak_kind = measured_peaks()
    ag_ms, rs_ms, ar_ms = op_ms
    if emulated:
        # one launch serves all 8 virtual ranks: every output byte written once, every input byte read once
        # (all_gather: S in + W*S out; reduce_scatter: W*S in + S out)
        alg = (W + 1) * S
        dom = ("pull_reduce_kernel<float,float> (reduce_scatter)", rs_ms) if rs_ms >= ag_ms else ("pull_copy_kernel (all_gather)", ag_ms)
        achieved = alg / (dom[1] * 1e-3) / 1e9
        # DRAM traffic per launch from the ncu capture of the same kernels at 128 MiB (summary under profiles/:
        # reduce 1.198 GB, copy 1.152 GB for 1.208 GB algorithmic), scaled with the tensor size - it grows in
        # proportion, every byte is touched once
        ratio = 0.992 if dom[0].startswith("pull_reduce") else 0.954
        roofline = {"bound": "hbm", "kernel": dom[0], "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "peak_kind": peak_kind, "traffic": int(ratio * alg),
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum at 128 MiB, scaled by size",
                    "algorithmic_bytes_per_launch": alg, "launch_ms": dom[1]}
    else:
        s = [L[r] * cols * es for r in range(W)]
        alg = max(max(s[r] * (W - 1), S - s[r]) for r in range(W))      # busiest NVLink port, busier direction
        dom = ("pull_reduce_kernel<float,float> (reduce_scatter)", rs_ms) if rs_ms >= ag_ms else ("pull_copy_kernel (all_gather)", ag_ms)
        achieved = alg / (dom[1] * 1e-3) / 1e9
        roofline = {"bound": "nvlink", "kernel": dom[0], "achieved": achieved, "peak": NVLINK_NOMINAL_GBS, "unit": "GB/s",
                    "frac": achieved / NVLINK_NOMINAL_GBS, "peak_kind": "nominal per direction per GPU",
                    "peer_copy_GBps": peer_copy, "frac_of_peer_copy": achieved / peer_copy if peer_copy else None,
                    "peer_copy_source": "measured in this run: rank 0 reads the tensor from rank 1 with the library's copy kernel, best of 3",
                    "traffic": None, "algorithmic_bytes_per_launch": alg, "launch_ms": dom[1]}

    ops = {}
    for name, ms, bb in (("all_gather", ag_ms, S * (W - 1) / W), ("reduce_scatter", rs_ms, S * (W - 1) / W),
                         ("all_reduce", ar_ms, 2 * S * (W - 1) / W)):
        ops[name] = {"ms": ms, "busbw_GBps": bb / (ms * 1e-3) / 1e9}

    result = {
        "metric": "uneven_collective_bus_bandwidth", "value": busbw * n_gpus, "unit": "GB/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": collective_config(W, args.size_mib, emulated),
        "ops": ops, "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
    }
    # release device memory before the next leg runs
    del shards, fulls, ag_out
    hap_b200.collectives.set_default_comm(None)
    comm.destroy()
    torch.cuda.empty_cache()
    return result


def run_parity(job):
    """Outside any timed region: the public collectives on small seeded tensors against the CPU oracle.

    N > 1: the drop-in ``hap_b200.collectives`` functions (forward and autograd backward), one process per
    GPU; every rank's inputs travel over gloo so that each rank can evaluate the oracle for itself.
    N = 1: the list API on 8 virtual ranks.  Inputs are ordinary torch tensors (copied into the staging
    area by the library) in one pass and heap-resident tensors (read in place) in another.
    Gathers / re-sharding must agree bit for bit; reductions within 1e-5 (fp32) / 1e-2 (bf16) relative."""
    import torch
    import hap_b200
    from hap_b200 import collectives as col
    from oracle import collectives_math as cm

    dev, rank = job.dev, job.rank
    emulated = job.dist is None
    W = 8 if emulated else job.n_gpus
    ratios = ratios_for(W)
    comm = (hap_b200.local_comm(W, dev, heap_bytes=96 << 20, stage_bytes=32 << 20) if emulated
            else hap_b200.init_process_comm(heap_bytes=96 << 20, stage_bytes=32 << 20))
    if not emulated:
        col.set_default_comm(comm)
    mine = comm.ranks()
    stats = {"cases": 0, "failed": [], "max_rel_err": 0.0, "exact_cases": 0}
    tol = {torch.float32: 1e-5, torch.bfloat16: 1e-2}

    def gen(shape, seed, dtype):
        return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).to(dtype)

    def place(t, where, i):
        if where == "heap":
            out = comm.symm_empty(tuple(t.shape), t.dtype, i)
            out.copy_(t)
            return out
        return t.to(dev)

    def all_ranks(per_local):
        """[tensor of rank 0, ..., tensor of rank W-1] on the host, from this process's local ranks."""
        if emulated:
            return [t.detach().cpu() for t in per_local]
        return job.everyone(per_local[0].detach().cpu())

    def judge(name, got_local, want_all, exact, dtype):
        stats["cases"] += 1
        for i, r in enumerate(mine):
            got, want = got_local[i].detach().cpu(), want_all[r]
            if exact:
                ok = got.shape == want.shape and torch.equal(got, want)
            else:
                err = float((got.double() - want.double()).abs().max()) if want.numel() else 0.0
                scale = float(want.double().abs().max()) if want.numel() else 1.0
                rel = err / max(scale, 1e-30)
                stats["max_rel_err"] = max(stats["max_rel_err"], rel)
                ok = got.shape == want.shape and rel <= tol[dtype]
            if not ok:
                stats["failed"].append(f"{name} rank {r}")
        if exact:
            stats["exact_cases"] += 1

    lc = hap_b200.LocalCollectives(comm) if emulated else None
    for where in ("staged", "heap"):
        for dtype in (torch.float32, torch.bfloat16):
            for total, other, dim in ((37, 129, 0), (256, 200, 1)):
                comm.symm_reset()
                Ls = hap_b200.sharding_round(total, ratios)
                tag = f"{where}/{str(dtype)[6:]}/dim{dim}"
                shard_shape = lambda r: [Ls[r] if d == dim else other for d in range(2)]
                full_shape = [total if d == dim else other for d in range(2)]
                # all_gather, both entry points, forward + backward (the uneven reduce_scatter of the gradients)
                xs = [place(gen(shard_shape(r), 1000 + r, dtype), where, i).requires_grad_(not emulated) for i, r in enumerate(mine)]
                ws = [gen(full_shape, 2000 + r, dtype).to(dev) for r in mine]
                for fname in ("all_gather", "all_gather_by_group_call"):
                    if emulated:
                        outs = getattr(lc, fname)(xs, dim, Ls)
                    else:
                        xs[0].grad = None
                        outs = [getattr(col, fname)(xs[0], dim, Ls, rank)]
                        (outs[0] * ws[0]).sum().backward()
                    x_all = all_ranks(xs)
                    judge(f"{fname} {tag}", outs, cm.all_gather(x_all, dim, Ls), True, dtype)
                    if not emulated:
                        judge(f"{fname} backward {tag}", [xs[0].grad], cm.all_gather_backward(all_ranks(ws), dim, Ls), False, dtype)
                # reduce_scatter, both entry points, forward + backward (the uneven all_gather of the gradients)
                comm.symm_reset()
                ys = [place(gen(full_shape, 3000 + r, dtype), where, i).requires_grad_(not emulated) for i, r in enumerate(mine)]
                vs = [gen(shard_shape(r), 4000 + r, dtype).to(dev) for r in mine]
                for fname in ("reduce_scatter", "reduce_scatter_by_group_call"):
                    if emulated:
                        outs = getattr(lc, fname)(ys, dim, Ls)
                    else:
                        ys[0].grad = None
                        outs = [getattr(col, fname)(ys[0], dim, Ls, rank)]
                        (outs[0] * vs[0]).sum().backward()
                    judge(f"{fname} {tag}", outs, cm.reduce_scatter(all_ranks(ys), dim, Ls), False, dtype)
                    if not emulated:
                        judge(f"{fname} backward {tag}", [ys[0].grad], cm.reduce_scatter_backward(all_ranks(vs), dim, Ls), True, dtype)
                # all_reduce
                outs = lc.all_reduce(ys) if emulated else [col.all_reduce(ys[0].detach())]
                judge(f"all_reduce {tag}", outs, cm.all_reduce(all_ranks(ys)), False, dtype)
            # all_to_all, both orders of the two dims
            sl, cl = hap_b200.sharding_round(24, ratios), hap_b200.sharding_round(40, ratios)
            for sd, cd in ((0, 1), (1, 0)):
                comm.symm_reset()
                shp = lambda r: [sum(sl) if d == sd else (cl[r] if d == cd else 5) for d in range(3)]
                zs = [place(gen(shp(r), 7000 + r, dtype), where, i) for i, r in enumerate(mine)]
                outs = lc.all_to_all(zs, sd, cd, sl, cl) if emulated else [col.all_to_all(zs[0], sd, cd, sl, cl, rank)]
                judge(f"all_to_all {where}/{str(dtype)[6:]}/{sd}{cd}", outs, cm.all_to_all(all_ranks(zs), sd, cd, sl, cl), True, dtype)
    comm.check()
    col.set_default_comm(None)
    comm.destroy()
    failed = [f for fl in job.everyone(stats["failed"]) for f in fl]
    max_rel = job.max_over_ranks(stats["max_rel_err"])
    return {"ok": not failed, "cases": stats["cases"], "exact_cases": stats["exact_cases"], "max_rel_err": max_rel,
            "failed": failed[:8], "world": W,
            "api": "hap_b200.LocalCollectives on 8 virtual ranks" if emulated else "hap_b200.collectives (drop-in, autograd) on one process per GPU",
            "inputs": ["ordinary torch tensors (staged)", "heap-resident (read in place)"],
            "oracle": "oracle/collectives_math.py", "tolerance": {"gathers": "bit-exact", "f32": 1e-5, "bf16": 1e-2}}


def run_default(args):
    job = Job(args.gpus)
    result = run_collective_bench(args, job)
    result["parity"] = run_parity(job)
    if not args.no_spmd_step:
        result["spmd_step"] = run_lm_step(args, job)
    if job.rank == 0 and job.n_gpus == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = run_cpu_arm(8, args.cpu_size_mib << 20, args.cpu_steps, 2)
        if "spmd_step" in result:
            result["spmd_step"]["cpu_baseline"] = run_lm_cpu(2, 2, 2)
    job.finish()
    if job.rank == 0:
        print(json.dumps(result), flush=True)



# ----------------------------------------------------------------------------------------------
# size sweep of the collective micro-benchmark (1 KiB ... 1 GiB in powers of 4, fp32 and bf16,
# both entry points), next to the reference's algorithm run on NCCL on the same GPUs
# ----------------------------------------------------------------------------------------------
def run_sweep(args):
    import torch
    import hap_b200
    from hap_b200 import _native as N

    n_gpus = args.gpus
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    emulated = n_gpus == 1
    W = 8 if emulated else n_gpus
    L = hap_b200.sharding_round(ROWS, ratios_for(W))
    max_bytes = args.sweep_max_mib << 20
    stage = (max_bytes // W + (64 << 20) + 255) // 256 * 256      # all_reduce keeps its reduced slice there
    heap = stage + 2 * max_bytes + max(L) * (max_bytes // ROWS) + int(max_bytes * max(ratios_for(W)) * 1.05) + (64 << 20)
    if emulated:
        comm = hap_b200.local_comm(W, dev, heap_bytes=heap, stage_bytes=stage)
        dist = None
        gp = None
    else:
        import torch.distributed as dist
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=n_gpus)
        comm = hap_b200.init_process_comm(heap_bytes=heap, stage_bytes=stage)
        from oracle import gloo_port as gp      # the reference's algorithm; here it runs on NCCL as the on-box bar
    ranks = comm.ranks()

    def sync():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, reps, warm=5, inner=1):
        """Median / min device time of one call; `inner` calls are queued back to back between the
        two events (as nccl-tests does), so the host's launch overhead overlaps with the previous call."""
        for _ in range(warm):
            fn()
        sync()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if dist is not None:
                dist.barrier()
            a.record()
            for _ in range(inner):
                fn()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b) / inner)
        if dist is not None:
            t = torch.tensor(ts, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts = t.tolist()
        return statistics.median(ts), min(ts)

    def graphed_ms(fn, inner, reps):
        """Device time per call with the host out of the way: `inner` calls recorded into a CUDA graph and replayed."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        sync()
        comm.set_stream_ordering(True)          # forget the event of the eager calls: it must not be waited on while capturing
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(max(2, inner)):
                fn()
        comm.set_stream_ordering(True)
        sync()
        for _ in range(2):
            graph.replay()
        sync()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if dist is not None:
                dist.barrier()
            a.record()
            graph.replay()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b) / max(2, inner))
        if dist is not None:
            t = torch.tensor(ts, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts = t.tolist()
        del graph
        return statistics.median(ts)

    rows = []
    sizes = [1 << k for k in range(10, 31, 2) if (1 << k) <= max_bytes]
    for dtype, dname, es in ((torch.float32, "f32", 4), (torch.bfloat16, "bf16", 2)):
        for S in sizes:
            cols = S // (ROWS * es)
            if cols < 1:
                continue
            comm.symm_reset()
            shards, fulls = [], []
            for i, r in enumerate(ranks):
                g = torch.Generator(dev).manual_seed(1000 + r)
                sh = comm.symm_empty((L[r], cols), dtype, i)
                sh.copy_(torch.randn(L[r], cols, device=dev, generator=g).to(dtype))
                fu = comm.symm_empty((ROWS, cols), dtype, i)
                fu.copy_(torch.randn(ROWS, cols, device=dev, generator=g).to(dtype))
                shards.append(sh)
                fulls.append(fu)
            out = [torch.empty(ROWS, cols, dtype=dtype, device=dev) for _ in ranks]
            ar_heap = [comm.symm_empty((ROWS, cols), dtype, i) for i in range(len(ranks))]
            reps = (20 if S <= (256 << 20) else 5) if not args.sweep_quick else (8 if S <= (256 << 20) else 3)
            inner = 10 if S <= (64 << 20) else 2
            s_r = [L[r] * cols * es for r in range(W)]
            alg_ag = max(max(s_r[r] * (W - 1), S - s_r[r]) for r in range(W))
            cases = [
                ("all_gather", lambda: comm.all_gather(shards, 0, L, N.MODE_PADDING, out=out), S * (W - 1) / W, alg_ag),
                ("all_gather_by_group_call", lambda: comm.all_gather(shards, 0, L, N.MODE_GROUP_CALL, out=out), S * (W - 1) / W, alg_ag),
                ("reduce_scatter", lambda: comm.reduce_scatter(fulls, 0, L, N.MODE_PADDING), S * (W - 1) / W, alg_ag),
                ("reduce_scatter_by_group_call", lambda: comm.reduce_scatter(fulls, 0, L, N.MODE_GROUP_CALL), S * (W - 1) / W, alg_ag),
                ("all_reduce", lambda: comm.all_reduce(fulls, scale=1.0 / W), 2 * S * (W - 1) / W, 2 * S * (W - 1) / W),
                # output in the peer-visible heap as well: slice owners write the sums into every rank's output
                ("all_reduce_heap_output", lambda: comm.all_reduce(fulls, scale=1.0 / W, out=ar_heap), 2 * S * (W - 1) / W, 2 * S * (W - 1) / W),
            ]
            if cols >= W:
                # uneven all_to_all in the reference profiler's convention (profiler.py:106-117): the (256, C) tensor is
                # held column-sharded (cat dim 1), cut on dim 0 and exchanged, giving a row-sharded (L[r], C) result
                LC = hap_b200.sharding_round(cols, ratios_for(W))
                a2a_in = []
                for i, r in enumerate(ranks):
                    t = comm.symm_empty((ROWS, LC[r]), dtype, i)
                    t.copy_(torch.randn(ROWS, LC[r], device=dev).to(dtype))
                    a2a_in.append(t)
                m = [[L[j] * LC[r] * es for j in range(W)] for r in range(W)]          # bytes r -> j
                alg_a2a = max(max(sum(m[r][j] for j in range(W) if j != r), sum(m[i][r] for i in range(W) if i != r)) for r in range(W))
                cases.append(("all_to_all", lambda: comm.all_to_all(a2a_in, 0, 1, L, LC), S * (W - 1) / W, alg_a2a))
            # the same calls on ordinary torch tensors: every call first copies its input into the staging area
            staged = {}
            if S <= (64 << 20) and dtype == torch.float32:
                t_sh = [s_.clone() for s_ in shards]
                t_fu = [f_.clone() for f_ in fulls]
                staged = {"all_gather": lambda: comm.all_gather(t_sh, 0, L, N.MODE_PADDING, out=out),
                          "reduce_scatter": lambda: comm.reduce_scatter(t_fu, 0, L, N.MODE_PADDING),
                          "all_reduce": lambda: comm.all_reduce(t_fu, scale=1.0 / W)}
            for name, fn, bus, alg in cases:
                med, best = timed(fn, reps, inner=inner)
                row = {"op": name, "dtype": dname, "bytes": S, "world": W, "ms_median": med, "ms_min": best, "calls_per_timing": inner,
                       "busbw_GBps": bus / (med * 1e-3) / 1e9, "alg_GBps": alg / (med * 1e-3) / 1e9}
                if S <= (256 << 20):
                    row["graph_ms"] = graphed_ms(fn, inner, max(5, reps // 2))
                    row["graph_alg_GBps"] = alg / (row["graph_ms"] * 1e-3) / 1e9
                if name in staged:
                    row["staged_ms"], _ = timed(staged[name], max(5, reps // 2), warm=2, inner=inner)
                if not emulated:
                    row["frac_nvlink_900"] = row["alg_GBps"] / NVLINK_NOMINAL_GBS
                    if "graph_ms" in row:
                        row["graph_frac_nvlink_900"] = row["graph_alg_GBps"] / NVLINK_NOMINAL_GBS
                    if dtype == torch.float32 or name.startswith("all_reduce"):      # the reference's buffers are fp32-only
                        ref = {"all_gather": lambda: gp.all_gather(shards[0], 0, L, rank),
                               "all_gather_by_group_call": lambda: gp.all_gather_by_group_call(shards[0], 0, L, rank),
                               "reduce_scatter": lambda: gp.reduce_scatter(fulls[0], 0, L, rank),
                               "reduce_scatter_by_group_call": lambda: gp.reduce_scatter_by_group_call(fulls[0], 0, L, rank),
                               "all_reduce": lambda: gp.all_reduce(fulls[0]),
                               "all_reduce_heap_output": lambda: gp.all_reduce(fulls[0]),
                               "all_to_all": lambda: gp.all_to_all(a2a_in[0], 0, 1, L, LC, rank)}[name]
                        rmed, rbest = timed(ref, max(3, reps // 2), warm=2, inner=inner)
                        row["reference_on_nccl_ms_median"] = rmed
                        row["speedup_vs_reference_on_nccl"] = rmed / med
                rows.append(row)
                if rank == 0:
                    _print_sweep_row(row)
            del out, shards, fulls, cases, staged
            t_sh = t_fu = None
            a2a_in = None
            torch.cuda.empty_cache()
    # Secondary sweep in the reference's own convention (profiler.py:85-104, plot_collective_by_group_call.py:15-23):
    # a 4 MiB (256, 4096) fp32 tensor split on dim 1 (strided shards, 256 runs per shard) with the largest ratio swept
    # from the even split to 0.95 and the rest shared evenly.
    cols = 4096
    for max_ratio in [1.0 / W, 0.25, 0.5, 0.75, 0.95]:
        if max_ratio < 1.0 / W - 1e-9 or args.sweep_quick:
            continue
        raw = [max_ratio] + [(1.0 - max_ratio) / (W - 1)] * (W - 1)
        LS = hap_b200.sharding_round(cols, [x / sum(raw) for x in raw])
        comm.symm_reset()
        shards, fulls = [], []
        for i, r in enumerate(ranks):
            g = torch.Generator(dev).manual_seed(1000 + r)
            sh = comm.symm_empty((ROWS, LS[r]), torch.float32, i)
            sh.copy_(torch.randn(ROWS, LS[r], device=dev, generator=g))
            fu = comm.symm_empty((ROWS, cols), torch.float32, i)
            fu.copy_(torch.randn(ROWS, cols, device=dev, generator=g))
            shards.append(sh)
            fulls.append(fu)
        S = ROWS * cols * 4
        s_r = [ROWS * LS[r] * 4 for r in range(W)]
        alg = max(max(s_r[r] * (W - 1), S - s_r[r]) for r in range(W))
        for name, fn in (("all_gather dim1", lambda: comm.all_gather(shards, 1, LS, N.MODE_PADDING)),
                         ("all_gather_by_group_call dim1", lambda: comm.all_gather(shards, 1, LS, N.MODE_GROUP_CALL)),
                         ("reduce_scatter dim1", lambda: comm.reduce_scatter(fulls, 1, LS, N.MODE_PADDING))):
            med, best = timed(fn, 20, inner=10)
            row = {"op": name, "dtype": "f32", "bytes": S, "world": W, "max_ratio": max_ratio, "lengths": LS, "ms_median": med,
                   "ms_min": best, "calls_per_timing": 10, "busbw_GBps": S * (W - 1) / W / (med * 1e-3) / 1e9,
                   "alg_GBps": alg / (med * 1e-3) / 1e9}
            if not emulated:
                row["frac_nvlink_900"] = row["alg_GBps"] / NVLINK_NOMINAL_GBS
                ref = {"all_gather dim1": lambda: gp.all_gather(shards[0], 1, LS, rank),
                       "all_gather_by_group_call dim1": lambda: gp.all_gather_by_group_call(shards[0], 1, LS, rank),
                       "reduce_scatter dim1": lambda: gp.reduce_scatter(fulls[0], 1, LS, rank)}[name]
                rmed, _ = timed(ref, 10, warm=2, inner=10)
                row["reference_on_nccl_ms_median"] = rmed
                row["speedup_vs_reference_on_nccl"] = rmed / med
            rows.append(row)
            if rank == 0:
                print(f"max ratio {max_ratio:5.3f}  ", end="")
                _print_sweep_row(row)
    comm.check()
    comm.destroy()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and args.sweep_out:
        os.makedirs(os.path.dirname(os.path.abspath(args.sweep_out)), exist_ok=True)
        with open(args.sweep_out, "w") as f:
            json.dump(rows, f, indent=1)


def _print_sweep_row(r):
    extra = ""
    if "frac_nvlink_900" in r:
        extra = f" nvlink {100 * r['frac_nvlink_900']:5.1f}%"
    if "graph_ms" in r:
        extra += f"  graph {r['graph_ms']:8.4f} ms"
        if "graph_frac_nvlink_900" in r:
            extra += f" ({100 * r['graph_frac_nvlink_900']:5.1f}%)"
    if "staged_ms" in r:
        extra += f"  staged {r['staged_ms']:8.4f} ms"
    if "speedup_vs_reference_on_nccl" in r:
        extra += f"  ref/NCCL {r['reference_on_nccl_ms_median']:9.4f} ms (x{r['speedup_vs_reference_on_nccl']:.2f})"
    print(f"{r['op']:30s} {r['dtype']:4s} {r['bytes']:>11d} B  {r['ms_median']:9.4f} ms  bus {r['busbw_GBps']:8.2f} GB/s"
          f"  alg {r['alg_GBps']:8.2f} GB/s{extra}", flush=True)



# ----------------------------------------------------------------------------------------------
# sharded F.linear GEMMs of the Transformer-LM configuration (per-GPU token count 32 x 256 = 8192),
# forward + dgrad + wgrad, next to cuBLAS (torch.matmul) on the same GPU
# ----------------------------------------------------------------------------------------------
LM_LAYERS = [("attn in-proj", 2304, 768), ("attn out-proj", 768, 768), ("ffn up", 3072, 768), ("ffn down", 768, 3072),
             ("lm head", 33280, 768)]


def run_gemm(args):
    import torch
    import hap_b200
    from hap_b200 import linear_ops as LO
    from hap_b200 import _native as N
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks, peak_kind = measured_peaks()
    M = args.gemm_tokens
    rows, tot_flops, tot_ms, tot_ms_ref = [], 0.0, 0.0, 0.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)       # > L2, written between timed iterations

    SETS = 6      # distinct operand sets visited round-robin: together larger than L2, so every call starts cold

    def timeit(fn):
        """Median device time per call over `steps` timings of SETS back-to-back calls (one per operand set)."""
        for _ in range(max(args.warmup, 3)):
            for i in range(SETS):
                fn(i)
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(SETS):
                fn(i)
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b) / SETS)
        return statistics.median(ts)

    launches0 = N.lib.hapx_launch_count()
    wanted = [x.strip() for x in args.gemm_layers.split(",") if x.strip()]
    for name, n, k in LM_LAYERS:
        if wanted and name not in wanted:
            continue
        g = torch.Generator(dev).manual_seed(39)
        xs = [torch.randn(M, k, device=dev, generator=g).to(torch.bfloat16) for _ in range(SETS)]
        ws = [(torch.randn(n, k, device=dev, generator=g) * k ** -0.5).to(torch.bfloat16) for _ in range(SETS)]
        bs = [torch.randn(n, device=dev, generator=g).to(torch.bfloat16) for _ in range(SETS)]
        gys = [torch.randn(M, n, device=dev, generator=g).to(torch.bfloat16) for _ in range(SETS)]
        flops = 2.0 * M * n * k
        cases = [("fwd", lambda i: LO.linear_forward(xs[i], ws[i], bs[i]), lambda i: torch.nn.functional.linear(xs[i], ws[i], bs[i])),
                 ("dgrad", lambda i: LO.linear_dgrad(gys[i], ws[i]), lambda i: gys[i] @ ws[i]),
                 ("wgrad", lambda i: LO.linear_wgrad(gys[i], xs[i], True, False), lambda i: gys[i].t() @ xs[i])]
        for what, ours, ref in cases:
            ms, ms_ref = timeit(ours), timeit(ref)
            rows.append({"layer": name, "op": what, "m": M, "n": n, "k": k, "ms": ms, "tflops": flops / ms / 1e9,
                         "frac_of_peak": flops / ms / 1e9 / peaks["bf16_tflops"], "cublas_ms": ms_ref,
                         "cublas_tflops": flops / ms_ref / 1e9})
            tot_flops += flops
            tot_ms += ms
            tot_ms_ref += ms_ref
    LO.gemm_status()
    launches = N.lib.hapx_launch_count() - launches0
    for r in rows:
        print(f"{r['layer']:14s} {r['op']:6s} m={r['m']} n={r['n']:6d} k={r['k']:5d}  {r['ms']:8.4f} ms {r['tflops']:8.1f} TF/s "
              f"({100 * r['frac_of_peak']:5.1f}% of {peaks['bf16_tflops']:.0f})   cuBLAS {r['cublas_ms']:8.4f} ms {r['cublas_tflops']:8.1f} TF/s",
              file=sys.stderr, flush=True)
    best = max(rows, key=lambda r: r["ms"])
    print(json.dumps({
        "metric": "sharded_linear_tflops", "value": tot_flops / tot_ms / 1e9, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": tot_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"forward + dgrad + wgrad of the 5 linear layers of the Transformer-LM configuration at {M} tokens per GPU",
                   "l2": "6 operand sets visited round-robin (larger than L2 together) + 256 MiB flush between timings"},
        "roofline": {"bound": "tensor", "kernel": f"gemm_bf16_kernel ({best['layer']} {best['op']})", "achieved": best["tflops"],
                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": best["frac_of_peak"], "peak_kind": peak_kind, "traffic": None},
        "cublas_tflops": tot_flops / tot_ms_ref / 1e9, "gpu_launches": int(launches), "layers": rows}), flush=True)


# ----------------------------------------------------------------------------------------------
# SPMD training step of the Transformer-LM configuration: samples/s at N GPUs
# (12 layers, d_model 768, 12 heads, FFN 3072, pre-LN, vocab 33278 padded to 33280, seq 256, bf16,
#  batch 32 per GPU of uniform token ids; data parallel with ratio-sharded FFN/attention weights)
# ----------------------------------------------------------------------------------------------
def _lm_cpu_worker(rank, world, store, batch_per_rank, out_path, layers):
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from types import SimpleNamespace
    sys.path.insert(0, ROOT)
    from hap_b200 import plan as P
    from oracle import gloo_port
    from oracle.cpu_executors import CpuProcessWorker
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}")
    torch.manual_seed(39)
    model = P.TransformerLM(nlayers=layers).to(torch.bfloat16)
    ns = SimpleNamespace(collectives=gloo_port, linear=F.linear, mha=F.multi_head_attention_forward, dropout=F.dropout)
    B = batch_per_rank * world
    graph = P.emit_lm(model, "dp_zero", ratios_for(world), rank, B, ns, dropout_p=0.1)
    worker = CpuProcessWorker(torch.fx.GraphModule(model, graph))
    g = torch.Generator().manual_seed(2024)
    tok = torch.randint(0, 33278, (B, 256), generator=g)
    tgt = torch.randint(0, 33278, (B, 256), generator=g)
    worker.step(tok, tgt)
    dist.barrier()
    t0 = time.perf_counter()
    worker.step(tok, tgt)
    dist.barrier()
    if rank == 0:
        json.dump({"s": time.perf_counter() - t0, "batch": B}, open(out_path, "w"))
    dist.destroy_process_group()


def run_lm_cpu(world, batch_per_rank, layers):
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "t.json")
        mp.spawn(_lm_cpu_worker, args=(world, os.path.join(d, "store"), batch_per_rank, out, layers), nprocs=world, join=True)
        r = json.load(open(out))
    cores = os.cpu_count() or 1
    # a step's cost is proportional to the layer count (the embedding/decoder part is counted once too often, in the CPU's favour)
    return {"value": r["batch"] / r["s"] * layers / 12.0, "unit": "samples/s", "cores": cores, "kind": "port",
            "sample": f"{world} gloo ranks x {max(1, cores // world)} threads, same fx program (dp_zero, dropout 0.1) with the CPU port of the "
                      f"collectives and torch CPU ops, {layers} of 12 layers, batch {batch_per_rank} per rank, 1 step after 1 warm-up; "
                      f"value scaled by {layers}/12",
            "step_s": r["s"]}


def lm_step(args, job, kind, plan, use_graph, dropout_p):
    """Time the training step of one program (``kind``: lm / vit / moe) at job.n_gpus GPUs: device time per
    step (CUDA events, max over ranks) and the end-to-end time with the inputs coming from pinned host memory
    every step and the loss read back on the host."""
    import torch
    import hap_b200
    from hap_b200 import plan as P
    from hap_b200 import _native as N
    from hap_b200.spmd import ProcessWorker
    n_gpus, rank, dev, dist = job.n_gpus, job.rank, job.dev, job.dist
    W = n_gpus
    per_gpu = args.lm_batch if args.lm_batch > 0 else {"lm": 32, "vit": 64, "moe": 16}[kind]
    B = per_gpu * W
    ratios = ratios_for(W)
    if kind == "vit" and W in (4, 8):      # the heterogeneous ratios of the ViT configuration, replicated to 8
        ratios = [x / (W // 4) for x in [0.3, 0.25, 0.2, 0.25] * (W // 4)]
    torch.manual_seed(39)
    L = args.lm_layers if args.lm_layers > 0 else {"lm": 12, "vit": 12, "moe": 8}[kind]
    g = torch.Generator().manual_seed(2024)
    lb = hap_b200.sharding_round(B, ratios)
    bmax = max(lb)
    if kind == "lm":
        model = P.TransformerLM(nlayers=L)
        emit = lambda m, r: P.emit_lm(m, plan, ratios, r, B, dropout_p=dropout_p)
        in_h = (torch.randint(0, 33278, (B, 256), generator=g), torch.randint(0, 33278, (B, 256), generator=g))
        M = bmax * 256
        fwd = L * (2.0 * M * 768 * (2304 + 768 + 3072 + 3072) + 2 * 2.0 * bmax * 12 * 256 * 256 * 64) + 2.0 * M * 768 * 33280
        desc = f"Transformer LM training step ({L} layers, d_model 768, 12 heads, FFN 3072, pre-LN, vocab 33280, seq 256, dropout {dropout_p}), plan {plan}"
    elif kind == "vit":
        model = P.ViT(nlayers=L)
        emit = lambda m, r: P.emit_vit(m, plan, ratios, r, B, dropout_p=dropout_p)
        in_h = (torch.randn(B, 3, 224, 224, generator=g).to(torch.bfloat16), torch.randint(0, 1000, (B,), generator=g))
        M = bmax * 197
        fwd = L * (2.0 * M * 768 * (2304 + 768 + 3072 + 3072) + 2 * 2.0 * bmax * 12 * 197 * 197 * 64) + 2.0 * bmax * 196 * 768 * 768
        desc = f"ViT-B/16 training step ({L} layers, d 768, 12 heads, MLP 3072, 224x224x3 images, 1000 classes, dropout {dropout_p}), plan {plan}"
    else:
        model = P.MoETransformerLM(nlayers=L)
        emit = lambda m, r: P.emit_moe(m, ratios, r, B, dropout_p=dropout_p)
        in_h = (torch.randint(0, 33278, (B, 512), generator=g), torch.randint(0, 33278, (B, 512), generator=g))
        M = bmax * 512
        e_max = max(hap_b200.sharding_round(32, ratios))
        fwd = L * (2.0 * M * 1024 * (3072 + 1024) + 2 * 2.0 * bmax * 16 * 512 * 512 * 64        # attention projections + core
                   + 2 * 2.0 * B * e_max * 20 * 1024 * 4096) + 2.0 * M * 1024 * 33280           # expert FFNs of the busiest rank
        desc = (f"MoE Transformer training step ({L} layers, d_model 1024, 16 heads, 32 experts FFN 4096, top-2 gating, capacity 20, "
                f"vocab 33280, seq 512, dropout {dropout_p}), expert parallel, experts per rank {hap_b200.sharding_round(32, ratios)}")
    model = model.to(torch.bfloat16).to(dev)
    n_params = sum(p.numel() for p in model.parameters())
    hap_b200.dropout.manual_seed(39 + rank)
    def program(r):
        graph = emit(model, r)
        if not args.lm_no_fuse:
            hap_b200.fxpass.fuse_elementwise(graph)     # dropout + residual add, activation + dropout: one pass each
        if not args.lm_no_fuse:
            hap_b200.fxpass.fuse_residual_norm(graph)   # pre-LN blocks: the residual gradient joins inside the norm's backward kernel
        if kind == "moe" and not args.lm_no_fuse:
            hap_b200.fxpass.sparsify_moe(graph)         # dispatch / combine as row gathers instead of dense one-hot contractions
        if W > 1 and not args.lm_no_prefetch:
            hap_b200.fxpass.prefetch_parameter_gathers(graph)   # parameter gathers early, on the side stream
        return torch.fx.GraphModule(model, graph)

    if W == 1:
        comm = hap_b200.single_comm(dev, stage_bytes=256 << 20, heap_bytes=(320 << 20) + 2 * n_params)
        hap_b200.collectives.set_default_comm(comm)
        worker = ProcessWorker(program(0), comm=comm)
    else:
        comm = hap_b200.init_process_comm(stage_bytes=256 << 20, heap_bytes=(320 << 20) + 2 * n_params)
        hap_b200.collectives.set_default_comm(comm)
        # the reference sums the partial losses with dist.reduce (worker.py:63-64); here through the package's all_reduce
        worker = ProcessWorker(program(rank),
                               reduce_loss=lambda t: comm.all_reduce([t.reshape(1).float()])[0], comm=comm)
    step = worker.step
    tok_h, tgt_h = in_h[0].pin_memory(), in_h[1].pin_memory()
    tok, tgt = tok_h.to(dev), tgt_h.to(dev)
    if use_graph:
        step = worker.capture(tok, tgt)
    barrier = job.barrier

    for _ in range(max(args.warmup, 3)):
        step(tok, tgt)
    barrier()
    sampler = ClockSampler(job.local_rank)
    sampler.start()
    l0 = N.lib.hapx_launch_count()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for _ in range(args.steps):
        loss = step(tok, tgt)
    b.record()
    barrier()
    launches = N.lib.hapx_launch_count() - l0
    if use_graph:       # a replay issues no host-side launches: count the kernels recorded into the graph
        launches = worker.captured_launches * args.steps
    clocks = sampler.finish()
    ms = a.elapsed_time(b) / args.steps

    # ---- end to end: every step's inputs come from pinned host memory, every step's loss goes back to the host.
    # The upload of step i+1 runs on a second stream while step i computes; the loss of step i is read after step
    # i+1 has been queued (the reference only logs it, worker.py:63-70), so the host never idles the GPU.
    e2e_steps = max(3, args.steps)
    up = torch.cuda.Stream()
    main = torch.cuda.current_stream()
    stage = [[torch.empty_like(tok), torch.empty_like(tgt)] for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    loss_h = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ev = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        k = i & 1
        with torch.cuda.stream(up):
            up.wait_event(consumed[k])
            stage[k][0].copy_(tok_h, non_blocking=True)
            stage[k][1].copy_(tgt_h, non_blocking=True)
            ready[k].record(up)

    def e2e_loop(n):
        losses = []
        for k in range(2):
            consumed[k].record(main)
        upload(0)
        for i in range(n):
            k = i & 1
            if i + 1 < n:
                upload(i + 1)
            main.wait_event(ready[k])
            out = step(stage[k][0], stage[k][1])
            consumed[k].record(main)
            loss_h[k].copy_(out.detach().reshape(1).float(), non_blocking=True)
            loss_ev[k].record(main)
            if i >= 1:
                loss_ev[k ^ 1].synchronize()
                losses.append(float(loss_h[k ^ 1]))
        loss_ev[(n - 1) & 1].synchronize()
        losses.append(float(loss_h[(n - 1) & 1]))
        return losses

    e2e_loop(3)
    c, d = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    c.record()
    losses = e2e_loop(e2e_steps)
    d.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    barrier()
    e2e_ms = c.elapsed_time(d) / e2e_steps
    ms, e2e_ms, wall_ms = job.max_over_ranks(ms, e2e_ms, wall_ms)
    comm.check()
    hap_b200.linear_ops.gemm_status()
    peaks, peak_kind = measured_peaks()
    # GEMM flops of one step on the busiest rank (largest batch share): 3 x forward, 2*M*N*K each
    achieved = 3 * fwd / (ms * 1e-3) / 1e12
    peak = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
    result = {
        "metric": "spmd_step_samples_per_s", "value": B / (ms * 1e-3), "unit": "samples/s", "n_gpus": n_gpus, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{desc}, global batch {B} split {lb}", "parameters": n_params, "plan": plan, "batch_split": lb,
                   "executor": "CUDA graph of the whole iteration" if use_graph else "eager fx GraphModule",
                   "l2": "activations and weights of a step exceed L2 by far", "loss": losses[-1]},
        "roofline": {"bound": "tensor", "kernel": "gemm2_bf16_kernel (all linear / attention contractions of the busiest rank)",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_kind": peak_kind + " (sustained: the kernels run inside a long step)", "traffic": None,
                     "note": "whole-step time, so this fraction also pays for every non-GEMM op of the step"},
        "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "samples/s",
                "h2d_bytes_per_step": int(tok_h.numel() * tok_h.element_size() + tgt_h.numel() * tgt_h.element_size()) * n_gpus,
                "d2h_bytes_per_step": 4 * n_gpus, "ms_per_step": e2e_ms, "host_wall_ms_per_step": wall_ms, "steps": e2e_steps,
                "pipeline": "inputs uploaded on a second stream one step ahead, loss read one step late"},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    del worker, step, model
    hap_b200.collectives.set_default_comm(None)
    comm.destroy()
    torch.cuda.empty_cache()
    return result


def run_lm_step(args, job):
    """The `spmd_step` object of the default line: the Transformer-LM configuration, plan dp_zero, graph replay,
    attention and residual dropout 0.1 as in the reference's throughput runs (config.py:33)."""
    r = lm_step(args, job, "lm", "dp_zero", True, args.lm_dropout)
    return {"samples_per_s": r["value"], "ms_per_step": r["ms_per_step"], "plan": r["config"]["plan"],
            "batch_split": r["config"]["batch_split"], "workload": r["config"]["workload"], "executor": r["config"]["executor"],
            "roofline": r["roofline"], "e2e": r["e2e"], "loss": r["config"]["loss"], "gpu_launches": r["gpu_launches"],
            "clocks": r["clocks"], "dtype": "bf16"}


def run_lm(args):
    job = Job(args.gpus)
    result = lm_step(args, job, args.lm_model, args.lm_plan, args.lm_graph, args.lm_dropout)
    if job.rank == 0 and job.n_gpus == 1 and not args.no_cpu_baseline and args.lm_model == "lm":
        result["cpu_baseline"] = run_lm_cpu(2, 2, 2)
    job.finish()
    if job.rank == 0:
        print(json.dumps(result), flush=True)


# ----------------------------------------------------------------------------------------------
# attention core and MoE einsums at the configurations' per-GPU shapes, next to torch's own kernels
# ----------------------------------------------------------------------------------------------
def run_ops(args):
    import torch
    import hap_b200
    from hap_b200 import attention as A
    from hap_b200.einsum import einsum
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    def graphed(fn):
        """fn recorded into a CUDA graph (after a warm-up on a side stream): its replay costs device time only."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return graph.replay

    rows = []
    parts = set(args.ops.split(","))
    g = torch.Generator(dev).manual_seed(39)
    for name, L, n, H, D, causal in (("LM attention", 256, 32, 12, 64, True), ("ViT attention", 197, 64, 12, 64, False),
                                     ("MoE attention", 512, 16, 16, 64, True)) if "attention" in parts else ():
        E = H * D
        qkv = torch.randn(L, n, 3 * E, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        go = torch.randn(L, n, E, device=dev, generator=g).to(torch.bfloat16)
        mask = "causal" if causal else None

        def ours():
            qkv.grad = None
            A.attention(qkv, H, mask).backward(go)

        def ours_dropout():
            qkv.grad = None
            A.attention(qkv, H, mask, dropout_p=0.1).backward(go)

        def ours_fwd():
            with torch.no_grad():
                A.attention(qkv, H, mask)

        def ref():
            qkv.grad = None
            q, k, v = (t.reshape(L, n * H, D).transpose(0, 1) for t in qkv.split(E, dim=2))
            o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)
            o.transpose(0, 1).reshape(L, n, E).backward(go)

        flops = 3.5 * 4.0 * n * H * L * L * D * (0.5 if causal else 1.0)     # fwd 2 GEMMs + bwd 5 GEMMs (2.5x fwd)
        t, tr = timeit(graphed(ours)), timeit(ref)
        td, tf = timeit(graphed(ours_dropout)), timeit(graphed(ours_fwd))
        # bytes that must move: qkv read + out written (forward); qkv, out, dout read + dqkv written (backward)
        io = (L * n * 3 * E + L * n * E + 2 * L * n * 3 * E + 2 * L * n * E) * 2
        rows.append({"op": name + " fwd+bwd", "shape": f"L={L} N={n} H={H} D={D}", "ms": t, "torch_ms": tr, "tflops": flops / t / 1e9,
                     "dropout_0.1_ms": td, "fwd_only_ms": tf, "gbs": io / t / 1e6, "frac_of_hbm_peak": io / t / 1e6 / float(measured_peaks()[0]["hbm_gbs"]),
                     "eager_ms": timeit(ours)})
    b, s, e, c, d, h = 16, 512, 32, 20, 1024, 4096
    x = torch.randn(b, s, d, device=dev, generator=g).to(torch.bfloat16)
    disp = (torch.rand(b, s, e, c, device=dev, generator=g) < 0.003).to(torch.bfloat16)
    for code, a_, b_, fl in (("bsd,bsec->becd", x, disp, 2.0 * b * s * e * c * d),
                             ("becd,bsec->bsd", torch.randn(b, e, c, d, device=dev, generator=g).to(torch.bfloat16), disp, 2.0 * b * s * e * c * d)) if "einsum" in parts else ():
        t, tr = timeit(lambda: einsum(code, a_, b_)), timeit(lambda: torch.einsum(code, a_, b_))
        rows.append({"op": code, "shape": f"b={b} s={s} e={e} c={c} d={d}", "ms": t, "torch_ms": tr, "tflops": fl / t / 1e9})
    for el in (7, 4, 2) if "einsum" in parts else ():        # experts on this GPU under the r8 split of 32 experts
        bg = 128
        w1 = (torch.randn(el, d, h, device=dev, generator=g) * d ** -0.5).to(torch.bfloat16)
        inp = torch.randn(bg, el, c, d, device=dev, generator=g).to(torch.bfloat16)
        fl = 2.0 * bg * el * c * d * h
        t, tr = timeit(lambda: einsum("edh,becd->bech", w1, inp)), timeit(lambda: torch.einsum("edh,becd->bech", w1, inp))
        rows.append({"op": "edh,becd->bech", "shape": f"b={bg} e={el} c={c} d={d} h={h}", "ms": t, "torch_ms": tr, "tflops": fl / t / 1e9})
    peak_gbs = float(measured_peaks()[0]["hbm_gbs"])
    if "norm" in parts:
        # layer_norm forward + backward on the activations of one Transformer-LM layer (8192 tokens x 768, bf16)
        from hap_b200.norm import layer_norm
        rows_, E_ = 8192, 768
        xn = torch.randn(rows_, E_, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        wn = torch.ones(E_, device=dev, dtype=torch.bfloat16, requires_grad=True)
        bn = torch.zeros(E_, device=dev, dtype=torch.bfloat16, requires_grad=True)
        dyn = torch.randn(rows_, E_, device=dev, generator=g).to(torch.bfloat16)

        def ln_step(fn):
            def run():
                xn.grad = wn.grad = bn.grad = None
                fn(xn, (E_,), wn, bn, 1e-5).backward(dyn)
            return run

        t_eager = timeit(ln_step(layer_norm))
        t, tr = timeit(graphed(ln_step(layer_norm))), timeit(graphed(ln_step(torch.nn.functional.layer_norm)))
        nbytes = 5 * rows_ * E_ * 2            # forward: x in, y out; backward: x, dy in, dx out
        rows.append({"op": "layer_norm fwd+bwd", "shape": f"rows={rows_} E={E_} bf16", "ms": t, "torch_ms": tr, "tflops": 0.0,
                     "gbs": nbytes / t / 1e6, "frac_of_hbm_peak": nbytes / t / 1e6 / peak_gbs, "eager_ms": t_eager})
    if "dropout" in parts:
        # F.dropout and its fusions with the neighbouring elementwise ops of an encoder layer, forward + backward,
        # on the activations of one Transformer-LM layer (8192 tokens x 768 after attention / FFN, x 3072 inside the FFN)
        from hap_b200 import dropout as DR
        F_ = torch.nn.functional
        for label, width, ours_fn, ref_fn, passes in (
                ("dropout", 768, lambda x_, r_: DR.dropout(x_, 0.1), lambda x_, r_: F_.dropout(x_, 0.1), 4),
                ("x + dropout(y)", 768, lambda x_, r_: DR.dropout_add(x_, r_, 0.1), lambda x_, r_: r_ + F_.dropout(x_, 0.1), 5),
                ("dropout(relu(x))", 3072, lambda x_, r_: DR.act_dropout(x_, "relu", 0.1), lambda x_, r_: F_.dropout(F_.relu(x_), 0.1), 5),
                ("dropout(gelu(x))", 3072, lambda x_, r_: DR.act_dropout(x_, "gelu", 0.1), lambda x_, r_: F_.dropout(F_.gelu(x_), 0.1), 5)):
            xd = torch.randn(8192, width, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
            rd = torch.randn(8192, width, device=dev, generator=g).to(torch.bfloat16)
            gd = torch.randn(8192, width, device=dev, generator=g).to(torch.bfloat16)

            def step_of(fn):
                def run():
                    xd.grad = None
                    fn(xd, rd).backward(gd)
                return run

            t_eager = timeit(step_of(ours_fn))
            t, tr = timeit(graphed(step_of(ours_fn))), timeit(graphed(step_of(ref_fn)))
            # forward reads x (and the residual) and writes y; backward reads dy (and x or y for an activation) and writes dx
            nbytes = passes * 8192 * width * 2
            rows.append({"op": label + " fwd+bwd", "shape": f"rows=8192 E={width} bf16 p=0.1", "ms": t, "torch_ms": tr, "tflops": 0.0,
                         "gbs": nbytes / t / 1e6, "frac_of_hbm_peak": nbytes / t / 1e6 / peak_gbs, "eager_ms": t_eager})
    if "moe" in parts:
        # dispatch / combine of one MoE layer as row gathers (top-2 gating, 32 experts, capacity 20) against the
        # dense one-hot contractions torch runs for the same einsums; forward + backward
        from hap_b200 import plan as P_
        from hap_b200.einsum import sparse_dispatch, sparse_combine
        bm, sm, em, cm, dm = 16, 512, 32, 20, 1024
        xm = torch.randn(bm, sm, dm, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        gate_w = (torch.randn(dm, em, device=dev, generator=g) * dm ** -0.5).to(torch.bfloat16)
        with torch.no_grad():
            disp_m, comb_m = P_.top2_gating(xm.detach(), gate_w, em, cm)
        disp_m, comb_m = disp_m.to(torch.bfloat16), comb_m.to(torch.bfloat16).requires_grad_(True)
        gm = torch.randn(bm, sm, dm, device=dev, generator=g).to(torch.bfloat16)

        def moe_step(dispatch_fn, combine_fn):
            def run():
                xm.grad = comb_m.grad = None
                combine_fn(dispatch_fn(xm, disp_m), comb_m).backward(gm)
            return run

        ours_m = moe_step(sparse_dispatch, sparse_combine)
        ref_m = moe_step(lambda a_, b_: torch.einsum("bsd,bsec->becd", a_, b_), lambda a_, b_: torch.einsum("becd,bsec->bsd", a_, b_))
        t_eager = timeit(ours_m)
        t, tr = timeit(graphed(ours_m)), timeit(graphed(ref_m))
        # rows of 2 KiB: dispatch reads <= e*c rows per sequence and writes e*c; combine reads them and writes s rows; same
        # again for the gradients; plus the dense dispatch / combine tensors read once each to build the index
        nbytes = 2 * (2 * bm * em * cm * dm * 2 + 2 * bm * sm * dm * 2) + 2 * bm * sm * em * cm * 2
        rows.append({"op": "MoE dispatch + combine fwd+bwd (row gathers)", "shape": f"b={bm} s={sm} e={em} c={cm} d={dm}", "ms": t, "torch_ms": tr,
                     "tflops": 0.0, "gbs": nbytes / t / 1e6, "frac_of_hbm_peak": nbytes / t / 1e6 / peak_gbs, "eager_ms": t_eager})
    if "loss" in parts:
        # log_softmax + summed nll_loss forward + backward on the LM head's logits (8192 tokens x 33280, bf16)
        from hap_b200.loss import nll_log_softmax_sum
        rows_, V_ = 8192, 33280
        lg = torch.randn(rows_, V_, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        tg = torch.randint(0, V_, (rows_,), device=dev, generator=g)

        def ours_loss():
            lg.grad = None
            nll_log_softmax_sum(lg, tg).backward()

        def ref_loss():
            lg.grad = None
            torch.nn.functional.nll_loss(torch.nn.functional.log_softmax(lg.float(), -1), tg, reduction="sum").backward()

        t_eager = timeit(ours_loss)
        t, tr = timeit(graphed(ours_loss)), timeit(graphed(ref_loss))
        nbytes = 3 * rows_ * V_ * 2            # forward reads the logits; backward reads them and writes the gradient
        rows.append({"op": "log_softmax + nll fwd+bwd", "shape": f"rows={rows_} V={V_} bf16", "ms": t, "torch_ms": tr, "tflops": 0.0,
                     "gbs": nbytes / t / 1e6, "frac_of_hbm_peak": nbytes / t / 1e6 / peak_gbs, "eager_ms": t_eager})
        del lg
    if "tail" in parts:
        # step tail: clip by the gradient norm + Adam over the parameter tensors of the Transformer-LM
        # configuration (bf16; 12 layers + embeddings + head), against torch's clip_grad_norm_ + Adam
        from hap_b200.optim import ClipAdam
        shapes = [(33280, 768), (256, 768)] + [s_ for _ in range(12) for s_ in
                  ((768,), (768,), (2304, 768), (2304,), (768, 768), (768,), (768,), (768,), (3072, 768), (3072,), (768, 3072), (768,))] + [(768,), (768,), (33280, 768), (33280,)]
        mine_p = [torch.nn.Parameter((torch.randn(s_, device=dev, generator=g) * 0.02).to(torch.bfloat16)) for s_ in shapes]
        ref_p = [torch.nn.Parameter(p_.detach().clone()) for p_ in mine_p]
        for p_, q_ in zip(mine_p, ref_p):
            p_.grad = (torch.randn(p_.shape, device=dev, generator=g) * 0.01).to(torch.bfloat16)
            q_.grad = p_.grad.clone()
        fused, ref_opt = ClipAdam(mine_p, lr=5e-4, max_norm=0.5), torch.optim.Adam(ref_p, lr=5e-4)

        def ref_tail():
            torch.nn.utils.clip_grad_norm_(ref_p, 0.5)
            ref_opt.step()

        elems = sum(p_.numel() for p_ in mine_p)
        tail_bytes = elems * 2 * 8                    # norm pass reads g; update reads g, p, m, v and writes p, m, v
        t_eager, tr = timeit(fused.step), timeit(ref_tail)
        # the kernels alone: the same step replayed from a CUDA graph (no host time between launches)
        side = torch.cuda.Stream()
        tail_graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            with torch.cuda.graph(tail_graph, stream=side):
                fused.step()
        t = timeit(tail_graph.replay)
        peak = float(measured_peaks()[0]["hbm_gbs"])
        rows.append({"op": "clip + Adam step tail", "shape": f"{len(shapes)} tensors, {elems / 1e6:.1f} M bf16 elements", "ms": t, "torch_ms": tr,
                     "eager_ms": t_eager, "tflops": 0.0, "gbs": tail_bytes / t / 1e6, "frac_of_hbm_peak": tail_bytes / t / 1e6 / peak})
    hap_b200.linear_ops.gemm_status()
    for r in rows:
        extra = f"  {r['gbs']:8.0f} GB/s ({100 * r['frac_of_hbm_peak']:.0f}% of measured HBM peak; {r['eager_ms']:.4f} ms issued eagerly)" if "gbs" in r else ""
        print(f"{r['op']:26s} {r['shape']:36s} {r['ms']:8.4f} ms {r['tflops']:8.1f} TF/s   torch {r['torch_ms']:8.4f} ms{extra}", file=sys.stderr, flush=True)
    print(json.dumps({"metric": "op_microbenchmarks", "rows": rows}), flush=True)

def run_reference_arm(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    emulated = args.gpus == 1
    W = 8 if emulated else args.gpus
    size = args.cpu_size_mib << 20
    base = run_cpu_arm(W, size, max(1, args.steps), max(1, args.warmup))
    line = {
        "impl": "reference", "metric": "uneven_collective_bus_bandwidth", "value": base["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": collective_config(W, args.size_mib, emulated),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="hapx", choices=["hapx", "reference"])
    ap.add_argument("--size-mib", type=int, default=1024, help="tensor size S of the GPU arm")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--cpu-size-mib", type=int, default=64, help="tensor size of the bounded CPU sample")
    ap.add_argument("--cpu-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-spmd-step", action="store_true", help="default run: skip the Transformer-LM training step")
    ap.add_argument("--lm-dropout", type=float, default=0.1, help="dropout of the lm workload (the reference trains with 0.1)")
    ap.add_argument("--sweep", action="store_true", help="size sweep instead of the single JSON line")
    ap.add_argument("--sweep-quick", action="store_true", help="fewer repetitions per size and no dim-1 skew sweep")
    ap.add_argument("--sweep-out", default="", help="write the sweep's rows to this JSON file")
    ap.add_argument("--sweep-max-mib", type=int, default=1024)
    ap.add_argument("--workload", default="collectives", choices=["collectives", "gemm", "lm", "ops"])
    ap.add_argument("--lm-model", default="lm", choices=["lm", "vit", "moe"], help="which program the lm workload steps")
    ap.add_argument("--lm-batch", type=int, default=0, help="samples per GPU (0: the configuration's 32 / 64 / 16)")
    ap.add_argument("--lm-layers", type=int, default=0, help="0: the configuration's 12 / 12 / 8")
    ap.add_argument("--lm-plan", default="dp_zero", choices=["dp", "dp_zero", "tp"])
    ap.add_argument("--lm-no-prefetch", action="store_true", help="gather sharded parameters where they are used, on the main stream")
    ap.add_argument("--lm-no-fuse", action="store_true", help="run the program as emitted, without the elementwise fusion pass")
    ap.add_argument("--lm-graph", action="store_true", help="capture the training step into a CUDA graph")
    ap.add_argument("--gemm-tokens", type=int, default=8192)
    ap.add_argument("--gemm-layers", default="", help="comma-separated layer names to restrict the gemm workload to")
    ap.add_argument("--ops", default="attention,einsum,norm,dropout,moe,loss,tail", help="parts of the ops workload to run")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "gemm":
        run_gemm(args)
    elif args.workload == "lm":
        run_lm(args)
    elif args.workload == "ops":
        run_ops(args)
    elif args.sweep:
        run_sweep(args)
    else:
        run_default(args)


if __name__ == "__main__":
    main()
