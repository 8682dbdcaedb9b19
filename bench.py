#!/usr/bin/env python
"""Headline benchmark: all-reduce bus bandwidth (NCCL convention, bytes*2(n-1)/n/t).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step = one sum all-reduce of a 128 MiB fp32 message per rank (inputs larger
than the 126 MB L2) between pre-allocated symmetric buffers.  N > 1 runs one rank
per GPU (torchrun exports RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*); N = 1 has no
peer, so two ranks are emulated on the one GPU by a single cooperative launch of
the same kernels (HBM-bound, no NVLink) and the line says so.  Timing: CUDA events
per step on the launching stream after W warm-up steps, barrier + synchronize on
both sides, max over ranks.  The line also carries p50/p99 latency of a 1 MiB
all-reduce (1000 calls replayed from one CUDA graph, rotating over buffers that
together exceed L2; every kernel stamps %globaltimer when its first CTA starts and
when its last CTA leaves, so the samples contain no host jitter; percentiles per
rank, then the max over ranks), the end-to-end number (pinned host -> device copy of the step's
input, all-reduce through the public API, device -> host copy of the result) next
to the same copies without the collective, an NCCL arm measured with the same
timing code on the same GPUs, and the clocks sampled during the timed region.

`--impl reference` runs the unmodified reference (its own benchmark_yali binary and
an end-to-end harness around its yali::allreduce, built by
baseline/build_reference.sh into baseline/_ref/) for the same message.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# 2x A100 NV4, 128 MB fp32, the reference's published bus bandwidth (its README.md:124,273).
BASELINE_GBPS_128MB = 79.2
MESSAGE_BYTES = 128 << 20


def bus_factor(n: int) -> float:
    return 2.0 * (n - 1) / n if n > 1 else 1.0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0) -> None:
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def gather_max(comm, value: float) -> float:
    """Max over ranks of a host float (control plane, outside any timed region)."""
    import struct
    if comm.nlocal != 1 or comm.world == 1:
        return value
    parts = comm.allgather_object_bytes(struct.pack("d", value))
    return max(struct.unpack("d", p)[0] for p in parts)


def time_steps(comm, torch, fn, steps: int, warmup: int, per_step_events: bool = True):
    """Runs fn(i) warmup+steps times; returns (total_ms max over ranks, per-step ms list of this rank).
    One CUDA event pair brackets the `steps` timed calls; with `per_step_events` an event is also recorded
    between the steps (each record keeps consecutive kernels a few microseconds apart)."""
    for i in range(warmup):
        fn(i)
    comm.barrier()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    launches0 = comm.launches
    evs[0].record()
    for i in range(steps):
        fn(warmup + i)
        if per_step_events or i == steps - 1:
            evs[i + 1].record()
    torch.cuda.synchronize()
    comm.barrier()
    comm.check()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)] if per_step_events else []
    total = evs[0].elapsed_time(evs[steps])
    time_steps.launches = comm.launches - launches0  # kernels this process launched inside the timed region
    return gather_max(comm, total), per


def time_steps_batched(comm, torch, fn, steps: int):
    """`steps` calls back to back with ONE event pair; returns (total_ms max over ranks, None)."""
    comm.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    comm.barrier()
    comm.check()
    return gather_max(comm, e0.elapsed_time(e1)), None


def percentile(xs, q):
    s = sorted(xs)
    if not s:
        return None
    k = min(len(s) - 1, max(0, int(round(q / 100.0 * (len(s) - 1)))))
    return s[k]


def run_nccl_arm(comm, n_gpus: int) -> dict:
    """NCCL on the same GPUs with the same timing code as the library's own C++ benchmark
    (bench/benchmark_nccl_mpi.cu: one process per GPU, CUDA events / one CUDA graph, max over ranks).
    Every rank of this job starts one rank of that binary; this job's GPUs are idle meanwhile."""
    if n_gpus < 2:
        return {"unavailable": "NCCL needs at least two GPUs"}
    exe = ROOT / "build" / "bin" / "benchmark_nccl_mpi"
    if not exe.exists():
        if int(os.environ.get("LOCAL_RANK", "0")) == 0:
            subprocess.run(["make", "-C", str(ROOT), "build/bin/benchmark_nccl_mpi"], capture_output=True, text=True)
        comm.barrier()
    if not exe.exists():
        return {"unavailable": "build/bin/benchmark_nccl_mpi is not built (make bench)"}
    env = dict(os.environ)
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 23)
    env["YALI_WARMUP"] = "20"
    out = {}
    for key, argv in (("busbw_128MiB_fp32", [str(MESSAGE_BYTES // 4), "20", "0", "auto", "0", "cuda-events", "fp32"]),
                      ("latency_1MiB", [str((1 << 20) // 4), "1000", "0", "auto", "0", "graph", "fp32"])):
        comm.barrier()
        try:
            r = subprocess.run([str(exe)] + argv, capture_output=True, text=True, timeout=300, env=env)
        except subprocess.TimeoutExpired:
            out[key] = {"unavailable": "timed out"}
            continue
        line = next((ln for ln in r.stdout.splitlines() if ln.startswith("{")), None)
        if r.returncode != 0 or (comm.rank == 0 and line is None):
            out[key] = {"unavailable": (r.stderr.strip() or r.stdout.strip())[-160:].replace("\n", " ")}
        elif line is not None:
            d = json.loads(line)
            out[key] = {"avg_us": d.get("avg_us"), "busbw_gbps": d.get("busbw_gbps"), "timing": d.get("timing")}
    out["how"] = "bench/benchmark_nccl_mpi.cu (ncclAllReduce, out of place, system libnccl), one process per GPU"
    return out


def run_own(args) -> dict:
    import torch

    import yali_b200 as yali
    from yali_b200 import _native

    n_gpus = args.gpus
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    elems = MESSAGE_BYTES // 4
    heap = 3 << 30
    emulated = n_gpus == 1
    if emulated:
        comm = yali.Comm.emulated(2, device=0, heap_bytes=heap)
        ranks = 2
    else:
        if world_env != n_gpus:
            raise SystemExit(f"--gpus {n_gpus} needs a launcher that starts {n_gpus} ranks (WORLD_SIZE={world_env})")
        comm = yali.Comm.from_env(heap_bytes=heap)
        ranks = n_gpus
    rank = comm.rank
    ext = _native.ext()
    aslist = (lambda t: t if isinstance(t, list) else [t])

    send = comm.symm_empty(elems, torch.float32)
    recv = comm.symm_empty(elems, torch.float32)
    for i, t in enumerate(aslist(send)):
        ext.fill_random(t, 0, 1234 + (i if emulated else rank))

    # ---- headline: 128 MiB fp32, device-timed ----
    sampler = ClockSampler(comm.device)

    def step(_i):
        comm.all_reduce(send, recv)

    if rank == 0:
        sampler.start()  # runs across all timed regions below (each alone is shorter than one sample period)
    total_ms, per = time_steps(comm, torch, step, args.steps, args.warmup, per_step_events=False)
    launches = time_steps.launches * (1 if emulated else ranks)  # every rank launches the same count
    variant = comm.last_call()
    ok = all(ext.validate_sum(t, torch.float32, 0, 1234, ranks)["mismatches"] == 0 for t in aslist(recv))
    ms_per_step = total_ms / args.steps
    busbw = MESSAGE_BYTES * bus_factor(ranks) / (ms_per_step * 1e-3) / 1e9

    # ---- latency at 1 MiB: rotate over 160 buffer pairs (320 MiB touched > L2) ----
    small = (1 << 20) // 4
    nbuf = 160
    pool_s = comm.symm_empty(small * nbuf, torch.float32)
    pool_r = comm.symm_empty(small * nbuf, torch.float32)
    views_s = [[t[k * small:(k + 1) * small] for t in aslist(pool_s)] for k in range(nbuf)]
    views_r = [[t[k * small:(k + 1) * small] for t in aslist(pool_r)] for k in range(nbuf)]
    unwrap = (lambda v: v if emulated else v[0])

    def small_step(i):
        comm.all_reduce(unwrap(views_s[i % nbuf]), unwrap(views_r[i % nbuf]))

    # Event pair per call (contains host launch jitter): kept for comparison only.
    ev_steps = 200
    _, lat = time_steps(comm, torch, small_step, ev_steps, max(args.warmup, 20))
    ev_p50, ev_p99 = gather_max(comm, percentile(lat, 50)), gather_max(comm, percentile(lat, 99))
    # The same calls without an event between them.
    batch_ms, _ = time_steps_batched(comm, torch, small_step, ev_steps)
    # 1000 calls in ONE CUDA graph (no host work between the kernels) with the device-side timeline on:
    # per call, duration = first CTA in -> last CTA out and cadence = end of the previous call -> end of
    # this call (what an event pair per call would see on a host without jitter).
    lat_steps = 1000
    comm.set_trace(True)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(lat_steps):
                small_step(i)
    comm.set_trace(False)
    graph.replay()
    torch.cuda.synchronize()
    comm.barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    graph.replay()
    g1.record()
    torch.cuda.synchronize()
    comm.barrier()
    comm.check()
    graph_us = gather_max(comm, g0.elapsed_time(g1) * 1e3 / lat_steps)
    # Per rank: cadence = end of the previous call -> end of this call (the time per call a stream of
    # calls sees), duration = first CTA in -> last CTA out.  Percentiles per rank, then the max over ranks
    # of each percentile (taking the max call by call would add the ranks' phase jitter to every sample).
    p50 = p99 = d50 = d99 = 0.0
    for li in range(len(aslist(send))):
        _calls, entries = comm.read_trace(li, lat_steps)
        assert len(entries) == lat_steps, (len(entries), lat_steps)
        dur = [(t1 - t0) * 1e-3 for (t0, t1) in entries]
        cad = [(entries[c][1] - entries[c - 1][1]) * 1e-3 for c in range(1, lat_steps)]
        p50, p99 = max(p50, percentile(cad, 50)), max(p99, percentile(cad, 99))
        d50, d99 = max(d50, percentile(dur, 50)), max(d99, percentile(dur, 99))
    p50, p99, d50, d99 = (gather_max(comm, v) for v in (p50, p99, d50, d99))
    del graph
    small_variant = comm.last_call()

    # ---- end to end through the public API: pinned H2D, all-reduce, D2H of the result ----
    n_local = len(aslist(send))
    h_in = [torch.empty(elems, dtype=torch.float32).pin_memory() for _ in range(n_local)]
    h_out = [torch.empty(elems, dtype=torch.float32).pin_memory() for _ in range(n_local)]
    for h, t in zip(h_in, aslist(send)):
        h.copy_(t)

    # The user's call for data that lives on the host: every step copies the whole input in from
    # pinned memory and the whole result out; the copies of both directions and the all-reduce
    # overlap chunk by chunk inside the call.
    def e2e_step(_i):
        comm.all_reduce_host(h_in if n_local > 1 else h_in[0], h_out if n_local > 1 else h_out[0])

    def copies_step(_i):
        comm.all_reduce_host(h_in if n_local > 1 else h_in[0], h_out if n_local > 1 else h_out[0], copies_only=True)

    e2e_steps = max(3, min(args.steps, 20))
    e2e_ms, _ = time_steps(comm, torch, e2e_step, e2e_steps, 3)
    e2e_busbw = MESSAGE_BYTES * bus_factor(ranks) / (e2e_ms / e2e_steps * 1e-3) / 1e9
    e2e_launches = time_steps.launches
    # The same host <-> device copies on the same streams without the collective: what the host link
    # allows for this step on this machine (all ranks copy at once).  Measured after the real step.
    copies_ms, _ = time_steps(comm, torch, copies_step, e2e_steps, 2)
    e2e_step(0)  # leave the reduced result in h_out for the check below
    torch.cuda.synchronize()
    comm.barrier()
    ok = ok and bool(torch.allclose(h_out[0], aslist(recv)[0].cpu(), rtol=1e-5, atol=1e-5))
    # Keep the GPU under the headline load until the sampler has a few readings.
    # (Same count on every rank: it is derived from the max-over-ranks step time.)
    for _ in range(max(1, min(5000, int(0.4 / max(ms_per_step * 1e-3, 1e-6))))):
        step(0)
    torch.cuda.synchronize()
    comm.barrier()
    clocks = sampler.stop() if rank == 0 else {}
    nccl = run_nccl_arm(comm, n_gpus)
    comm.close()

    return {
        "metric": "allreduce_busbw_GBps_128MiB_fp32",
        "value": round(busbw, 2),
        "unit": "GB/s",
        "n_gpus": n_gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 5),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(busbw / BASELINE_GBPS_128MB, 3),
        "dtype": "fp32",
        "data": "synthetic U(-1,1), seed 1234+rank; result verified on device: " + ("ok" if ok else "MISMATCH"),
        "impl": "yali_b200",
        "config": {
            "model": "sum all-reduce, 128 MiB fp32 per rank, pre-allocated symmetric buffers",
            "global_batch": MESSAGE_BYTES * ranks,
            "seq_len": elems,
            "parallelism": ("1 GPU: 2 ranks emulated in one cooperative launch (HBM-bound, no NVLink)" if emulated
                            else f"{ranks} ranks, one GPU per process"),
            "l2": "inputs (128 MiB per rank) larger than L2; 1 MiB latency rotates over 320 MiB of buffers",
            "metric_note": "busBw = bytes per rank x 2(N-1)/N / time: a per-link rate that ideal scaling keeps "
                           "CONSTANT as N grows (the job reduces N x 128 MiB per step); the 1-GPU figure moves "
                           "no bytes over NVLink and is bound by HBM",
            "kernel": variant,
            "baseline": "reference README: 79.2 GB/s at 128 MB fp32 on 2x A100 NV4",
        },
        "latency_1MiB_us": {"p50": round(p50, 2), "p99": round(p99, 2),
                            "p99_over_p50": round(p99 / p50, 3) if p50 else None, "samples": lat_steps - 1,
                            "kernel_p50": round(d50, 2), "kernel_p99": round(d99, 2),
                            "kernel_p99_over_p50": round(d99 / d50, 3) if d50 else None,
                            "avg_back_to_back": round(batch_ms * 1e3 / ev_steps, 2),
                            "avg_cuda_graph": round(graph_us, 2),
                            "host_event_p50": round(ev_p50 * 1e3, 2), "host_event_p99": round(ev_p99 * 1e3, 2),
                            "kernel": small_variant,
                            "note": "p50/p99: 1000 calls replayed from one CUDA graph; every kernel stamps "
                                    "%globaltimer at first-CTA entry and last-CTA exit; sample = end of previous call "
                                    "to end of this call on one rank (kernel_*: entry to exit); percentiles per rank, "
                                    "then the max over ranks; "
                                    "host_event_*: one CUDA event pair per call from Python (contains host jitter); "
                                    "the averages: one event pair around all calls"},
        "e2e": {"value": round(e2e_busbw, 2), "unit": "GB/s", "h2d_bytes_per_step": MESSAGE_BYTES * n_local,
                "d2h_bytes_per_step": MESSAGE_BYTES * n_local, "steps": e2e_steps,
                "ms_per_step": round(e2e_ms / e2e_steps, 3),
                "copies_only_ms_per_step": round(copies_ms / e2e_steps, 3),
                "fraction_of_copies_only": round(copies_ms / e2e_ms, 3) if e2e_ms else None,
                "gpu_launches": int(e2e_launches * (1 if emulated else ranks)),
                "api": "Comm.all_reduce_host(pinned_in, pinned_out): H2D, all-reduce and D2H of 4 MiB chunks "
                       "overlap on three streams; copies_only = the same copies without the collective, all "
                       "ranks at once (the ceiling of the host link)"},
        "nccl": nccl,
        "gpu_launches": int(launches),
        "clocks": clocks,
    }


def run_reference(args) -> dict:
    """The unmodified reference, through its own benchmark binary (device-timed number) and its
    own ops API inside a small timing harness (end-to-end number).  It supports exactly two
    GPUs driven by one process, so only rank 0 of a 2-rank launch runs it."""
    ref_dir = ROOT / "baseline" / "_ref"
    rank = int(os.environ.get("RANK", "0"))
    if args.gpus != 2:
        return {"impl": "reference",
                "unavailable": f"the reference runs on exactly 2 GPUs (asked for {args.gpus}): "
                               "src/ops/allreduce_mpi.cuh:113-118, README.md:199-203"}
    binary, harness = ref_dir / "benchmark_yali", ref_dir / "ref_e2e"
    if not binary.exists() or not harness.exists():
        return {"impl": "reference", "unavailable": "baseline/_ref is not built (run baseline/build_reference.sh)"}
    if rank != 0:
        return {}
    elems = MESSAGE_BYTES // 4
    sampler = ClockSampler(0)
    sampler.start()
    # argv: elements calls verify mode lanes timing dtype (bench/benchmark_yali.cu:764-789); its
    # warm-up count is fixed at 100 calls in the source.
    try:
        out = subprocess.run([str(binary), str(elems), str(args.steps), "0", "auto", "0", "cuda-events", "fp32"],
                             capture_output=True, text=True, timeout=600)
    except subprocess.TimeoutExpired:
        sampler.stop()
        return {"impl": "reference", "unavailable": "reference benchmark_yali did not finish within 600 s"}
    clocks = sampler.stop()
    import re
    # Flash prints "... us/call avg, Y GB/s (Z% SoL)", Stream prints "... us/call, Y GB/s, Z% SoL".
    m = re.search(r"YALI \(([^)]*)\): (\d+) calls, ([\d.]+) us/call(?: avg)?, ([\d.]+) GB/s", out.stdout)
    if out.returncode != 0 or not m:
        return {"impl": "reference", "unavailable": "reference benchmark_yali failed: " +
                (out.stderr.strip() or out.stdout.strip())[-200:].replace("\n", " ")}
    us, gbps = float(m.group(3)), float(m.group(4))
    small = subprocess.run([str(binary), str((1 << 20) // 4), "1000", "0", "auto", "0", "cuda-events", "fp32"],
                           capture_output=True, text=True, timeout=600)
    ms = re.search(r"([\d.]+) us/call(?: avg)?, ([\d.]+) GB/s", small.stdout)
    # The reference's own NCCL benchmark (bench/benchmark_nccl.cu, argv: elements calls timing dtype), the
    # comparator its README quotes: one process, two communicators, event pair on GPU 0.
    ref_nccl = {}
    nccl_bin = ref_dir / "benchmark_nccl"
    if nccl_bin.exists():
        for key, n, calls in (("busbw_128MiB_fp32", elems, args.steps), ("latency_1MiB", (1 << 20) // 4, 1000)):
            try:
                rn = subprocess.run([str(nccl_bin), str(n), str(calls), "cuda-events", "fp32"], capture_output=True,
                                    text=True, timeout=600)
                mn = re.search(r"NCCL \([^)]*\): (\d+) calls, ([\d.]+) us/call avg, ([\d.]+) GB/s", rn.stdout)
                ref_nccl[key] = ({"avg_us": float(mn.group(2)), "busbw_gbps": float(mn.group(3))} if mn else
                                 {"unavailable": (rn.stderr.strip() or rn.stdout.strip())[-160:].replace("\n", " ")})
            except subprocess.TimeoutExpired:
                ref_nccl[key] = {"unavailable": "timed out"}
        ref_nccl["how"] = "the reference's bench/benchmark_nccl.cu built unmodified against the system libnccl"
    else:
        ref_nccl = {"unavailable": "baseline/_ref/benchmark_nccl is not built"}
    e2e = subprocess.run([str(harness), str(elems), str(max(3, min(args.steps, 20))), "3"], capture_output=True,
                         text=True, timeout=600)
    me = re.search(r"REF_E2E fp32 (\d+) (\d+) (\d+) ([\d.]+) ([\d.]+)", e2e.stdout)
    e2e_val = MESSAGE_BYTES / (float(me.group(4)) * 1e-6) / 1e9 if me else None
    return {
        "metric": "allreduce_busbw_GBps_128MiB_fp32", "value": gbps, "unit": "GB/s", "n_gpus": 2,
        "steps": args.steps, "warmup": 100, "ms_per_step": round(us / 1e3, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": round(gbps / BASELINE_GBPS_128MB, 3), "dtype": "fp32",
        "data": "synthetic (the reference's constant fill)", "impl": "reference",
        "config": {"model": "sum all-reduce, 128 MiB fp32 per rank", "global_batch": MESSAGE_BYTES * 2,
                   "seq_len": elems, "parallelism": "2 GPUs, one process (the reference's single-process mode)",
                   "kernel": m.group(1),
                   "note": "reference times with one event pair on GPU 0's first lane stream only "
                           "(bench/benchmark_yali.cu:587-622); warm-up is fixed at 100 calls in its source"},
        "latency_1MiB_us": {"avg": float(ms.group(1)) if ms else None},
        "e2e": {"value": round(e2e_val, 2) if e2e_val else None, "unit": "GB/s",
                "h2d_bytes_per_step": MESSAGE_BYTES * 2, "d2h_bytes_per_step": MESSAGE_BYTES * 2,
                "timing": "wall clock around H2D + yali::allreduce + D2H on both GPUs"},
        "nccl": ref_nccl,
        "gpu_launches": 0, "clocks": clocks,
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    res = run_reference(args) if args.impl == "reference" else run_own(args)
    if int(os.environ.get("RANK", "0")) == 0 and res:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
