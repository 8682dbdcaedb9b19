#!/usr/bin/env python
"""Size sweep of the all-reduce variants against NCCL on the same GPUs.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/sweep.py \
        [--min-bytes 4096] [--max-bytes 2147483648] [--dtypes fp32,bf16] \
        [--variants auto,flash,stream,nvls,stream_direct] [--torch-nccl] [--out sweep.jsonl] [--tuning-out tuning.json]

Every (size, dtype, variant) is timed on the device (CUDA events around the timed
calls on the launching stream, 20 warm-up calls, barrier + synchronize on both
sides, max over ranks) and reported as NCCL-convention bus bandwidth; small
messages rotate over buffers that together exceed L2.  Every row also carries the
device-side timeline of the timed calls (the kernels stamp their own start and end):
p50 / p99 / max of the time per call without host jitter, call by call the max over
ranks.  The NCCL baseline of a campaign comes from build/bin/nccl_sweep (same timing
code in C++, started by bench/run_sweep.py); `--torch-nccl` additionally times
torch.distributed.all_reduce with this file's loop (rows of impl "nccl_torch": the
Python binding of NCCL costs several microseconds per call inside a CUDA graph, so
these rows are context, not the baseline).
`--tuning-out` writes the fastest variant per size as a table the library loads
through YALI_TUNING_FILE.

Reference counterpart: scripts/sweep.py (phases 'YALI/NCCL x single/MPI sweeps'),
which shells out to the benchmark binaries and regexes their stdout."""
from __future__ import annotations

import argparse
import json
import struct
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import yali_b200 as yali  # noqa: E402

DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
L2_BYTES = 126 << 20


def gather_max(comm, v: float) -> float:
    if comm.world == 1 or comm.nlocal != 1:
        return v
    return max(struct.unpack("d", p)[0] for p in comm.allgather_object_bytes(struct.pack("d", v)))


def timed(comm, fn, iters: int, warmup: int, graph: bool = False) -> float:
    """Average microseconds per call, max over ranks.  graph=True captures the `iters` calls in one CUDA
    graph and times one replay (after one untimed replay): no host launch work between the kernels."""
    for i in range(warmup):
        fn(i)
    comm.barrier()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(iters):
                    fn(warmup + i)
        g.replay()
        torch.cuda.synchronize()
        comm.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        comm.barrier()
        del g
        return gather_max(comm, e0.elapsed_time(e1) * 1e3 / iters)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    comm.barrier()
    return gather_max(comm, e0.elapsed_time(e1) * 1e3 / iters)


def device_times(comm, iters: int) -> dict:
    """p50 / p99 / max microseconds of the last `iters` traced calls (first CTA in -> last CTA out), call by
    call the max over ranks."""
    n = min(iters, 4096)
    dur = [0.0] * n
    for li in range(comm.nlocal):
        _calls, entries = comm.read_trace(li, n)
        if len(entries) != n:
            return {}
        for c, (t0, t1) in enumerate(entries):
            dur[c] = max(dur[c], (t1 - t0) * 1e-3)
    if comm.nlocal == 1 and comm.world > 1:
        for p in comm.allgather_object_bytes(struct.pack(f"{n}d", *dur)):
            dur = [max(x, y) for x, y in zip(dur, struct.unpack(f"{n}d", p))]
    s = sorted(dur)
    pick = (lambda q: s[min(n - 1, int(round(q * (n - 1))))])
    return {"dev_p50_us": round(pick(0.5), 2), "dev_p99_us": round(pick(0.99), 2), "dev_max_us": round(s[-1], 2),
            "dev_samples": n}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--dtypes", default="fp32")
    ap.add_argument("--variants", default="auto,flash,stream,nvls,stream_direct")
    ap.add_argument("--torch-nccl", dest="nccl", action="store_true")
    ap.add_argument("--emulate", type=int, default=0, help="emulate this many ranks on one GPU (no launcher)")
    ap.add_argument("--out", default="")
    ap.add_argument("--tuning-out", default="")
    ap.add_argument("--iters", type=int, default=0, help="0: scaled by size")
    ap.add_argument("--graph-max-bytes", type=int, default=0,
                    help="sizes up to this are timed as one CUDA-graph replay of all calls (both arms)")
    args = ap.parse_args()

    heap = 2 * args.max_bytes + (3 << 30)
    if args.emulate:
        comm = yali.Comm.emulated(args.emulate, heap_bytes=heap)
    else:
        comm = yali.Comm.from_env(heap_bytes=heap)
    world, rank = comm.world, comm.rank
    emu = bool(args.emulate)
    lst = (lambda t: t if isinstance(t, list) else [t])
    if args.nccl and not emu:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", comm.device))
    factor = 2.0 * (world - 1) / world
    variants = [v for v in args.variants.split(",") if v]
    rows, best = [], {}
    out_f = open(args.out, "w") if (args.out and rank == 0) else None
    pool_bytes = max(args.max_bytes, L2_BYTES * 2 + (64 << 20))
    comm.symm_reset()
    pool_s = comm.symm_empty(pool_bytes, torch.uint8)
    pool_r = comm.symm_empty(pool_bytes, torch.uint8)

    for dname in args.dtypes.split(","):
        dt = DT[dname]
        esz = torch.empty(0, dtype=dt).element_size()
        for t in lst(pool_s):
            t.view(dt).normal_()
        size = args.min_bytes
        while size <= args.max_bytes:
            n = size // esz
            nbuf = max(1, min(256, (2 * L2_BYTES) // size)) if size < L2_BYTES else 1
            views_s = [[t[k * size:(k + 1) * size].view(dt) for t in lst(pool_s)] for k in range(nbuf)]
            views_r = [[t[k * size:(k + 1) * size].view(dt) for t in lst(pool_r)] for k in range(nbuf)]
            pick = (lambda v: v if emu else v[0])
            iters = args.iters or (200 if size <= (1 << 20) else 50 if size <= (64 << 20) else 15)
            for var in variants:
                def call(i, var=var):
                    comm.all_reduce(pick(views_s[i % nbuf]), pick(views_r[i % nbuf]), mode=var)
                try:
                    comm.set_trace(True)
                    us = timed(comm, call, iters, 20 if size <= (16 << 20) else 5, graph=size <= args.graph_max_bytes)
                    comm.set_trace(False)
                    comm.check()
                except RuntimeError as e:
                    comm.set_trace(False)
                    if "cannot run" in str(e) or "Unsupported" in str(e):
                        continue
                    raise
                lc = comm.last_call()
                row = {"impl": "yali_b200", "world": world, "dtype": dname, "bytes": size, "variant": var,
                       "kernel": lc["variant"], "ctas": lc["ctas"], "slot_bytes": lc["slot_bytes"], "us": round(us, 2),
                       "busbw_gbps": round(size * factor / us / 1e3, 2), "emulated": emu,
                       "timing": "graph" if size <= args.graph_max_bytes else "events"}
                row.update(device_times(comm, iters))
                rows.append(row)
                if var != "auto":
                    key = (dname, size)
                    if key not in best or us < best[key]["us"]:
                        best[key] = row
                if rank == 0:
                    print(json.dumps(row), flush=True)
                    if out_f:
                        out_f.write(json.dumps(row) + "\n")
            if args.nccl and not emu:
                import torch.distributed as dist
                bufs = [v[0].clone() for v in views_s] if size <= (64 << 20) else [views_r[0][0]]

                def ncall(i):
                    dist.all_reduce(bufs[i % len(bufs)])
                us = timed(comm, ncall, iters, 20 if size <= (16 << 20) else 5, graph=size <= args.graph_max_bytes)
                row = {"impl": "nccl_torch", "world": world, "dtype": dname, "bytes": size, "variant": "nccl_torch",
                       "us": round(us, 2), "busbw_gbps": round(size * factor / us / 1e3, 2),
                       "timing": "graph" if size <= args.graph_max_bytes else "events"}
                if rank == 0:
                    print(json.dumps(row), flush=True)
                    if out_f:
                        out_f.write(json.dumps(row) + "\n")
                del bufs
            size *= 2
    if args.tuning_out and rank == 0:
        trows = []
        for (dname, size), row in sorted(best.items(), key=lambda kv: (kv[0][0], kv[0][1])):
            name = row["kernel"]  # flash, stream, nvls1, nvls2, flash_pull, stream_direct: the planner's names
            trows.append({"world": world, "elem_bytes": 4 if dname == "fp32" else 2, "max_bytes": size,
                          "variant": name, "ctas": 0, "slot_bytes": 0, "busbw": row["busbw_gbps"]})
        Path(args.tuning_out).write_text(json.dumps({"rows": trows}, indent=1))
    if out_f:
        out_f.close()
    if args.nccl and not emu:
        import torch.distributed as dist
        dist.destroy_process_group()
    comm.close()


if __name__ == "__main__":
    main()
