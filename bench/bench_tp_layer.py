#!/usr/bin/env python
"""Tensor-parallel output projection + all-reduce + residual + RMSNorm: fused kernel vs
the unfused compositions, on the Llama-3-8B shapes (hidden 4096, K = 4096 / TP per rank,
bf16, W ~ N(0, 0.02), x ~ N(0, 1), eps 1e-5), T in {1, 16, 128, 2048}.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/bench_tp_layer.py
    python bench/bench_tp_layer.py --emulate 8         # one GPU, ranks emulated (no NVLink)

Arms: `fused_*` = one kernel per rank (tcgen05 GEMM, peer pushes, reduce + norm): the 128 x 128
tile form one-shot / two-shot (peer stores, in-switch reduce, multicast delivery), `fused_decode` =
the few-token form (T <= 64), `fused_auto` = the form RowParallelLinearNorm picks by size;
`gemm+ar_norm` = library GEMM, then this library's all-reduce fused with residual +
RMSNorm; `nccl` = library GEMM, NCCL all-reduce, PyTorch residual + RMSNorm (the baseline;
not available with --emulate).  Times are device times (CUDA events, max over ranks).
The roofline is the slower of the GEMM at the measured bf16 peak and the bytes one rank
must send over NVLink at the measured 770 GB/s per direction."""
from __future__ import annotations

import argparse
import json
import struct
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import yali_b200 as yali  # noqa: E402
from yali_b200.parallel import tensor_parallel as tp  # noqa: E402

LINK_GBS = 770.0


def peaks():
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("bf16_tflops", 1590.0), "measured"
    return 1590.0, "fallback"


def gather_max(comm, v):
    if comm.world == 1 or comm.nlocal != 1:
        return v
    return max(struct.unpack("d", p)[0] for p in comm.allgather_object_bytes(struct.pack("d", v)))


def timed(comm, fn, iters, warmup=10, graph=False):
    for _ in range(warmup):
        fn()
    comm.barrier()
    torch.cuda.synchronize()
    if graph:  # all calls in one CUDA graph, one replay timed: no host work between the kernels
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for _ in range(iters):
                    fn()
        g.replay()
        torch.cuda.synchronize()
        comm.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        comm.barrier()
        comm.check()
        return gather_max(comm, e0.elapsed_time(e1) * 1e3 / iters)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    comm.barrier()
    comm.check()
    return gather_max(comm, e0.elapsed_time(e1) * 1e3 / iters)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--emulate", type=int, default=0)
    ap.add_argument("--tokens", default="1,16,128,2048")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--k-per-rank", type=int, default=0,
                    help="K of every rank's slice (default hidden / ranks); lets a 2-rank run use the TP = 8 shape K = 512")
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--graph", action="store_true", help="time one CUDA-graph replay of all calls")
    ap.add_argument("--arms", default="", help="comma list to restrict the arms")
    ap.add_argument("--trace", action="store_true",
                    help="also print the in-kernel timeline of the fused arms (CTA 0 of rank 0: microseconds from "
                         "kernel entry to barriers ready, first accumulator, first tile announced, all tiles done, "
                         "partial rows present, own rows reduced, output complete; the few-token form: entry, barriers "
                         "ready, accumulator complete, all pushes issued and CTA synchronised, rows written, first "
                         "half of the columns stored into the first peer landing zone, this warp pushes issued, first half "
                         "packed and transposed)")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    emu = args.emulate > 0
    comm = yali.Comm.emulated(args.emulate) if emu else yali.Comm.from_env()
    W, rank = comm.world, comm.rank
    N, K = args.hidden, (args.k_per_rank or args.hidden // W)
    tflops, src = peaks()
    use_nccl = not emu
    if use_nccl:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", comm.device))
    nl = comm.nlocal
    dev = [f"cuda:{d}" for d in comm.devices]
    rows = []
    for T in [int(t) for t in args.tokens.split(",")]:
        g = torch.Generator(device="cpu").manual_seed(1234 + rank)
        xs = [torch.randn(T, K, generator=g).to(torch.bfloat16).to(dev[i]) for i in range(nl)]
        ws = [(torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).to(dev[i]) for i in range(nl)]
        nw = [torch.ones(N, dtype=torch.bfloat16, device=dev[i]) for i in range(nl)]
        res = [torch.randn(T, N, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(dev[i])
               for i in range(nl)]
        outs = comm.symm_empty([T, N], torch.bfloat16)
        outs = outs if isinstance(outs, list) else [outs]
        one = (lambda v: v if nl > 1 else v[0])
        arms = {}
        has_nvls = bool(comm.has_multicast) and not comm.emulated_ranks
        for label, oneshot, nvls in (("fused_oneshot", True, 0), ("fused_twoshot", False, 0),
                                     ("fused_twoshot_nvls", False, 1), ("fused_twoshot_mcast", False, 2)):
            if oneshot and T * N * 2 > comm.layout()["gemm_cap"]:
                continue
            if not oneshot and -(-T // W) * N * 2 > comm.layout()["gemm_cap"]:
                continue
            if nvls and not has_nvls:
                continue
            arms[label] = lambda oneshot=oneshot, nvls=nvls: comm.fused_linear_rmsnorm(
                one(xs), one(ws), one(nw), one(res), out=one(outs), oneshot=oneshot, nvls=nvls, decode=False)
        if T <= 64 and W > 1:  # the few-token form: 256-column tiles split along K, partial rows as flag-in-data lines
            arms["fused_decode"] = lambda: comm.fused_linear_rmsnorm(one(xs), one(ws), one(nw), one(res), out=one(outs),
                                                                     decode=True)
        # What RowParallelLinearNorm runs: the form picked by size.
        arms["fused_auto"] = lambda: comm.fused_linear_rmsnorm(one(xs), one(ws), one(nw), one(res), out=one(outs))
        arms["gemm+ar_norm"] = lambda: tp.unfused_row_parallel(comm, xs, ws, nw, res) if nl > 1 else \
            comm.all_reduce_rmsnorm(xs[0] @ ws[0].T, nw[0], res[0])
        if use_nccl:
            def nccl_arm():
                p = xs[0] @ ws[0].T
                dist.all_reduce(p)
                h = p.float() + res[0].float()
                return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16) * nw[0]
            arms["gemm+nccl+norm"] = nccl_arm
        iters = args.iters if T <= 128 else max(20, args.iters // 4)
        flops = 2.0 * T * K * N
        t_gemm = flops / (tflops * 1e12) * 1e6
        bytes_two = 2.0 * (W - 1) / W * T * N * 2
        bytes_one = (W - 1) * T * N * 2.0
        for label, fn in arms.items():
            if args.arms and label not in args.arms.split(","):
                continue
            us = timed(comm, fn, iters, args.warmup, graph=args.graph)
            one_shot_traffic = label in ("fused_oneshot", "fused_decode") or (label == "fused_auto" and T <= 64)
            link_bytes = 0.0 if emu else (bytes_one if one_shot_traffic else bytes_two)
            roof = max(t_gemm, link_bytes / (LINK_GBS * 1e9) * 1e6)
            row = {"T": T, "world": W, "arm": label, "us": round(us, 2), "roofline_us": round(roof, 3),
                   "fraction_of_roofline": round(roof / us, 4), "peaks": src, "emulated": emu,
                   "timing": "graph" if args.graph else "events"}
            if args.trace and label.startswith("fused_"):
                mode = {"fused_oneshot": (True, 0, False), "fused_twoshot": (False, 0, False),
                        "fused_twoshot_nvls": (False, 1, False), "fused_twoshot_mcast": (False, 2, False),
                        "fused_decode": (None, None, True), "fused_auto": (None, None, None)}[label]
                tr = [torch.zeros(8, dtype=torch.int64, device=dev[i]) for i in range(nl)]
                for _ in range(3):
                    comm.fused_linear_rmsnorm(one(xs), one(ws), one(nw), one(res), out=one(outs), oneshot=mode[0],
                                              nvls=mode[1], decode=mode[2], trace=one(tr))
                comm.sync()
                comm.barrier()
                t = tr[0].cpu().tolist()
                row["timeline_us"] = [round((v - t[0]) / 1e3, 1) for v in t]
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
        comm.symm_reset()
    if args.out and rank == 0:
        Path(args.out).write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    if use_nccl:
        import torch.distributed as dist
        dist.destroy_process_group()
    comm.close()


if __name__ == "__main__":
    main()
