"""Tensor-parallel output projection in one kernel per rank.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/03_python/tp_layer.py
    python examples/03_python/tp_layer.py --emulate 2          # two ranks on one GPU

Every rank holds a [T, 4096/W] slice of the activations and a [4096, 4096/W] slice of the
weight (nn.Linear layout); the result RMSNorm(residual + sum_r x_r @ W_r^T) * g lands in every
rank's `out`.  The reference has no such layer; this is the fused path that the tensor-parallel
modules of `yali_b200.parallel.tensor_parallel` use.
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))  # run from a checkout without installing
import yali_b200 as yali  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--emulate", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=256)
    args = ap.parse_args()
    comm = yali.Comm.emulated(args.emulate) if args.emulate else yali.Comm.from_env()
    W, N, T = comm.world, 4096, args.tokens
    K = N // W
    ranks = list(range(W)) if args.emulate else [comm.rank]
    dev = [f"cuda:{d}" for d in comm.devices]
    gens = {r: torch.Generator().manual_seed(100 + r) for r in range(W)}
    x_all = {r: torch.randn(T, K, generator=gens[r]).to(torch.bfloat16) for r in range(W)}
    w_all = {r: (torch.randn(N, K, generator=gens[r]) * 0.02).to(torch.bfloat16) for r in range(W)}
    res = torch.randn(T, N, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
    g = torch.ones(N, dtype=torch.bfloat16)

    xs = [x_all[r].to(dev[i]) for i, r in enumerate(ranks)]
    ws = [w_all[r].to(dev[i]) for i, r in enumerate(ranks)]
    one = (lambda v: v[0]) if len(ranks) == 1 else (lambda v: v)
    out = comm.symm_empty([T, N], torch.bfloat16)  # symmetric: the row owners write into every rank's copy
    comm.fused_linear_rmsnorm(one(xs), one(ws), one([g.to(d) for d in dev]), one([res.to(d) for d in dev]), out=out)
    comm.sync()
    comm.barrier()

    h = sum(x_all[r].float() @ w_all[r].float().T for r in range(W)) + res.float()
    want = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)
    got = (out[0] if isinstance(out, list) else out).float().cpu()
    err = (got - want).abs().max().item()
    if comm.rank == 0:
        print(f"world {W}, T {T}: max |fused - fp32 reference| = {err:.4f}")
    comm.close()


if __name__ == "__main__":
    main()
