"""All-reduce of data that lives in pinned host memory.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/03_python/host_allreduce.py
    python examples/03_python/host_allreduce.py --emulate 2

`all_reduce_host` cuts the message into chunks and overlaps the host-to-device copy of chunk
i+1, the all-reduce of chunk i and the device-to-host copy of chunk i-1 on three streams.
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
    ap.add_argument("--mib", type=int, default=64)
    args = ap.parse_args()
    comm = yali.Comm.emulated(args.emulate) if args.emulate else yali.Comm.from_env()
    n = args.mib * (1 << 20) // 4
    ranks = list(range(comm.world)) if args.emulate else [comm.rank]
    src = [torch.full((n,), float(r + 1)).pin_memory() for r in ranks]
    dst = [torch.empty(n).pin_memory() for _ in ranks]
    one = (lambda v: v[0]) if len(ranks) == 1 else (lambda v: v)
    comm.all_reduce_host(one(src), one(dst))
    torch.cuda.synchronize()
    comm.check()
    want = comm.world * (comm.world + 1) / 2
    ok = all(bool((d == want).all()) for d in dst)
    if comm.rank == 0:
        print(f"{args.mib} MiB per rank, world {comm.world}: every element == {want}: {ok}")
    comm.close()


if __name__ == "__main__":
    main()
