"""`python -m yali_b200.launch -np N [--] program args...`: starts N copies of a program
on this node, one per GPU, with RANK / WORLD_SIZE / LOCAL_RANK / YALI_JOB_ID set — what
`mpirun -np N` does for the reference's MPI programs, without needing MPI.  If one rank
exits with an error the others are terminated (by the PIDs this launcher started)."""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="yali_b200.launch")
    ap.add_argument("-np", "--nproc", type=int, required=True)
    ap.add_argument("--job-id", default="")
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    cmd = args.cmd[1:] if args.cmd and args.cmd[0] == "--" else args.cmd
    if not cmd:
        ap.error("no program given")
    job = args.job_id or f"launch{os.getpid()}-{time.time_ns() & 0xffffff}"
    procs = []
    for r in range(args.nproc):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(args.nproc), LOCAL_RANK=str(r), YALI_JOB_ID=job)
        procs.append(subprocess.Popen(cmd, env=env))
    rc = 0
    alive = set(range(args.nproc))
    while alive:
        for r in list(alive):
            code = procs[r].poll()
            if code is None:
                continue
            alive.discard(r)
            if code != 0 and rc == 0:
                rc = code
                for o in alive:
                    procs[o].terminate()
        time.sleep(0.05)
    return rc


if __name__ == "__main__":
    sys.exit(main())
