"""Control plane between processes on one node, exercised with CPU-only child
processes: rendezvous, allgather / broadcast / barrier, descriptor passing, and the
failures that must end in an error on every rank instead of a hang (a rank that
never joins, a world-size disagreement, ranks in different collectives, a rank that
leaves).

Reference counterpart: the MPI bootstrap (src/comm/comm.cu:67-216) is only tested
through `mpirun -np 2` examples (tests/run_mpi_example.sh); it has no failure tests."""
import ctypes
import multiprocessing as mp
import os
import time

import pytest

from yali_b200 import _native

CTX = mp.get_context("spawn")


def _create(lib, rank, world, job, timeout_ms=10000):
    err = ctypes.create_string_buffer(256)
    bs = lib.yali_c_bootstrap_create(rank, world, rank, job.encode(), timeout_ms, err, 256)
    return bs, err.value.decode()


def _worker_basic(rank, world, job, q):
    lib = _native.lib()
    bs, err = _create(lib, rank, world, job)
    if not bs:
        q.put((rank, "create failed: " + err))
        return
    ok = lib.yali_c_bootstrap_rank(bs) == rank and lib.yali_c_bootstrap_world(bs) == world
    mine = bytes([rank + 1] * 5)
    out = ctypes.create_string_buffer(5 * world)
    ok &= lib.yali_c_bootstrap_allgather(bs, mine, out, 5) == 0
    ok &= out.raw == b"".join(bytes([r + 1] * 5) for r in range(world))
    for root in range(world):
        buf = ctypes.create_string_buffer(bytes([root + 10] * 3) if rank == root else b"\0\0\0", 3)
        ok &= lib.yali_c_bootstrap_broadcast(bs, buf, 3, root) == 0
        ok &= buf.raw == bytes([root + 10] * 3)
    ok &= lib.yali_c_bootstrap_barrier(bs) == 0
    # descriptor passing: every rank shares a pipe; rank r writes into the pipe of rank (r+1)%world
    rd, wr = os.pipe()
    fds = (ctypes.c_int * world)()
    ok &= lib.yali_c_bootstrap_allgather_fd(bs, wr, fds) == 0
    os.write(fds[(rank + 1) % world], bytes([100 + rank]))
    ok &= lib.yali_c_bootstrap_barrier(bs) == 0
    got = os.read(rd, 1)
    ok &= got == bytes([100 + (rank - 1) % world])
    one = ctypes.c_int(wr if rank == 0 else -1)
    ok &= lib.yali_c_bootstrap_broadcast_fd(bs, ctypes.byref(one)) == 0
    if rank == 1:
        os.write(one.value, b"Z")
    ok &= lib.yali_c_bootstrap_barrier(bs) == 0
    if rank == 0:
        ok &= os.read(rd, 1) == b"Z"
    lib.yali_c_bootstrap_destroy(bs)
    q.put((rank, "ok" if ok else "mismatch"))


def _run(target, world, extra=(), timeout=60):
    q = CTX.Queue()
    job = f"t{os.getpid()}-{time.time_ns()}"
    procs = [CTX.Process(target=target, args=(r, world, job, q) + tuple(extra)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    deadline = time.time() + timeout
    while len(res) < len(procs) and time.time() < deadline:
        try:
            r, msg = q.get(timeout=0.5)
            res[r] = msg
        except Exception:  # noqa: BLE001
            if all(not p.is_alive() for p in procs) and q.empty():
                break
    for p in procs:
        p.join(5)
        if p.is_alive():
            p.kill()
    return res


@pytest.mark.parametrize("world", [2, 4, 8])
def test_collectives_and_fd_passing(world):
    res = _run(_worker_basic, world)
    assert res == {r: "ok" for r in range(world)}


def _worker_missing(rank, world, job, q):
    lib = _native.lib()
    if rank == world - 1:
        q.put((rank, "absent"))  # this rank never joins
        return
    t0 = time.time()
    bs, err = _create(lib, rank, world, job, timeout_ms=1500)
    q.put((rank, f"{'created' if bs else 'error'}:{time.time() - t0:.1f}:{err}"))


def test_rank_that_never_joins_gives_error_not_hang():
    res = _run(_worker_missing, 3)
    assert res[2] == "absent"
    for r in (0, 1):
        kind, secs, _ = res[r].split(":", 2)
        assert kind == "error" and float(secs) < 10


def _worker_world_mismatch(rank, world, job, q):
    lib = _native.lib()
    claimed = world if rank == 0 else world + 1
    bs, err = _create(lib, rank, claimed, job, timeout_ms=1500)
    q.put((rank, "created" if bs else "error"))


def test_world_size_disagreement_is_rejected():
    res = _run(_worker_world_mismatch, 2)
    assert res == {0: "error", 1: "error"}


def _worker_divergent(rank, world, job, q):
    lib = _native.lib()
    bs, err = _create(lib, rank, world, job, timeout_ms=2000)
    if not bs:
        q.put((rank, "create failed"))
        return
    out = ctypes.create_string_buffer(64)
    if rank == 1:
        rc = lib.yali_c_bootstrap_allgather(bs, b"12345678", out, 8)  # the others send 4 bytes
    else:
        rc = lib.yali_c_bootstrap_allgather(bs, b"1234", out, 4)
    msg = lib.yali_c_bootstrap_last_error(bs).decode()
    q.put((rank, f"{rc}:{msg}"))


def test_mismatched_collective_fails_cleanly():
    res = _run(_worker_divergent, 3)
    assert len(res) == 3
    rc0, msg0 = res[0].split(":", 1)
    assert int(rc0) != 0 and "different collective" in msg0
    assert all(int(v.split(":", 1)[0]) != 0 for v in res.values())


def _worker_leaver(rank, world, job, q):
    lib = _native.lib()
    bs, err = _create(lib, rank, world, job, timeout_ms=2000)
    if not bs:
        q.put((rank, "create failed"))
        return
    lib.yali_c_bootstrap_barrier(bs)
    if rank == 1:
        q.put((rank, "left"))
        q.close()
        q.join_thread()
        os._exit(0)  # leaves between steps, nothing in flight
    t0 = time.time()
    rc = lib.yali_c_bootstrap_barrier(bs)
    q.put((rank, f"{rc}:{time.time() - t0:.1f}"))


def test_rank_that_leaves_is_detected():
    res = _run(_worker_leaver, 3)
    assert res[1] == "left"
    for r in (0, 2):
        rc, secs = res[r].split(":")
        assert int(rc) != 0 and float(secs) < 10


def _worker_env(rank, world, job, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), YALI_JOB_ID=job)
    lib = _native.lib()
    err = ctypes.create_string_buffer(256)
    ok = True
    for _ in range(2):  # two communicators in a row use distinct socket names
        bs = lib.yali_c_bootstrap_from_env(err, 256)
        ok &= bool(bs) and lib.yali_c_bootstrap_barrier(bs) == 0
        if bs:
            lib.yali_c_bootstrap_destroy(bs)
    q.put((rank, "ok" if ok else "fail:" + err.value.decode()))


def test_environment_rendezvous_twice():
    assert _run(_worker_env, 2) == {0: "ok", 1: "ok"}


def test_self_bootstrap_without_env(native_lib, monkeypatch):
    for k in ("RANK", "WORLD_SIZE", "OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID"):
        monkeypatch.delenv(k, raising=False)
    err = ctypes.create_string_buffer(64)
    bs = native_lib.yali_c_bootstrap_from_env(err, 64)
    assert bs and native_lib.yali_c_bootstrap_world(bs) == 1 and native_lib.yali_c_bootstrap_barrier(bs) == 0
    out = ctypes.create_string_buffer(4)
    assert native_lib.yali_c_bootstrap_allgather(bs, b"abcd", out, 4) == 0 and out.raw == b"abcd"
    native_lib.yali_c_bootstrap_destroy(bs)
