"""Real peer-to-peer paths: one process driving several GPUs (yali::Comm style) and
one process per GPU (yali::MPIComm style, environment rendezvous + cuMem file
descriptors), including the NVLS kernels when the box offers multicast.  Child
processes run with NCCL_NVLS_ENABLE=0 for any library they load; this library's own
multicast use is exercised only by ranks that all exit in an orderly way.

Reference counterparts: tests/test_ops_allreduce.cu, tests/test_ops_allreduce_mpi.cu."""
import multiprocessing as mp
import os
import time

import pytest
import torch

import yali_b200 as yali
from yali_b200 import _native

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu(2)]
CTX = mp.get_context("spawn")


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worlds():
    n = _ngpu()
    return [w for w in (2, 4, 8) if w <= n] or [2]


def _fill(ts, dist=0, seed=1234, ranks=None):
    ext = _native.ext()
    for i, t in enumerate(ts):
        with torch.cuda.device(t.device):
            ext.fill_random(t, dist, seed + (ranks[i] if ranks else i))


def _check(outs, in_dtype, world, dist=0, seed=1234, scale=1.0):
    ext = _native.ext()
    for o in outs:
        with torch.cuda.device(o.device):
            rep = ext.validate_sum(o, in_dtype, dist, seed, world, scale)
        assert rep["mismatches"] == 0, rep


@pytest.mark.parametrize("world", _worlds())
def test_single_process_all_variants(world):
    with yali.Comm.single_process(list(range(world)), heap_bytes=2 << 30) as comm:
        assert comm.world == world and comm.nlocal == world
        modes = ["flash", "stream", "flash_pull", "stream_direct", "auto"] + (["nvls"] if comm.has_multicast else [])
        for dtype in (torch.float32, torch.bfloat16, torch.float16):
            for n in (1, 33, 4099, 262144, (1 << 21) + 16):
                xs = [torch.empty(n, dtype=dtype, device=f"cuda:{d}") for d in range(world)]
                _fill(xs)
                for mode in modes:
                    if mode == "nvls" and (n * xs[0].element_size()) % 16:
                        continue
                    if mode == "flash" and n * xs[0].element_size() > comm.layout()["flash_cap"]:
                        continue
                    outs = comm.all_reduce(xs, mode=mode)
                    comm.sync()
                    _check(outs, dtype, world)
        # symmetric buffers: zero-copy NVLS and direct all-gather
        n = 1 << 20
        send, recv = comm.symm_empty(n, torch.bfloat16), comm.symm_empty(n, torch.bfloat16)
        _fill(send, dist=1)
        for mode in modes:
            for _ in range(5):  # back to back, no sync
                comm.all_reduce(send, recv, mode=mode)
            comm.sync()
            _check(recv, torch.bfloat16, world, dist=1)
        # in place on symmetric memory: the pipelined two-shot, then (fresh data) a small message through
        # the switch, where the planner must avoid the one-shot form (it would overwrite operands of
        # the peers' multimem.ld_reduce)
        comm.all_reduce(send, send, mode="stream_direct")
        comm.sync()
        _check(send, torch.bfloat16, world, dist=1)
        if comm.has_multicast:
            small = [t[:32768] for t in send]  # 64 KiB
            _fill(small, dist=1, seed=4242)
            comm.all_reduce(small, small, mode="nvls")
            comm.sync()
            assert comm.last_call()["variant"] == "nvls2"
            _check([t.clone() for t in small], torch.bfloat16, world, dist=1, seed=4242)
        # the copy-engine path is for one process per GPU only
        with pytest.raises(RuntimeError, match="cannot run"):
            comm.all_reduce(send, recv, mode="copy_engine")
        # one rank's buffers one element off a 16-byte boundary (cudaMalloc memory, all variants by size)
        for n in (4096, 100001, 1 << 20):
            xs, outs = [], []
            for d in range(world):
                off = 1 if d == 1 else 0
                xs.append(torch.empty(n + 8, dtype=torch.float32, device=f"cuda:{d}")[off:off + n])
                outs.append(torch.empty(n + 8, dtype=torch.float32, device=f"cuda:{d}")[off:off + n])
            _fill(xs, seed=777)
            comm.all_reduce(xs, outs)
            comm.sync()
            _check([o.clone() for o in outs], torch.float32, world, seed=777)
        # fused row epilogue across real GPUs
        rows, hidden = 16, 4096
        xs = [torch.empty(rows, hidden, dtype=torch.bfloat16, device=f"cuda:{d}") for d in range(world)]
        _fill(xs, dist=1)
        ws = [torch.ones(hidden, dtype=torch.bfloat16, device=f"cuda:{d}") for d in range(world)]
        ys = comm.all_reduce_rmsnorm(xs, ws, None, eps=1e-5)
        comm.sync()
        ref, _ = yali.reference.residual_rmsnorm(yali.reference.all_reduce_sum(xs), ws[0].cpu().double(), None, 1e-5)
        for y in ys:
            torch.testing.assert_close(y.cpu().double(), ref, rtol=2e-2, atol=2e-2)


def _rank_main(rank, world, port, q, scenario):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        import yali_b200 as yl
        from yali_b200 import _native as nat
        ext = nat.ext()
        # A rank that leaves must not hold memory bound to an NVSwitch multicast object.
        comm = yl.Comm.from_env(heap_bytes=2 << 30, timeout_ms=1000 if scenario == "plan_mismatch" else 3000,
                                want_multicast=scenario not in ("leave_between_steps", "plan_mismatch"))
        dev = f"cuda:{comm.device}"
        info = {"kind": comm.heap_kind, "mc": comm.has_multicast}
        ok = True
        if scenario == "collectives":
            modes = ["flash", "stream"] + (["nvls"] if comm.has_multicast else [])
            for dtype in (torch.float32, torch.bfloat16):
                for n in (7, 4096, 300000, (1 << 22)):
                    x = torch.empty(n, dtype=dtype, device=dev)
                    ext.fill_random(x, 0, 1234 + rank)
                    for mode in modes:
                        if mode == "nvls" and (n * x.element_size()) % 16:
                            continue
                        if mode == "flash" and n * x.element_size() > comm.layout()["flash_cap"]:
                            continue
                        y = comm.all_reduce(x, mode=mode)
                        comm.sync()
                        ok &= ext.validate_sum(y, dtype, 0, 1234, world)["mismatches"] == 0
            # Rank 1 alone passes buffers one element off a 16-byte boundary: every rank must still pick
            # the same kernel and the sums must be right (sizes for the flag-in-data form, the flagged
            # one-shot, and the ring / staged in-switch kernels).
            for n in (4096, 100001, 1 << 22):
                off = 1 if rank == 1 else 0
                x = torch.empty(n + 8, dtype=torch.float32, device=dev)[off:off + n]
                y = torch.empty(n + 8, dtype=torch.float32, device=dev)[off:off + n]
                ext.fill_random(x, 0, 555 + rank)
                comm.all_reduce(x, y)
                comm.sync()
                ok &= ext.validate_sum(y.clone(), torch.float32, 0, 555, world)["mismatches"] == 0
            n = 1 << 20
            s, r = comm.symm_empty(n, torch.float32), comm.symm_empty(n, torch.float32)
            ext.fill_random(s, 1, 99 + rank)
            for mode in modes + ["flash_pull", "stream_direct", "auto"]:
                for _ in range(4):
                    comm.all_reduce(s, r, mode=mode)
                comm.sync()
                ok &= ext.validate_sum(r, torch.float32, 1, 99, world)["mismatches"] == 0
            # the copy-engine path: out of place, then in place with fresh data per call, several chunks per rank
            for _ in range(3):
                comm.all_reduce(s, r, mode="copy_engine", slot_bytes=512 << 10)
            comm.sync()
            ok &= comm.last_call()["variant"] == "copy_engine"
            ok &= ext.validate_sum(r, torch.float32, 1, 99, world)["mismatches"] == 0
            t = comm.symm_empty(n, torch.float32)
            for rep in range(3):
                ext.fill_random(t, 1, 300 + 10 * rep + rank)
                comm.all_reduce(t, t, mode="copy_engine", slot_bytes=512 << 10)
                comm.sync()
                ok &= ext.validate_sum(t.clone(), torch.float32, 1, 300 + 10 * rep, world)["mismatches"] == 0
                comm.barrier()  # nobody refills its buffer while a peer still reads the sums out of its own
            sh = comm.reduce_scatter(s)
            full = comm.all_gather(sh, n)
            comm.sync()
            ok &= ext.validate_sum(full, torch.float32, 1, 99, world)["mismatches"] == 0
            # the same all-gather between symmetric buffers: the ring kernel writes straight into the peers' outputs
            sh_sym, full_sym = comm.symm_empty(sh.numel(), torch.float32), comm.symm_empty(n, torch.float32)
            sh_sym.copy_(sh)
            comm.barrier()
            for _ in range(3):
                comm.all_gather(sh_sym, n, full_sym)
            comm.sync()
            ok &= bool(comm.last_call()["flags"] & 2)  # direct all-gather
            ok &= ext.validate_sum(full_sym, torch.float32, 1, 99, world)["mismatches"] == 0
        elif scenario == "fused_linear":
            # Row-parallel GEMM + all-reduce + residual + RMSNorm in one kernel per rank: the push
            # forms and (with a multicast object) the in-switch form against an fp32 reference.
            N, K = 1024, 256
            for T in (1, 16, 100, 300, 1000):
                gens = [torch.Generator().manual_seed(4321 + 17 * q + T) for q in range(world)]
                xs = [torch.randn(T, K, generator=g).to(torch.bfloat16) for g in gens]
                ws = [(torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16) for g in gens]
                res = torch.randn(T, N, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
                nw = (1 + 0.1 * torch.randn(N, generator=torch.Generator().manual_seed(6))).to(torch.bfloat16)
                h = sum(x.float() @ w.float().T for x, w in zip(xs, ws)) + res.float()
                want = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.float()
                x, w = xs[rank].to(dev), ws[rank].to(dev)
                forms = [(True, 0, False), (False, 0, False)] + \
                    ([(False, 1, False), (False, 2, False)] if comm.has_multicast else []) + \
                    ([(None, None, True)] if T <= 64 else [])  # the few-token form
                for oneshot, nvls, decode in forms:
                    out = comm.symm_empty([T, N], torch.bfloat16)
                    ro = comm.symm_empty([T, N], torch.bfloat16)
                    for _ in range(3):  # both call parities, and a repeat
                        out.zero_()
                        comm.sync()
                        comm.barrier()
                        comm.fused_linear_rmsnorm(x, w, nw.to(dev), res.to(dev), out=out, residual_out=ro,
                                                  oneshot=oneshot, nvls=nvls, decode=decode)
                        comm.sync()
                        err = (out.float().cpu() - want).abs().max().item()
                        err_h = (ro.float().cpu() - h).abs().max().item()
                        good = err < 0.08 and err_h < 0.06 * max(1.0, h.abs().max().item())
                        if not good:
                            info[f"T{T}_one{oneshot}_nvls{nvls}_decode{decode}"] = (err, err_h)
                        ok &= good
                        comm.barrier()  # nobody clears `out` while a peer still writes rows into it
                comm.symm_reset()
        elif scenario == "plan_mismatch":
            # Rank 0 passes symmetric buffers, rank 1 plain ones (a usage error): at 64 MiB the first
            # picks the pipelined two-shot, the second the ring kernel.  Their waits run out (1 s limit,
            # set above), the status names both kernels, and after reset() the communicator works again.
            n = 16 << 20
            sym_s, sym_r = comm.symm_empty(n, torch.float32), comm.symm_empty(n, torch.float32)
            x = torch.empty(n, dtype=torch.float32, device=dev)
            ext.fill_random(x, 0, 1234 + rank)
            sym_s.copy_(x)
            if rank == 0:
                comm.all_reduce(sym_s, sym_r)
            else:
                comm.all_reduce(x, torch.empty_like(x))
            try:
                comm.sync()
                ok = False
            except Exception as e:  # noqa: BLE001
                info["msg"] = str(e)[-260:]
                ok &= "different kernels" in str(e) and "stream_direct" in str(e) and "symmetric buffers" in str(e)
            comm.reset()
            comm.all_reduce(sym_s, sym_r)
            comm.sync()
            ok &= ext.validate_sum(sym_r, torch.float32, 0, 1234, world)["mismatches"] == 0
        elif scenario == "leave_between_steps":
            x = torch.empty(65536, dtype=torch.float32, device=dev)
            ext.fill_random(x, 0, 1234 + rank)
            y = comm.all_reduce(x, mode="flash")
            comm.sync()
            ok &= ext.validate_sum(y, torch.float32, 0, 1234, world)["mismatches"] == 0
            comm.barrier()  # nothing in flight anywhere
            if rank == world - 1:
                # This rank stops taking part (its process stays alive until the others are done, so
                # its heap stays mapped); the others' next collective must time out, not hang.
                q.put((rank, True, info))
                q.close()
                q.join_thread()
                time.sleep(8)
                os._exit(0)
            comm.all_reduce(x, mode="flash")
            try:
                comm.sync()
                ok = False
            except Exception as e:  # noqa: BLE001
                ok &= "waiting for rank" in str(e)
            q.put((rank, bool(ok), info))
            q.close()
            q.join_thread()
            os._exit(0)  # the communicator cannot be closed collectively any more
        comm.close()
        q.put((rank, bool(ok), info))
    except Exception as e:  # noqa: BLE001
        q.put((rank, False, {"error": repr(e)[:300]}))


def _spawn(world, scenario, free_port, timeout=300):
    q = CTX.Queue()
    procs = [CTX.Process(target=_rank_main, args=(r, world, free_port, q, scenario)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    deadline = time.time() + timeout
    while len(res) < world and time.time() < deadline:
        try:
            r, ok, info = q.get(timeout=1.0)
            res[r] = (ok, info)
        except Exception:  # noqa: BLE001
            if all(not p.is_alive() for p in procs):
                break
    for p in procs:
        p.join(20)
        if p.is_alive():
            p.kill()
    return res


@pytest.mark.parametrize("world", _worlds())
def test_one_process_per_gpu(world, free_port):
    res = _spawn(world, "collectives", free_port)
    assert len(res) == world, res
    assert all(ok for ok, _ in res.values()), res
    assert all(info["kind"] in ("cumem-fd", "cuda-ipc") for _, info in res.values())


@pytest.mark.parametrize("world", _worlds())
def test_fused_linear_one_process_per_gpu(world, free_port):
    res = _spawn(world, "fused_linear", free_port + 2)
    assert len(res) == world, res
    assert all(ok for ok, _ in res.values()), res


def test_ranks_with_different_arguments_get_a_precise_error(free_port, monkeypatch):
    monkeypatch.setenv("YALI_NVLS_DISABLE", "1")  # plain peer loads/stores only: the waits of both ranks run out
    res = _spawn(2, "plan_mismatch", free_port + 3, timeout=120)
    assert len(res) == 2 and all(ok for ok, _ in res.values()), res


def test_rank_that_stops_between_steps_times_out_the_others(free_port, monkeypatch):
    monkeypatch.setenv("YALI_NVLS_DISABLE", "1")  # plain peer loads/stores only
    res = _spawn(2, "leave_between_steps", free_port + 1, timeout=120)
    assert len(res) == 2 and all(ok for ok, _ in res.values()), res
