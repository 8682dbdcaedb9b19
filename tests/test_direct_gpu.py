"""The pipelined kernels that read the peers' inputs in place (one-shot pull and two-shot
pull + push), odd world sizes, and ranks whose buffers differ in alignment.  Ranks are
emulated on one GPU (one cooperative launch), data is seeded per rank and per element and
checked element-wise on the device against the fp64 sum of the generators.

Reference counterpart: tests/test_ops_allreduce.cu exercises the 2-GPU prefetching kernel
with constant fills only; odd sizes, in place and mixed alignment are not covered there."""
import pytest
import torch

import yali_b200 as yali
from yali_b200 import _native

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
UNIFORM, NORMAL = 0, 1


@pytest.fixture(scope="module", params=[2, 3, 4, 5, 6, 7, 8])
def comm(request):
    c = yali.Comm.emulated(request.param, device=0, timeout_ms=2000)
    yield c
    c.close()


def make_inputs(comm, n, dtype, dist=UNIFORM, seed=1234):
    ext = _native.ext()
    xs = []
    for r in range(comm.world):
        t = torch.empty(n, dtype=dtype, device="cuda:0")
        ext.fill_random(t, dist, seed + r)
        xs.append(t)
    return xs


def check(comm, outs, in_dtype, dist=UNIFORM, seed=1234, scale=1.0):
    ext = _native.ext()
    for r, o in enumerate(outs):
        rep = ext.validate_sum(o, in_dtype, dist, seed, comm.world, scale)
        assert rep["mismatches"] == 0, (r, rep)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("mode", ["flash_pull", "stream_direct"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 7, 33, 4099, 262144, (1 << 22) + 5])
def test_pipelined_random_data(comm, mode, dtype, n):
    xs = make_inputs(comm, n, dtype, NORMAL, seed=91)
    outs = comm.all_reduce(xs, mode=mode)
    comm.sync()
    lc = comm.last_call()
    assert lc["variant"] == mode and lc["stages"] >= 2
    check(comm, outs, dtype, NORMAL, seed=91)


@pytest.mark.parametrize("mode", ["flash_pull", "stream_direct"])
@pytest.mark.parametrize("ctas,chunk,stages", [(1, 1024, 2), (3, 2048, 3), (16, 4096, 0)])
def test_small_chunks_wrap_the_stage_ring(comm, mode, ctas, chunk, stages, monkeypatch):
    # Many chunks per CTA: every stage is reused several times and both mbarrier phases occur.
    if stages:
        monkeypatch.setenv("YALI_DEV_STAGES", str(stages))
    n = 300001
    xs = make_inputs(comm, n, torch.float32)
    outs = comm.all_reduce(xs, mode=mode, ctas=ctas, slot_bytes=chunk)
    comm.sync()
    lc = comm.last_call()
    assert lc["ctas"] == ctas and lc["slot_bytes"] == chunk and (not stages or lc["stages"] == stages)
    check(comm, outs, torch.float32)


def test_two_shot_in_place_and_back_to_back(comm):
    n = 70001
    xs = make_inputs(comm, n, torch.bfloat16)
    first = [x.clone() for x in xs]
    outs = None
    for _ in range(12):  # un-synced calls, alternating the two forms
        outs = comm.all_reduce(first, mode="stream_direct")
        outs2 = comm.all_reduce(first, mode="flash_pull")
    comm.all_reduce(xs, xs, mode="stream_direct")  # in place
    comm.sync()
    check(comm, outs, torch.bfloat16)
    check(comm, outs2, torch.bfloat16)
    check(comm, xs, torch.bfloat16)
    with pytest.raises(RuntimeError, match="cannot run"):
        comm.all_reduce(first, first, mode="flash_pull")  # the one-shot pull cannot run in place


def test_auto_mode_in_place_avoids_the_pull(comm):
    n = 1 << 20  # 4 MiB fp32
    xs = make_inputs(comm, n, torch.float32)
    comm.all_reduce(xs, xs)
    comm.sync()
    assert comm.last_call()["variant"] != "flash_pull"
    check(comm, xs, torch.float32)


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                                (torch.float16, torch.float16)])
@pytest.mark.parametrize("mode", ["flash_pull", "stream_direct"])
def test_scale_and_cast_epilogue(comm, mode, in_dtype, out_dtype):
    n = 123457
    scale = 1.0 / comm.world
    xs = make_inputs(comm, n, in_dtype)
    outs = comm.all_reduce(xs, mode=mode, scale=scale, out_dtype=out_dtype)
    comm.sync()
    assert outs[0].dtype == out_dtype
    ext = _native.ext()
    for o in outs:
        rep = ext.validate_sum(o, in_dtype, UNIFORM, 1234, comm.world, scale)
        assert rep["mismatches"] == 0, rep


def test_cuda_graph_replay_of_pipelined_calls(comm):
    n = 200000
    xs = make_inputs(comm, n, torch.float32)
    outs_a = [torch.empty_like(x) for x in xs]
    outs_b = [torch.empty_like(x) for x in xs]
    comm.all_reduce(xs, outs_a, mode="flash_pull")  # first launch outside the capture (attribute set-up)
    comm.all_reduce(xs, outs_b, mode="stream_direct")
    comm.sync()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(3):
                comm.all_reduce(xs, outs_a, mode="flash_pull")
                comm.all_reduce(xs, outs_b, mode="stream_direct")
    for o in outs_a + outs_b:
        o.zero_()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    comm.check()
    check(comm, outs_a, torch.float32)
    check(comm, outs_b, torch.float32)


@pytest.mark.parametrize("mode", ["flash", "stream", "auto"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_only_one_rank_misaligned(comm, mode, dtype):
    """Rank 1 passes buffers one element off a 16-byte boundary, the others aligned ones: all
    ranks must still cut the message into the same pieces."""
    ext = _native.ext()
    for n in (40001, 10007, 4096):  # 4096: whole vectors, so small enough for the flag-in-data form
        xs, outs = [], []
        for r in range(comm.world):
            off = 1 if r == 1 else 0
            base = torch.empty(n + 8, dtype=dtype, device="cuda:0")
            x = base[off:off + n]
            tmp = torch.empty(n, dtype=dtype, device="cuda:0")
            ext.fill_random(tmp, UNIFORM, 1234 + r)
            x.copy_(tmp)
            xs.append(x)
            outs.append(torch.empty(n + 8, dtype=dtype, device="cuda:0")[off:off + n])
        assert xs[1].data_ptr() % 16 != 0 and xs[0].data_ptr() % 16 == 0
        comm.all_reduce(xs, outs, mode=mode, ctas=2 if mode == "flash" else 0)
        comm.sync()
        check(comm, [o.clone() for o in outs], dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_odd_worlds_flash_stream_and_rmsnorm(comm, dtype):
    n_rows, hidden = 9, 1024
    xs = make_inputs(comm, n_rows * hidden, dtype, NORMAL, seed=5)
    for mode in ("flash", "stream"):
        outs = comm.all_reduce(xs, mode=mode)
        comm.sync()
        check(comm, outs, dtype, NORMAL, seed=5)
    w = torch.rand(hidden, dtype=dtype, device="cuda:0") + 0.5
    res = torch.randn(n_rows * hidden, dtype=dtype, device="cuda:0")
    ys = comm.all_reduce_rmsnorm(xs, [w] * comm.world, [res] * comm.world, eps=1e-5)
    comm.sync()
    total = yali.reference.all_reduce_sum(xs)
    ref, _ = yali.reference.residual_rmsnorm(total, w.cpu().double(), res.cpu().double(), 1e-5)
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(ys[0].cpu().double().view(n_rows, hidden), ref.view(n_rows, hidden), **tol)


def test_device_timeline(comm):
    n = 65536
    xs = make_inputs(comm, n, torch.float32)
    comm.sync()
    before, _ = comm.read_trace(0, 16)
    comm.set_trace(True)
    for mode in ("flash", "stream", "flash_pull", "stream_direct", "auto"):
        comm.all_reduce(xs, mode=mode)
    comm.set_trace(False)
    comm.all_reduce(xs)  # not traced
    comm.sync()
    calls, entries = comm.read_trace(0, 5)
    assert calls == before + 5 and len(entries) == 5
    for start, end in entries:
        assert 0 < end - start < 2_000_000_000  # finished, and within the wait limit
    assert all(entries[i][1] <= entries[i + 1][0] for i in range(4))  # stream order
