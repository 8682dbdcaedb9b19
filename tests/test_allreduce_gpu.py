"""All collective kernels on a real GPU.  With a single GPU the ranks are emulated:
every rank has its own heap on that GPU and one cooperative launch runs the CTAs of
all ranks, so the flag protocols, staging, rings and epilogues are the code that
runs across NVLink on a multi-GPU box.  Data is seeded per rank and per element and
checked element-wise on the device against the fp64 sum of the generators, and in
some cases against a plain PyTorch fp32 reference on the host.

Reference counterparts: tests/test_ops_allreduce.cu (1 Ki / 1 Mi elements, constant
fills, 3 dtypes), tests/test_bw_ops.cu (128 MiB fp32 through the stream kernel)."""
import pytest
import torch

import yali_b200 as yali
from yali_b200 import _native

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
UNIFORM, NORMAL = 0, 1


@pytest.fixture(scope="module", params=[2, 4, 8])
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
    # all ranks hold bit-identical results (fixed summation order)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 7, 31, 32, 33, 1024, 4099, 262144, 1 << 20])
def test_flash_random_data(comm, dtype, n):
    xs = make_inputs(comm, n, dtype)
    outs = comm.all_reduce(xs, mode="flash")
    comm.sync()
    assert comm.last_call()["variant"] == "flash"
    check(comm, outs, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 33, 4099, 262144, (1 << 22) + 5])
def test_stream_random_data(comm, dtype, n):
    xs = make_inputs(comm, n, dtype, NORMAL, seed=77)
    outs = comm.all_reduce(xs, mode="stream")
    comm.sync()
    assert comm.last_call()["variant"] == "stream"
    check(comm, outs, dtype, NORMAL, seed=77)


@pytest.mark.parametrize("slot_bytes,lanes", [(256, 1), (1024, 3), (8192, 16)])
def test_stream_small_slots_reuse_the_ring(comm, slot_bytes, lanes):
    # Many iterations per lane: every slot of the 4-deep rings is reused and credits gate the producer.
    n = 300001
    xs = make_inputs(comm, n, torch.float32)
    outs = comm.all_reduce(xs, mode="stream", ctas=lanes, slot_bytes=slot_bytes)
    comm.sync()
    lc = comm.last_call()
    assert lc["slot_bytes"] == slot_bytes and lc["ctas"] == lanes
    check(comm, outs, torch.float32)


def test_matches_pytorch_reference_on_host(comm):
    n = 50000
    xs = make_inputs(comm, n, torch.bfloat16, NORMAL)
    ref = yali.reference.all_reduce_sum(xs)
    for mode in ("flash", "stream"):
        outs = comm.all_reduce(xs, mode=mode)
        comm.sync()
        torch.testing.assert_close(outs[0].cpu().double(), ref, rtol=1e-2, atol=2e-2 * comm.world)


def test_in_place_and_back_to_back_without_sync(comm):
    n = 70001
    for mode in ("flash", "stream"):
        xs = make_inputs(comm, n, torch.float32)
        first = [x.clone() for x in xs]
        # 12 un-synced calls, alternating fresh outputs and in-place
        outs = None
        for it in range(12):
            outs = comm.all_reduce(first, mode=mode)
        comm.all_reduce(xs, xs, mode=mode)  # in place
        comm.sync()
        check(comm, outs, torch.float32)
        check(comm, xs, torch.float32)


def test_alternating_variants_back_to_back(comm):
    n = 100003
    xs = make_inputs(comm, n, torch.float16)
    results = []
    for it in range(10):
        results.append(comm.all_reduce(xs, mode="flash" if it % 2 else "stream"))
    comm.sync()
    for outs in results:
        check(comm, outs, torch.float16)


def test_misaligned_buffers_take_the_scalar_path(comm):
    n = 10007
    ext = _native.ext()
    for dtype in (torch.float32, torch.bfloat16):
        bases = [torch.empty(n + 1, dtype=dtype, device="cuda:0") for _ in range(comm.world)]
        xs = [b[1:] for b in bases]  # 4 / 2 bytes off a 16-byte boundary
        for r in range(comm.world):
            tmp = torch.empty(n, dtype=dtype, device="cuda:0")
            ext.fill_random(tmp, UNIFORM, 1234 + r)
            xs[r].copy_(tmp)
        outs = [torch.empty(n + 1, dtype=dtype, device="cuda:0")[1:] for _ in xs]
        assert xs[0].data_ptr() % 16 != 0 and outs[0].data_ptr() % 16 != 0
        for mode in ("flash", "stream"):
            comm.all_reduce(xs, outs, mode=mode)
            comm.sync()
            check(comm, [o.clone() for o in outs], dtype)


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.bfloat16), (torch.float32, torch.float16),
                                                (torch.bfloat16, torch.float32), (torch.float16, torch.float32),
                                                (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_scale_and_cast_epilogue(comm, in_dtype, out_dtype):
    n = 123457
    scale = 1.0 / comm.world
    xs = make_inputs(comm, n, in_dtype, NORMAL)
    for mode in ("flash", "stream"):
        outs = comm.all_reduce(xs, mode=mode, scale=scale, out_dtype=out_dtype)
        comm.sync()
        assert outs[0].dtype == out_dtype
        check(comm, outs, in_dtype, NORMAL, scale=scale)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,hidden", [(1, 4096), (16, 4096), (5, 1024), (3, 8192), (128, 4096), (7, 256)])
def test_residual_rmsnorm_epilogue(comm, dtype, rows, hidden):
    if dtype == torch.float32 and hidden > 8192:
        pytest.skip("row does not fit four vectors per thread")
    n = rows * hidden
    xs = [x.view(rows, hidden) for x in make_inputs(comm, n, dtype, NORMAL)]
    g = torch.Generator(device="cpu").manual_seed(5)
    weight = (torch.rand(hidden, generator=g) + 0.5).to(dtype).cuda()
    residual = torch.randn(rows, hidden, generator=g).to(dtype).cuda()
    ws = [weight] * comm.world
    rs = [residual] * comm.world
    res_out = [torch.empty_like(x) for x in xs]
    outs = comm.all_reduce_rmsnorm(xs, ws, rs, eps=1e-5, residual_out=res_out)
    comm.sync()
    summed = yali.reference.all_reduce_sum(xs)
    ref, pre = yali.reference.residual_rmsnorm(summed, weight.cpu().double(), residual.cpu().double(), 1e-5)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=1e-4, atol=1e-4)
    for o, ro in zip(outs, res_out):
        torch.testing.assert_close(o.cpu().double(), ref, **tol)
        torch.testing.assert_close(ro.cpu().double(), pre, rtol=tol["rtol"], atol=tol["atol"] * comm.world)
    # without residual
    outs2 = comm.all_reduce_rmsnorm(xs, ws, None, eps=1e-5)
    comm.sync()
    ref2, _ = yali.reference.residual_rmsnorm(summed, weight.cpu().double(), None, 1e-5)
    torch.testing.assert_close(outs2[0].cpu().double(), ref2, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [16, 4099, 500000])
def test_reduce_scatter_then_all_gather(comm, dtype, n):
    xs = make_inputs(comm, n, dtype, NORMAL)
    shards = comm.reduce_scatter(xs)
    comm.sync()
    s = comm.shard_elems(n)
    ref = yali.reference.all_reduce_sum(xs)
    tol = dict(rtol=1e-2, atol=2e-2 * comm.world) if dtype != torch.float32 else dict(rtol=1e-5, atol=1e-5)
    for r, sh in enumerate(shards):
        lo, hi = min(r * s, n), min(r * s + s, n)
        torch.testing.assert_close(sh[:hi - lo].cpu().double(), ref[lo:hi], **tol)
    full = comm.all_gather(shards, n)
    comm.sync()
    for f in full:
        torch.testing.assert_close(f.cpu().double(), ref, **tol)
    # the halves can be followed by a full all-reduce at once (slots drained)
    outs = comm.all_reduce(xs, mode="stream")
    comm.sync()
    torch.testing.assert_close(outs[0].cpu().double(), ref, **tol)


def test_symmetric_buffers(comm):
    n = 65536
    send = comm.symm_empty(n, torch.float32)
    recv = comm.symm_empty(n, torch.float32)
    ext = _native.ext()
    for r, t in enumerate(send):
        ext.fill_random(t, UNIFORM, 1234 + r)
    for mode in ("flash", "stream"):
        comm.all_reduce(send, recv, mode=mode)
        comm.sync()
        check(comm, recv, torch.float32)
    assert comm.last_call()["flags"] & 2  # direct all-gather was used


def test_auto_mode_picks_by_size(comm):
    small = make_inputs(comm, 1024, torch.float32)
    comm.all_reduce(small)
    assert comm.last_call()["variant"] == "flash"
    big_n = (comm.layout()["flash_cap"] // 4) + 1024
    big = make_inputs(comm, big_n, torch.float32)
    outs = comm.all_reduce(big)
    comm.sync()
    # ranks of one process can address each other's buffers: the pipelined two-shot kernel
    assert comm.last_call()["variant"] == "stream_direct"
    check(comm, outs, torch.float32)


def test_errors_are_clean(comm):
    xs = make_inputs(comm, 128, torch.float32)
    with pytest.raises(RuntimeError, match="expected"):
        comm._impl.all_reduce(xs[:1], xs[:1], "auto", None, 0, 0, -1)
    with pytest.raises(RuntimeError, match="mode"):
        comm.all_reduce(xs, mode="warp-speed")
    with pytest.raises(RuntimeError, match="cannot run"):
        comm.all_reduce(xs, mode="nvls")  # emulated ranks have no multicast object
    with pytest.raises(RuntimeError, match="dtype"):
        comm.all_reduce([x.to(torch.int32) for x in xs])
    too_big = torch.empty(comm.layout()["flash_cap"] // 4 + 16, dtype=torch.float32, device="cuda:0")
    with pytest.raises(RuntimeError, match="cannot run"):
        comm.all_reduce([too_big] * comm.world, mode="flash")
    comm.sync()  # the communicator is still usable
    outs = comm.all_reduce(xs)
    comm.sync()
    check(comm, outs, torch.float32)


def test_cuda_graph_replay(comm):
    """Launches carry no per-call number (the kernels keep their call counters on the device), so a
    captured sequence of collectives can be replayed."""
    n = 50000
    xs = make_inputs(comm, n, torch.float32)
    ys = make_inputs(comm, 4 * n, torch.bfloat16, NORMAL, seed=5)
    out_a = [torch.empty_like(x) for x in xs]
    out_b = [torch.empty_like(y) for y in ys]
    out_c = [torch.empty_like(x) for x in xs]
    comm.all_reduce(xs, out_a, mode="flash")  # warm-up outside the capture
    comm.all_reduce(ys, out_b, mode="stream")
    comm.sync()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            comm.all_reduce(xs, out_a, mode="flash")
            comm.all_reduce(ys, out_b, mode="stream")
            comm.all_reduce(xs, out_c, mode="flash", scale=0.5)
    for _ in range(6):
        for o in out_a + out_b + out_c:
            o.zero_()
        graph.replay()
        comm.all_reduce(xs, mode="flash")  # eager calls may be mixed with replays
    torch.cuda.synchronize()
    comm.check()
    check(comm, out_a, torch.float32)
    check(comm, out_b, torch.bfloat16, NORMAL, seed=5)
    check(comm, out_c, torch.float32, scale=0.5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_flag_in_data_form_for_small_messages(comm, dtype):
    """Small aligned messages take the flag-in-data protocol (flags bit 6); larger or ragged ones the flagged one."""
    for n, expect_ll in [(8, True), (4096, True), (65536, True), (65537, False), (1 << 20, False)]:
        xs = make_inputs(comm, n, dtype, NORMAL, seed=n)
        for _ in range(3):  # consecutive calls reuse the two staging halves
            outs = comm.all_reduce(xs, mode="flash")
        comm.sync()
        lc = comm.last_call()
        nbytes = n * xs[0].element_size()
        assert bool(lc["flags"] & 64) == (expect_ll and nbytes % 16 == 0 and nbytes <= 256 * 1024), (n, lc)
        check(comm, outs, dtype, NORMAL, seed=n)
    # scale epilogue on the same path
    xs = make_inputs(comm, 2048, dtype)
    outs = comm.all_reduce(xs, mode="flash", scale=0.25)
    comm.sync()
    assert comm.last_call()["flags"] & 64
    check(comm, outs, dtype, scale=0.25)


def test_rmsnorm_beyond_the_one_shot_capacity_uses_two_launches(comm):
    hidden = 4096
    rows = comm.layout()["flash_cap"] // (hidden * 2) + 64  # just above the one-shot staging
    xs = [x.view(rows, hidden) for x in make_inputs(comm, rows * hidden, torch.bfloat16, NORMAL)]
    g = torch.Generator(device="cpu").manual_seed(11)
    weight = (torch.rand(hidden, generator=g) + 0.5).to(torch.bfloat16).cuda()
    before = comm.launches
    outs = comm.all_reduce_rmsnorm(xs, [weight] * comm.world, None, eps=1e-5)
    comm.sync()
    assert comm.launches - before == 1 + comm.world  # one cooperative all-reduce + one norm kernel per rank
    ref, _ = yali.reference.residual_rmsnorm(yali.reference.all_reduce_sum(xs), weight.cpu().double(), None, 1e-5)
    torch.testing.assert_close(outs[0][:256].cpu().double(), ref[:256], rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(outs[-1][-256:].cpu().double(), ref[-256:], rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("n,chunk_bytes", [(1000, 8 << 20), (3 * 65536 + 77, 65536 * 4), (1 << 20, 1 << 20)])
def test_host_to_host_all_reduce_overlaps_copies_chunk_by_chunk(comm, n, chunk_bytes):
    # pinned host tensors in, pinned host tensors out; more chunks than staging slots in the second case
    g = torch.Generator(device="cpu").manual_seed(77)
    srcs = [torch.rand(n, generator=g).sub_(0.5).pin_memory() for _ in range(comm.world)]
    dsts = [torch.zeros(n).pin_memory() for _ in range(comm.world)]
    want = torch.stack([s.double() for s in srcs]).sum(0)
    for _ in range(2):  # the staging ring is reused by the second call
        for d in dsts:
            d.zero_()
        comm.all_reduce_host(srcs, dsts, chunk_bytes=chunk_bytes)
        torch.cuda.synchronize()
        comm.check()
        for d in dsts:
            torch.testing.assert_close(d.double(), want, rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        comm.all_reduce_host([torch.zeros(8) for _ in range(comm.world)])  # pageable memory
    comm.symm_reset()
