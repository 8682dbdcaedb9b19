"""The framework layer without a GPU: `yali_b200.all_reduce` on CPU tensors runs
over torch.distributed/gloo with world_size 2.  Covers the baseline configuration
"2-rank fp32 sum of 262144 elements, rank r ~ N(0,1) from seed 1234+r, checked
element-wise against a host-computed sum with rtol 1e-6"."""
import multiprocessing as mp
import os

import pytest
import torch

CTX = mp.get_context("spawn")


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import yali_b200 as yali
    comm = yali.init_process_group(backend="gloo")
    n = 262144
    inputs = [torch.randn(n, generator=torch.Generator().manual_seed(1234 + r)) for r in range(world)]
    out = yali.all_reduce(inputs[rank])
    expect = yali.reference.all_reduce_sum(inputs)
    ok = torch.allclose(out.double(), expect, rtol=1e-6, atol=1e-6)
    # fused forms through the same surface
    scaled = yali.all_reduce(inputs[rank], scale=0.5, out_dtype=torch.bfloat16)
    ok &= torch.allclose(scaled.double(), (expect * 0.5).to(torch.bfloat16).double(), rtol=2e-2, atol=2e-2)
    h = 256
    w = torch.rand(h) + 0.5
    res = torch.randn(n)
    y = yali.all_reduce_rmsnorm(inputs[rank], w, res, eps=1e-5)
    ref, _ = yali.reference.residual_rmsnorm(expect, w.double(), res.double(), 1e-5)
    ok &= torch.allclose(y.double(), ref, rtol=1e-4, atol=1e-4)
    shard = yali.reduce_scatter(inputs[rank])
    s = comm.shard_elems(n)
    ok &= torch.allclose(shard.double()[:min(s, n - rank * s)], expect[rank * s:rank * s + s], rtol=1e-6, atol=1e-6)
    full = yali.all_gather(shard, n)
    ok &= torch.allclose(full.double(), expect, rtol=1e-6, atol=1e-6)
    # the fused tensor-parallel layer through the same call as on a GPU
    T, K, N = 5, 16, 64
    xs = [torch.randn(T, K, generator=torch.Generator().manual_seed(50 + r)) for r in range(world)]
    wts = [torch.randn(N, K, generator=torch.Generator().manual_seed(60 + r)) * 0.1 for r in range(world)]
    g = torch.rand(N, generator=torch.Generator().manual_seed(70)) + 0.5
    resid = torch.randn(T, N, generator=torch.Generator().manual_seed(71))
    buf = comm.symm_empty([T, N], torch.float32)
    got = comm.fused_linear_rmsnorm(xs[rank], wts[rank], g, resid, out=buf)
    hsum = sum(a.double() @ b.double().T for a, b in zip(xs, wts)) + resid.double()
    want = hsum * torch.rsqrt(hsum.pow(2).mean(-1, keepdim=True) + 1e-5) * g.double()
    ok &= got is buf and torch.allclose(got.double(), want, rtol=1e-4, atol=1e-4)
    import yali_b200.ops.registry  # noqa: F401
    got2 = torch.ops.yali.fused_linear_rmsnorm(xs[rank], wts[rank], g, resid)
    ok &= torch.allclose(got2.double(), want, rtol=1e-4, atol=1e-4)
    # host-to-host call: same surface as on a GPU box, nothing to stage on CPU
    hh = yali.all_reduce_host(inputs[rank])
    ok &= torch.allclose(hh.double(), expect, rtol=1e-6, atol=1e-6)
    # the torch.ops surface dispatches CPU tensors to the same path
    import yali_b200.ops.registry  # noqa: F401
    out2 = torch.ops.yali.all_reduce(inputs[rank])
    ok &= torch.equal(out2, out)
    # shape / dtype rules of the operators under a tracer (no data, nothing runs)
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        fx = torch.empty(n)
        ok &= torch.ops.yali.all_reduce(fx).shape == (n,)
        ok &= torch.ops.yali.all_reduce_scaled(fx, 0.5, torch.bfloat16).dtype == torch.bfloat16
        ok &= torch.ops.yali.fused_linear_rmsnorm(torch.empty(T, K), torch.empty(N, K), torch.empty(N)).shape == (T, N)
        ok &= torch.ops.yali.reduce_scatter(fx).shape == (s,)
        ok &= torch.ops.yali.all_gather(torch.empty(s), n).shape == (n,)
    yali.destroy_process_group()
    q.put((rank, bool(ok)))


def test_two_rank_gloo_allreduce(free_port):
    q = CTX.Queue()
    procs = [CTX.Process(target=_worker, args=(r, 2, free_port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(30)
    assert res == {0: True, 1: True}
