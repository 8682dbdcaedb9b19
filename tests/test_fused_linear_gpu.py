"""The fused tensor-parallel layer: row-parallel GEMM on tcgen05/TMEM whose epilogue
pushes partial rows to their owner, then all-reduce + residual + RMSNorm, against a
plain PyTorch fp64 reference of the same layer.  Ranks are emulated on one GPU (one
cooperative launch runs all ranks' CTAs).  Shapes follow the Llama-3-8B o_proj with
tensor parallelism 8: K = 512 per rank, hidden 4096, T in {1, 16, 128, 2048}."""
import pytest
import torch

import yali_b200 as yali

pytestmark = pytest.mark.gpu


def make_layer(world, T, K, N, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    xs = [torch.randn(T, K, generator=g).to(torch.bfloat16).cuda() for _ in range(world)]
    ws = [(torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).cuda() for _ in range(world)]
    nw = (torch.rand(N, generator=g) + 0.5).to(torch.bfloat16).cuda()
    res = torch.randn(T, N, generator=g).to(torch.bfloat16).cuda()
    return xs, ws, nw, res


def reference(xs, ws, nw, res, eps=1e-5):
    # Partials are rounded to bf16 before the cross-rank sum, as in the unfused composition
    # (bf16 GEMM output, then all-reduce).
    acc = None
    for x, w in zip(xs, ws):
        p = (x.double().cpu() @ w.double().cpu().T).to(torch.bfloat16).double()
        acc = p if acc is None else acc + p
    return yali.reference.residual_rmsnorm(acc, nw.double().cpu(), None if res is None else res.double().cpu(), eps)


@pytest.fixture(scope="module", params=[2, 8])
def comm(request):
    c = yali.Comm.emulated(request.param, device=0, timeout_ms=3000)
    yield c
    c.close()


@pytest.mark.parametrize("T", [1, 16, 128, 300, 2048])
@pytest.mark.parametrize("oneshot", [True, False])
def test_fused_linear_matches_reference(comm, T, oneshot):
    K, N = 512, 4096
    if oneshot and T * N * 2 > comm.layout()["gemm_cap"]:
        pytest.skip("one-shot landing zone too small for this many rows")
    xs, ws, nw, res = make_layer(comm.world, T, K, N, seed=T)
    W = comm.world
    res_out = [torch.empty(T, N, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    outs = comm.fused_linear_rmsnorm(xs, ws, [nw] * W, [res] * W, eps=1e-5, residual_out=res_out, oneshot=oneshot)
    comm.sync()
    ref, pre = reference(xs, ws, nw, res)
    for o in outs:
        torch.testing.assert_close(o.double().cpu(), ref, rtol=3e-2, atol=3e-2)
    for q in range(W):
        torch.testing.assert_close(res_out[q].double().cpu(), pre, rtol=2e-2, atol=2e-2 * W)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("T", [1, 2, 9, 16, 17, 31, 33, 64])
def test_few_token_form_matches_reference(comm, T):
    """T <= 64: 128 x 256 tiles split along K, partial rows to every rank as flag-in-data lines, every rank normalises all rows."""
    K, N = 512, 4096
    W = comm.world
    xs, ws, nw, res = make_layer(W, T, K, N, seed=100 + T)
    ref, pre = reference(xs, ws, nw, res)
    res_out = [torch.empty(T, N, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    results = []
    for it in range(5):  # back to back without synchronisation: the two landing parities alternate
        results.append(comm.fused_linear_rmsnorm(xs, ws, [nw] * W, [res] * W, eps=1e-5, residual_out=res_out, decode=True))
    comm.sync()
    for outs in results:
        for o in outs:
            torch.testing.assert_close(o.double().cpu(), ref, rtol=3e-2, atol=3e-2)
        for o in outs[1:]:
            assert torch.equal(o, outs[0])
    for q in range(W):
        torch.testing.assert_close(res_out[q].double().cpu(), pre, rtol=2e-2, atol=2e-2 * W)
    with pytest.raises(RuntimeError, match="at most"):
        big = make_layer(W, 65, K, N, seed=1)
        comm.fused_linear_rmsnorm(big[0], big[1], [big[2]] * W, None, decode=True)


def test_few_token_form_other_shapes_and_alternation(comm):
    W = comm.world
    for (T, K, N) in [(8, 64, 128), (40, 1024, 2048), (5, 192, 512)]:
        xs, ws, nw, _ = make_layer(W, T, K, N, seed=K + 1)
        ref, _ = reference(xs, ws, nw, None)
        results = []
        for it in range(6):  # alternate with the tile form (its counters and landing zone are separate)
            results.append(comm.fused_linear_rmsnorm(xs, ws, [nw] * W, None, decode=bool(it % 2 == 0)))
        comm.sync()
        for outs in results:
            for o in outs:
                torch.testing.assert_close(o.double().cpu(), ref, rtol=3e-2, atol=3e-2)


def test_fused_linear_back_to_back_and_other_shapes(comm):
    W = comm.world
    for (T, K, N) in [(64, 64, 128), (200, 1024, 2048), (33, 192, 512)]:
        xs, ws, nw, _ = make_layer(W, T, K, N, seed=K)
        ref, _ = reference(xs, ws, nw, None)
        results = []
        for it in range(6):
            results.append(comm.fused_linear_rmsnorm(xs, ws, [nw] * W, None, oneshot=bool(it % 2)))
        comm.sync()
        for outs in results:
            for o in outs:
                torch.testing.assert_close(o.double().cpu(), ref, rtol=3e-2, atol=3e-2)


def test_fused_linear_rejects_bad_shapes(comm):
    W = comm.world
    xs, ws, nw, _ = make_layer(W, 8, 96, 256, seed=1)  # K not a multiple of 64
    with pytest.raises(RuntimeError, match="multiple"):
        comm.fused_linear_rmsnorm(xs, ws, [nw] * W, None)
    xs, ws, nw, _ = make_layer(W, 8, 64, 200, seed=1)  # N not a multiple of 128
    with pytest.raises(RuntimeError, match="multiple"):
        comm.fused_linear_rmsnorm(xs, ws, [nw] * W, None)
    comm.sync()
