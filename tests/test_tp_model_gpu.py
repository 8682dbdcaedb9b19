"""A tensor-parallel Llama-style block (reduced widths) on emulated ranks: the fused path
(two fused GEMM + all-reduce + residual + RMSNorm kernels per block) against the unfused
composition and against an fp64 CPU restatement of the whole block."""
import pytest
import torch

import yali_b200 as yali
from yali_b200.models.llama_tp import LlamaTPConfig, TPBlockRank, reference_block, run_block

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_block_fused_matches_unfused_and_reference(world):
    cfg = LlamaTPConfig(hidden=512, heads=8, kv_heads=4, intermediate=1024, world=world)
    with yali.Comm.emulated(world, device=0) as comm:
        ranks = [TPBlockRank(cfg, device="cuda", seed=10 + r) for r in range(world)]
        B, S = 2, 24
        g = torch.Generator(device="cpu").manual_seed(0)
        normed = torch.randn(B, S, cfg.hidden, generator=g).to(torch.bfloat16).cuda()
        residual = torch.randn(B, S, cfg.hidden, generator=g).to(torch.bfloat16).cuda()
        y_f, r_f = run_block(comm, ranks, [normed] * world, [residual] * world, fused=True)
        y_u, r_u = run_block(comm, ranks, [normed] * world, [residual] * world, fused=False)
        comm.sync()
        for a, b in zip(y_f, y_u):
            torch.testing.assert_close(a.float(), b.float(), rtol=6e-2, atol=6e-2)
        y_ref, r_ref = reference_block(ranks, normed, residual)
        torch.testing.assert_close(y_f[0].double().cpu(), y_ref, rtol=8e-2, atol=8e-2)
        torch.testing.assert_close(r_f[0].double().cpu(), r_ref, rtol=8e-2, atol=8e-2)
