"""Tensor-parallel building blocks on top of the fused kernels.

`RowParallelLinearNorm` is the row-parallel projection of a transformer block (the
attention `o_proj` or the MLP `down_proj`) followed by the all-reduce, the residual
add and the next RMSNorm: on CUDA it is ONE kernel per rank
(`Comm.fused_linear_rmsnorm`, tcgen05 GEMM + peer pushes + reduce + norm); on CPU it
is the PyTorch reference over gloo.  `unfused_*` are the compositions the fused
kernel is compared against (library GEMM, all-reduce, separate norm).

Reference parity: the reference has no tensor-parallel layer; its all-reduce is the
primitive such a layer would call (README.md:9)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
from torch import nn

from ..ops import reference


class RowParallelLinearNorm(nn.Module):
    """y = RMSNorm(residual + all_reduce(x_local @ W_local^T)) * norm_weight.

    `weight` is this rank's [hidden, in_features / world] slice in nn.Linear layout."""

    def __init__(self, in_features_local: int, hidden: int, eps: float = 1e-5, device=None,
                 dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(hidden, in_features_local, device=device, dtype=dtype),
                                   requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(hidden, device=device, dtype=dtype), requires_grad=False)
        self.eps = eps
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, comm, x_local: torch.Tensor, residual: Optional[torch.Tensor] = None,
                residual_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        shape = x_local.shape
        x2 = x_local.reshape(-1, shape[-1])
        if x2.is_cuda:
            r2 = None if residual is None else residual.reshape(x2.shape[0], -1)
            # One kernel per rank for every token count: up to 64 rows the few-token form (256-column tiles split
            # along K, flag-in-data pushes), above that the 128 x 256 tile form.  No library GEMM on this path.
            y = comm.fused_linear_rmsnorm(x2, self.weight, self.norm_weight, r2, eps=self.eps, out=out,
                                          residual_out=residual_out)
        else:
            part = x2.float() @ self.weight.float().T
            y = comm.all_reduce_rmsnorm(part, self.norm_weight.float(), None if residual is None else
                                        residual.reshape(part.shape).float(), eps=self.eps,
                                        residual_out=residual_out).to(x_local.dtype)
        return y.reshape(*shape[:-1], -1)


def fused_row_parallel(comm, xs: Sequence[torch.Tensor], ws: Sequence[torch.Tensor], norm_w: Sequence[torch.Tensor],
                       residual: Optional[Sequence[torch.Tensor]] = None, eps: float = 1e-5, **kw) -> List[torch.Tensor]:
    """All local ranks at once (one process driving several GPUs, or emulated ranks)."""
    return comm.fused_linear_rmsnorm(list(xs), list(ws), list(norm_w), None if residual is None else list(residual),
                                     eps=eps, **kw)


def unfused_row_parallel(comm, xs: Sequence[torch.Tensor], ws: Sequence[torch.Tensor], norm_w: Sequence[torch.Tensor],
                         residual: Optional[Sequence[torch.Tensor]] = None, eps: float = 1e-5,
                         fuse_norm: bool = True) -> List[torch.Tensor]:
    """Baseline composition: library GEMM per rank, then this library's all-reduce fused with
    residual + RMSNorm (`fuse_norm`) or its plain all-reduce followed by a PyTorch RMSNorm."""
    parts = [x @ w.T for x, w in zip(xs, ws)]
    if fuse_norm:
        return comm.all_reduce_rmsnorm(parts, list(norm_w), None if residual is None else list(residual), eps=eps)
    summed = comm.all_reduce(parts)
    outs = []
    for i, s in enumerate(summed):
        y, _ = reference.residual_rmsnorm(s.float(), norm_w[i].float(), None if residual is None else residual[i].float(),
                                          eps)
        outs.append(y.to(s.dtype))
    return outs


def smoke_fused_layer(comm) -> None:
    """Tiny forward of the fused layer on the communicator's ranks, checked against the reference."""
    W = comm.world
    T, K, N = 16, 128, 256
    g = torch.Generator(device="cpu").manual_seed(3)
    devs = comm.devices
    xs = [torch.randn(T, K, generator=g).to(torch.bfloat16).to(f"cuda:{d}") for d in devs]
    ws = [(torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(f"cuda:{d}") for d in devs]
    nw = [torch.ones(N, dtype=torch.bfloat16, device=f"cuda:{d}") for d in devs]
    res = [torch.zeros(T, N, dtype=torch.bfloat16, device=f"cuda:{d}") for d in devs]
    ys = fused_row_parallel(comm, xs, ws, nw, res)
    comm.sync()
    ref, _ = reference.row_parallel_linear_rmsnorm(xs, [w.T for w in ws], nw[0], None, 1e-5)
    torch.testing.assert_close(ys[0].cpu().double(), ref, rtol=5e-2, atol=5e-2)
    assert W == len(ys)
