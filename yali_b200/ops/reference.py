"""Plain PyTorch fp32 references of every fused operation.  The numerics tests
compare the CUDA kernels against these; the gloo (CPU) path uses them directly."""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch


def all_reduce_sum(inputs: Sequence[torch.Tensor], scale: Optional[float] = None) -> torch.Tensor:
    """Sum of the ranks' inputs in fp64, optionally scaled."""
    acc = torch.zeros_like(inputs[0], dtype=torch.float64, device="cpu")
    for x in inputs:
        acc += x.detach().to("cpu", torch.float64)
    if scale is not None:
        acc *= scale
    return acc


def residual_rmsnorm(summed: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor],
                     eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(RMSNorm(summed + residual) * weight, summed + residual), computed in fp32 or wider."""
    wide = torch.float64 if summed.dtype == torch.float64 else torch.float32
    h = weight.numel()
    pre = summed.to(wide).reshape(-1, h)
    if residual is not None:
        pre = pre + residual.to(pre.device, wide).reshape(-1, h)
    var = pre.pow(2).mean(dim=-1, keepdim=True)
    y = pre * torch.rsqrt(var + eps) * weight.to(pre.device, wide).reshape(1, h)
    return y.reshape(summed.shape), pre.reshape(summed.shape)


def row_parallel_linear_rmsnorm(xs: Sequence[torch.Tensor], ws: Sequence[torch.Tensor], norm_weight: torch.Tensor,
                                residual: Optional[torch.Tensor], eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Tensor-parallel layer: y = RMSNorm(residual + sum_r xs[r] @ ws[r]) * norm_weight.
    xs[r]: [T, K_r], ws[r]: [K_r, H] (already the rank's slice).  fp64 on the CPU."""
    acc = None
    for x, w in zip(xs, ws):
        p = x.detach().to("cpu", torch.float64) @ w.detach().to("cpu", torch.float64)
        acc = p if acc is None else acc + p
    return residual_rmsnorm(acc, norm_weight.detach().to("cpu", torch.float64),
                            None if residual is None else residual.detach().to("cpu", torch.float64), eps)
