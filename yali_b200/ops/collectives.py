"""Functional collectives on the default communicator (or an explicit one).

CUDA tensors run the native kernels; CPU tensors go through `GlooComm`.  The same
functions back the `torch.ops.yali.*` operators (see `registry.py`)."""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel import comm as _comm


def _pick(comm):
    return comm if comm is not None else _comm.get_default_comm()


def all_reduce(x: torch.Tensor, *, comm=None, out: Optional[torch.Tensor] = None, scale: Optional[float] = None,
               out_dtype: Optional[torch.dtype] = None, mode: str = "auto") -> torch.Tensor:
    """Sum over all ranks (optionally scaled and cast)."""
    return _pick(comm).all_reduce(x, out, mode=mode, scale=scale, out_dtype=out_dtype)


def all_reduce_rmsnorm(x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None, *,
                       eps: float = 1e-5, comm=None, out: Optional[torch.Tensor] = None,
                       residual_out: Optional[torch.Tensor] = None, mode: str = "auto") -> torch.Tensor:
    """RMSNorm(sum over ranks of x + residual) * weight in one kernel."""
    return _pick(comm).all_reduce_rmsnorm(x, weight, residual, eps=eps, out=out, residual_out=residual_out, mode=mode)


def fused_linear_rmsnorm(x: torch.Tensor, w: torch.Tensor, norm_weight: torch.Tensor,
                         residual: Optional[torch.Tensor] = None, *, eps: float = 1e-5, comm=None,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm(residual + sum over ranks of x @ w.T) * norm_weight in one kernel per rank (x: [T, K] and
    w: [N, K] are this rank's slices).  Without `out` the result is a fresh tensor (copied out of the
    communicator's symmetric output buffer, which the next call reuses)."""
    c = _pick(comm)
    y = c.fused_linear_rmsnorm(x, w, norm_weight, residual, eps=eps, out=out)
    return y if out is not None or not y.is_cuda else y.clone()


def all_reduce_host(src: torch.Tensor, dst: Optional[torch.Tensor] = None, *, comm=None,
                    chunk_bytes: int = 0, scale: Optional[float] = None) -> torch.Tensor:
    """Sum over all ranks of a tensor in pinned host memory, result in pinned host memory; the copies in
    both directions and the all-reduce overlap chunk by chunk (Comm.all_reduce_host)."""
    return _pick(comm).all_reduce_host(src, dst, chunk_bytes=chunk_bytes, scale=scale)


def reduce_scatter(x: torch.Tensor, *, comm=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _pick(comm).reduce_scatter(x, out)


def all_gather(shard: torch.Tensor, count: int, *, comm=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _pick(comm).all_gather(shard, count, out)
