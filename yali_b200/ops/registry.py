"""`torch.ops.yali.*`: the collectives as registered PyTorch operators.

    torch.ops.yali.all_reduce(x)                       -> Tensor
    torch.ops.yali.all_reduce_scaled(x, scale, dtype)  -> Tensor
    torch.ops.yali.all_reduce_rmsnorm(x, weight, residual, eps) -> Tensor
    torch.ops.yali.fused_linear_rmsnorm(x, w, norm_weight, residual, eps) -> Tensor

All of them act on the default communicator (`yali_b200.init_process_group`).  CUDA
tensors run the native sm_100a kernels; CPU tensors run over gloo."""
from __future__ import annotations

from typing import Optional

import torch

from . import collectives

_lib = torch.library.Library("yali", "DEF")
_lib.define("all_reduce(Tensor x) -> Tensor")
_lib.define("all_reduce_scaled(Tensor x, float scale, ScalarType? out_dtype=None) -> Tensor")
_lib.define("all_reduce_rmsnorm(Tensor x, Tensor weight, Tensor? residual=None, float eps=1e-05) -> Tensor")
_lib.define("fused_linear_rmsnorm(Tensor x, Tensor w, Tensor norm_weight, Tensor? residual=None, float eps=1e-05) -> Tensor")
_lib.define("reduce_scatter(Tensor x) -> Tensor")
_lib.define("all_gather(Tensor shard, int count) -> Tensor")


def _all_reduce(x: torch.Tensor) -> torch.Tensor:
    return collectives.all_reduce(x)


def _all_reduce_scaled(x: torch.Tensor, scale: float, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    return collectives.all_reduce(x, scale=scale, out_dtype=out_dtype)


def _all_reduce_rmsnorm(x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None,
                        eps: float = 1e-5) -> torch.Tensor:
    return collectives.all_reduce_rmsnorm(x, weight, residual, eps=eps)


def _fused_linear_rmsnorm(x: torch.Tensor, w: torch.Tensor, norm_weight: torch.Tensor,
                          residual: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    return collectives.fused_linear_rmsnorm(x, w, norm_weight, residual, eps=eps)


def _reduce_scatter(x: torch.Tensor) -> torch.Tensor:
    return collectives.reduce_scatter(x)


def _all_gather(shard: torch.Tensor, count: int) -> torch.Tensor:
    return collectives.all_gather(shard, count)


for _key in ("CPU", "CUDA"):
    _lib.impl("all_reduce", _all_reduce, _key)
    _lib.impl("all_reduce_scaled", _all_reduce_scaled, _key)
    _lib.impl("all_reduce_rmsnorm", _all_reduce_rmsnorm, _key)
    _lib.impl("fused_linear_rmsnorm", _fused_linear_rmsnorm, _key)
    _lib.impl("reduce_scatter", _reduce_scatter, _key)
    _lib.impl("all_gather", _all_gather, _key)


# ---- shape / dtype rules ("fake" kernels): what a tracer (FakeTensor, torch.export, the meta device) needs to
# know about the operators without running them.  Shapes follow the eager implementations above.
def _shard_elems(count: int) -> int:
    from ..parallel import comm as _comm
    world = _comm.get_default_comm().world
    per = -(-count // world)
    return -(-per // 16) * 16  # ceil(count / world) rounded up to 16 elements, as ShardElems in csrc/ops/tuning.cc


@torch.library.register_fake("yali::all_reduce")
def _fake_all_reduce(x):
    return torch.empty_like(x)


@torch.library.register_fake("yali::all_reduce_scaled")
def _fake_all_reduce_scaled(x, scale, out_dtype=None):
    return torch.empty_like(x, dtype=out_dtype or x.dtype)


@torch.library.register_fake("yali::all_reduce_rmsnorm")
def _fake_all_reduce_rmsnorm(x, weight, residual=None, eps=1e-5):
    return torch.empty_like(x)


@torch.library.register_fake("yali::fused_linear_rmsnorm")
def _fake_fused_linear_rmsnorm(x, w, norm_weight, residual=None, eps=1e-5):
    return x.new_empty((x.shape[0], w.shape[0]))


@torch.library.register_fake("yali::reduce_scatter")
def _fake_reduce_scatter(x):
    return x.new_empty((_shard_elems(x.numel()),))


@torch.library.register_fake("yali::all_gather")
def _fake_all_gather(shard, count):
    return shard.new_empty((count,))
