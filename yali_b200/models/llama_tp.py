"""A Llama-style decoder block under tensor parallelism, built on the fused kernels.

Per rank: attention over this rank's heads (QKV column-parallel, local), `o_proj`
row-parallel fused with all-reduce + residual + post-attention RMSNorm, MLP gate/up
column-parallel (local), `down_proj` row-parallel fused with all-reduce + residual +
the next block's input RMSNorm.  The two row-parallel projections are the
communication points of the block; each is one kernel per rank.  Defaults are the
Llama-3-8B shapes (hidden 4096, 32 heads, 8 KV heads, intermediate 14336).

`TPBlockRank` holds one rank's parameters.  `run_block` drives all local ranks of a
communicator (one process per GPU: one; one process for several GPUs or emulated
ranks: all).  Weights are random-initialised; there are no checkpoints here."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import reference
from ..parallel.tensor_parallel import RowParallelLinearNorm


@dataclass
class LlamaTPConfig:
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    intermediate: int = 14336
    eps: float = 1e-5
    world: int = 8

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


class TPBlockRank(nn.Module):
    """One rank's slice of a decoder block."""

    def __init__(self, cfg: LlamaTPConfig, device=None, dtype: torch.dtype = torch.bfloat16, seed: int = 0) -> None:
        super().__init__()
        assert cfg.heads % cfg.world == 0 and cfg.intermediate % cfg.world == 0
        self.cfg = cfg
        self.h_local = cfg.heads // cfg.world
        self.kv_local = max(1, cfg.kv_heads // cfg.world)
        hd = cfg.head_dim
        g = torch.Generator(device="cpu").manual_seed(seed)

        def rnd(*shape):
            return nn.Parameter((torch.randn(*shape, generator=g) * 0.02).to(dtype).to(device), requires_grad=False)

        self.wq = rnd(self.h_local * hd, cfg.hidden)
        self.wk = rnd(self.kv_local * hd, cfg.hidden)
        self.wv = rnd(self.kv_local * hd, cfg.hidden)
        self.o_proj = RowParallelLinearNorm(self.h_local * hd, cfg.hidden, cfg.eps, device, dtype)
        self.w_gate = rnd(cfg.intermediate // cfg.world, cfg.hidden)
        self.w_up = rnd(cfg.intermediate // cfg.world, cfg.hidden)
        self.down_proj = RowParallelLinearNorm(cfg.intermediate // cfg.world, cfg.hidden, cfg.eps, device, dtype)
        with torch.no_grad():
            self.o_proj.weight.copy_((torch.randn(self.o_proj.weight.shape, generator=g) * 0.02).to(dtype))
            self.down_proj.weight.copy_((torch.randn(self.down_proj.weight.shape, generator=g) * 0.02).to(dtype))

    def attention_local(self, normed: torch.Tensor) -> torch.Tensor:
        """normed: [B, S, hidden] -> this rank's heads' context [B*S, h_local*head_dim]."""
        B, S, _ = normed.shape
        hd = self.cfg.head_dim
        q = (normed @ self.wq.T).view(B, S, self.h_local, hd).transpose(1, 2)
        k = (normed @ self.wk.T).view(B, S, self.kv_local, hd).transpose(1, 2)
        v = (normed @ self.wv.T).view(B, S, self.kv_local, hd).transpose(1, 2)
        rep = self.h_local // self.kv_local
        if rep > 1:
            k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        ctx = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return ctx.transpose(1, 2).reshape(B * S, self.h_local * hd)

    def mlp_local(self, normed2d: torch.Tensor) -> torch.Tensor:
        return F.silu(normed2d @ self.w_gate.T) * (normed2d @ self.w_up.T)


def run_block(comm, ranks: Sequence[TPBlockRank], normed: Sequence[torch.Tensor], residual: Sequence[torch.Tensor],
              fused: bool = True) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
    """One decoder block for all local ranks.  normed / residual: per rank [B, S, hidden] (replicated across
    ranks): the normalised input and the residual stream.  Returns (normed input of the next block, residual)."""
    from ..parallel import tensor_parallel as tp
    B, S, H = normed[0].shape
    n = len(ranks)
    ctx = [ranks[i].attention_local(normed[i]) for i in range(n)]
    res2d = [r.reshape(B * S, H) for r in residual]
    res_mid = _residual_buffers(comm, res2d, "res_mid")
    run = tp.fused_row_parallel if fused else None
    if fused:
        h = run(comm, ctx, [m.o_proj.weight for m in ranks], [m.o_proj.norm_weight for m in ranks], res2d,
                eps=ranks[0].cfg.eps, residual_out=res_mid)
    else:
        h, res_mid = _unfused(comm, ctx, [m.o_proj.weight for m in ranks], [m.o_proj.norm_weight for m in ranks],
                              res2d, ranks[0].cfg.eps)
    act = [ranks[i].mlp_local(h[i]) for i in range(n)]
    res_out = _residual_buffers(comm, res2d, "res_out")
    if fused:
        y = run(comm, act, [m.down_proj.weight for m in ranks], [m.down_proj.norm_weight for m in ranks], res_mid,
                eps=ranks[0].cfg.eps, residual_out=res_out)
    else:
        y, res_out = _unfused(comm, act, [m.down_proj.weight for m in ranks],
                              [m.down_proj.norm_weight for m in ranks], res_mid, ranks[0].cfg.eps)
    return [t.reshape(B, S, H) for t in y], [t.reshape(B, S, H) for t in res_out]


def _residual_buffers(comm, like: Sequence[torch.Tensor], tag: str) -> List[torch.Tensor]:
    """Where a fused layer writes the updated residual stream.  With one GPU per process the row owners
    write every rank's copy, so the buffer must sit at the same offset of every rank's symmetric heap:
    one cached buffer per (tag, shape), reused by every block (the next block has consumed it by then,
    in stream order on this rank and, through the layer's own counters, on the peers)."""
    one_gpu_per_process = getattr(comm, "nlocal", 1) == 1 and getattr(comm, "world", 1) > 1 and like[0].is_cuda
    if not one_gpu_per_process or not hasattr(comm, "symm_empty"):
        return [torch.empty_like(r) for r in like]
    cache = comm.__dict__.setdefault("_fused_out", {})  # cleared by symm_reset()
    key = (tag, tuple(like[0].shape), like[0].dtype)
    if key not in cache:
        cache[key] = comm.symm_empty(list(like[0].shape), like[0].dtype)
    return [cache[key]]


def _unfused(comm, xs, ws, nws, res, eps):
    parts = [x @ w.T for x, w in zip(xs, ws)]
    res_out = [torch.empty_like(r) for r in res]
    ys = comm.all_reduce_rmsnorm(parts, nws, res, eps=eps, residual_out=res_out)
    return ys, res_out


def reference_block(ranks: Sequence[TPBlockRank], normed: torch.Tensor, residual: torch.Tensor):
    """fp64 CPU restatement of run_block over all ranks of the group."""
    B, S, H = normed.shape
    cfg = ranks[0].cfg
    ctxs = [m.double().cpu().attention_local(normed.double().cpu()) for m in ranks]
    h, res_mid = reference.row_parallel_linear_rmsnorm(ctxs, [m.o_proj.weight.T for m in ranks],
                                                       ranks[0].o_proj.norm_weight, residual.reshape(B * S, H), cfg.eps)
    acts = [m.mlp_local(h) for m in ranks]
    y, res_out = reference.row_parallel_linear_rmsnorm(acts, [m.down_proj.weight.T for m in ranks],
                                                       ranks[0].down_proj.norm_weight, res_mid, cfg.eps)
    return y.reshape(B, S, H), res_out.reshape(B, S, H)
