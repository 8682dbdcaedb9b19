"""Communicators.

`Comm` wraps the native communicator (`yali_b200._C.Comm`) and accepts either a
single tensor (one GPU per process) or one tensor per local rank (one process
driving several GPUs, or several ranks emulated on one GPU).  `GlooComm` offers
the same calls for CPU tensors on top of `torch.distributed` (gloo): it is the
plumbing path that lets programs and tests run without a GPU, never a substitute
on a machine that has one.

Reference parity: `yali::Comm` (src/ops/allreduce.cuh:78-323) and `yali::MPIComm`
(src/ops/allreduce_mpi.cuh:76-298) are the C++ counterparts; the reference has no
Python layer.
"""
from __future__ import annotations

import atexit
import os
import weakref
from typing import List, Optional, Sequence, Union

import torch

from .. import _native
from ..ops import reference

TensorOrList = Union[torch.Tensor, Sequence[torch.Tensor]]

_live: "weakref.WeakSet[Comm]" = weakref.WeakSet()


def _close_all() -> None:
    # Multicast bindings and peer mappings must be released in an orderly way before the
    # process goes away.
    for c in list(_live):
        try:
            c.close()
        except Exception:  # noqa: BLE001
            pass


atexit.register(_close_all)


class YaliTimeout(RuntimeError):
    """A device-side wait ran out; the communicator must be reset()."""


def _translate(exc: RuntimeError) -> RuntimeError:
    return YaliTimeout(str(exc)) if "YaliTimeout" in str(exc) else exc


class Comm:
    """Native communicator over NVLink peer memory."""

    def __init__(self, impl) -> None:
        self._impl = impl
        self._symm_keepalive: List[torch.Tensor] = []
        _live.add(self)

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def single_process(cls, devices: Sequence[int], heap_bytes: int = 0, want_multicast: bool = True,
                       timeout_ms: int = -1) -> "Comm":
        return cls(_native.ext().Comm.single_process(list(devices), heap_bytes, want_multicast, timeout_ms))

    @classmethod
    def emulated(cls, world: int, device: int = 0, heap_bytes: int = 0, timeout_ms: int = -1) -> "Comm":
        """`world` ranks on ONE GPU, run by a single cooperative launch per collective."""
        return cls(_native.ext().Comm.emulated(world, device, heap_bytes, timeout_ms))

    @classmethod
    def from_env(cls, device: Optional[int] = None, heap_bytes: int = 0, want_multicast: bool = True,
                 timeout_ms: int = -1) -> "Comm":
        """One GPU per process; RANK / WORLD_SIZE / LOCAL_RANK / MASTER_PORT as exported by torchrun."""
        dev = -1 if device is None else device
        comm = cls(_native.ext().Comm.from_env(dev, heap_bytes, want_multicast, timeout_ms))
        torch.cuda.set_device(comm.device)
        return comm

    # ---- facts ----------------------------------------------------------------------------
    @property
    def world(self) -> int:
        return self._impl.world

    @property
    def nlocal(self) -> int:
        return self._impl.nlocal

    @property
    def rank(self) -> int:
        return self._impl.rank(0)

    @property
    def device(self) -> int:
        return self._impl.device(0)

    @property
    def devices(self) -> List[int]:
        return [self._impl.device(i) for i in range(self.nlocal)]

    @property
    def emulated_ranks(self) -> bool:
        return self._impl.is_emulated

    @property
    def has_multicast(self) -> bool:
        return self._impl.has_multicast

    @property
    def heap_kind(self) -> str:
        return self._impl.heap_kind

    @property
    def launches(self) -> int:
        return self._impl.launches

    def layout(self) -> dict:
        return self._impl.layout()

    def last_call(self) -> dict:
        return self._impl.last_call()

    # ---- device-side timeline ------------------------------------------------------------
    def set_trace(self, on: bool) -> None:
        """While on, every collective records %globaltimer when its first CTA starts and when its
        last CTA checks out, in a ring of 4096 entries in this rank's heap (no host work per call)."""
        self._impl.set_trace(bool(on))

    def read_trace(self, local_index: int = 0, max_entries: int = 4096):
        """(traced calls so far, [(start_ns, end_ns), ...]) of the most recent calls, oldest first.
        Synchronise the streams first."""
        return self._impl.read_trace(local_index, max_entries)

    # ---- helpers --------------------------------------------------------------------------
    def _as_list(self, t: TensorOrList, what: str) -> List[torch.Tensor]:
        if isinstance(t, torch.Tensor):
            if self.nlocal != 1:
                raise ValueError(f"{what}: this communicator drives {self.nlocal} ranks; pass one tensor per rank")
            return [t]
        ts = list(t)
        if len(ts) != self.nlocal:
            raise ValueError(f"{what}: expected {self.nlocal} tensors, got {len(ts)}")
        return ts

    @staticmethod
    def _like_input(t: TensorOrList, out: List[torch.Tensor]):
        return out[0] if isinstance(t, torch.Tensor) else out

    # ---- collectives ----------------------------------------------------------------------
    def all_reduce(self, send: TensorOrList, recv: Optional[TensorOrList] = None, *, mode: str = "auto",
                   scale: Optional[float] = None, out_dtype: Optional[torch.dtype] = None, ctas: int = 0,
                   slot_bytes: int = 0, _skip_rank: int = -1):
        """recv = cast(scale * sum over ranks of send).  `recv=None` allocates; pass `recv=send` for in place.
        `_skip_rank` makes that rank's kernel leave at once: only for testing that the others time out."""
        s = self._as_list(send, "send")
        if recv is None:
            r = [torch.empty_like(x, dtype=out_dtype or x.dtype) for x in s]
        else:
            r = self._as_list(recv, "recv")
        try:
            self._impl.all_reduce(s, r, mode, scale, ctas, slot_bytes, _skip_rank)
        except RuntimeError as e:  # noqa: PERF203
            raise _translate(e) from None
        return self._like_input(send, r)

    def all_reduce_rmsnorm(self, x: TensorOrList, weight: TensorOrList, residual: Optional[TensorOrList] = None, *,
                           eps: float = 1e-5, out: Optional[TensorOrList] = None,
                           residual_out: Optional[TensorOrList] = None, mode: str = "auto", ctas: int = 0):
        """out = RMSNorm(sum over ranks of x + residual) * weight, row length = weight.numel()."""
        s = self._as_list(x, "x")
        w = self._as_list(weight, "weight")
        r = [torch.empty_like(t) for t in s] if out is None else self._as_list(out, "out")
        res = None if residual is None else self._as_list(residual, "residual")
        ro = None if residual_out is None else self._as_list(residual_out, "residual_out")
        try:
            self._impl.all_reduce_rmsnorm(s, r, res, ro, w, eps, mode, ctas)
        except RuntimeError as e:
            raise _translate(e) from None
        return self._like_input(x, r)

    def fused_linear_rmsnorm(self, x: TensorOrList, w: TensorOrList, norm_weight: TensorOrList,
                             residual: Optional[TensorOrList] = None, *, eps: float = 1e-5,
                             out: Optional[TensorOrList] = None, residual_out: Optional[TensorOrList] = None,
                             oneshot: Optional[bool] = None, ctas: int = 0, trace: Optional[TensorOrList] = None,
                             nvls: Union[None, bool, int] = None, decode: Optional[bool] = None):
        """out = RMSNorm(residual + sum over ranks of x @ w.T) * norm_weight in ONE kernel per rank
        (tcgen05 GEMM whose epilogue pushes partial rows to their owner over NVLink, then reduce + norm).
        x: [T, K], w: [N, K] (this rank's slice, nn.Linear layout), bf16.  With one GPU per process the
        two-shot form (T above a few dozen rows) needs `out` from symm_empty(); without `out` the call
        returns the first T rows of a per-width symmetric buffer of its own that the next call of that width overwrites.  `trace`: int64 CUDA
        tensor(s) of 8 elements that receive CTA 0's %globaltimer at the phase boundaries.  `nvls`: how the
        two-shot form uses the NVSwitch multicast object: None = by measurement, 0/False = not at all
        (peer pushes and peer stores), 1/True = in-switch reduce + multicast store, 2 = peer pushes +
        multicast store; 1 and 2 need the multicast object and `out` from symm_empty().  `decode`: the
        few-token form (up to 64 rows: 128 x 256 tiles whose K extent is split over CTAs, partial rows sent to every rank as
        flag-in-data lines, every rank normalises all rows): None = by size, False = never, True = required."""
        xs, ws, nws = self._as_list(x, "x"), self._as_list(w, "w"), self._as_list(norm_weight, "norm_weight")
        if out is None:
            T, N = xs[0].shape[0], ws[0].shape[0]
            if self.nlocal == 1 and self.world > 1:
                # Symmetric memory is never freed piecemeal: keep ONE output per row width, large enough for the
                # most rows seen so far (grown by doubling, so a program that varies its token count holds at
                # most twice its largest output per width), and hand out its first T rows.  The tensor returned
                # by a call is therefore overwritten by the next call of that width.
                cache = self.__dict__.setdefault("_fused_out", {})
                buf = cache.get(N)
                if buf is None or buf.shape[0] < T:
                    rows = T if buf is None else max(T, 2 * buf.shape[0])
                    buf = cache[N] = self.symm_empty([rows, N], torch.bfloat16)
                outs = [buf[:T]]
            else:
                outs = [torch.empty(T, N, dtype=torch.bfloat16, device=t.device) for t in xs]
        else:
            outs = self._as_list(out, "out")
        res = None if residual is None else self._as_list(residual, "residual")
        ro = None if residual_out is None else self._as_list(residual_out, "residual_out")
        try:
            tr = None if trace is None else self._as_list(trace, "trace")
            self._impl.fused_linear(xs, ws, nws, outs, res, ro, eps, -1 if oneshot is None else int(oneshot), ctas, tr,
                                    -1 if nvls is None else int(nvls), -1 if decode is None else int(decode))
        except RuntimeError as e:
            raise _translate(e) from None
        return self._like_input(x, outs)

    def all_reduce_host(self, src: TensorOrList, dst: Optional[TensorOrList] = None, *,
                        chunk_bytes: int = 0, scale: Optional[float] = None, mode: str = "auto",
                        copies_only: bool = False):
        """All-reduce of tensors that live in pinned host memory: dst = scale * sum over ranks of src.

        The message is cut into chunks (`chunk_bytes`; 0 = about 32 chunks of 1-8 MiB) that move through three streams per GPU: host-to-device copy,
        all-reduce, device-to-host copy.  Chunk i+1 is copied in while chunk i is reduced and chunk i-1
        is copied out, so both PCIe directions and NVLink are busy at the same time and a call costs
        about one direction's copy time instead of the sum of the three phases.  Staging is a ring of
        four symmetric chunk buffers per direction, allocated on first use and reused by every later
        call that fits (every rank must make the same calls).  The call returns with the work queued;
        the caller's current stream waits for it.  `copies_only=True` leaves the collective out
        (dst = src through the device): the ceiling the host link sets for the same call."""
        srcs = self._as_list(src, "src")
        if dst is None:
            dsts = [torch.empty_like(t).pin_memory() for t in srcs]
        else:
            dsts = self._as_list(dst, "dst")
        for t in list(srcs) + list(dsts):
            if t.is_cuda or not t.is_pinned() or not t.is_contiguous():
                raise ValueError("all_reduce_host takes contiguous tensors in pinned host memory")
        try:
            self._impl.all_reduce_host(srcs, dsts, int(chunk_bytes), scale, mode, bool(copies_only))
        except RuntimeError as e:
            raise _translate(e) from None
        return self._like_input(src, dsts)

    def shard_elems(self, count: int) -> int:
        return _native.ext().shard_elems(count, self.world)

    def reduce_scatter(self, send: TensorOrList, recv: Optional[TensorOrList] = None, *, ctas: int = 0,
                       slot_bytes: int = 0):
        """Rank q receives elements [q*S, (q+1)*S) of the sum, S = shard_elems(count) (tail padded, not written)."""
        s = self._as_list(send, "send")
        n = self.shard_elems(s[0].numel()) if self.world > 1 else s[0].numel()
        r = [torch.empty(n, dtype=x.dtype, device=x.device) for x in s] if recv is None else self._as_list(recv, "recv")
        try:
            self._impl.reduce_scatter(s, r, ctas, slot_bytes)
        except RuntimeError as e:
            raise _translate(e) from None
        return self._like_input(send, r)

    def all_gather(self, send: TensorOrList, count: int, recv: Optional[TensorOrList] = None, *, ctas: int = 0,
                   slot_bytes: int = 0):
        """Inverse of reduce_scatter: every rank contributes its shard, all receive `count` elements."""
        s = self._as_list(send, "send")
        r = [torch.empty(count, dtype=x.dtype, device=x.device) for x in s] if recv is None \
            else self._as_list(recv, "recv")
        try:
            self._impl.all_gather(s, r, ctas, slot_bytes)
        except RuntimeError as e:
            raise _translate(e) from None
        return self._like_input(send, r)

    # ---- symmetric memory -----------------------------------------------------------------
    def symm_empty(self, shape, dtype: torch.dtype = torch.float32):
        """Pre-allocated buffer at the same heap offset on every rank (zero-copy paths, NVLS in place).
        Every process must issue the same sequence of symm_empty calls.  Valid until close()."""
        if isinstance(shape, int):
            shape = [shape]
        ts = self._impl.symm_empty(list(shape), dtype)
        return ts[0] if self.nlocal == 1 else ts

    def symm_reset(self) -> None:
        self.__dict__.pop("_fused_out", None)  # cached outputs lived in the symmetric heap
        self._impl.symm_reset()

    # ---- control --------------------------------------------------------------------------
    def sync(self) -> None:
        try:
            self._impl.sync()
        except RuntimeError as e:
            raise _translate(e) from None

    def check(self) -> None:
        try:
            self._impl.check()
        except RuntimeError as e:
            raise _translate(e) from None

    def reset(self) -> None:
        self._impl.reset()

    def barrier(self) -> None:
        self._impl.barrier()

    def status(self) -> str:
        return self._impl.status()

    def allgather_object_bytes(self, data: bytes) -> List[bytes]:
        """Host-side all-gather of equally sized byte strings over the control plane."""
        out = self._impl.allgather_bytes(data)
        n = len(data)
        return [out[i * n:(i + 1) * n] for i in range(self.world if self.nlocal == 1 else 1)]

    def raw_handle(self) -> int:
        return self._impl.raw()

    def close(self) -> None:
        if self._impl is not None:
            self._impl.close()
            self._impl = None
            _live.discard(self)

    def __enter__(self) -> "Comm":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


class GlooComm:
    """Same surface over torch.distributed for CPU tensors (no GPU needed)."""

    def __init__(self, group=None) -> None:
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self._dist = dist
        self._group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nlocal = 1
        self.has_multicast = False
        self.heap_kind = "gloo"
        self.launches = 0

    def all_reduce(self, send: torch.Tensor, recv: Optional[torch.Tensor] = None, *, mode: str = "auto",
                   scale: Optional[float] = None, out_dtype: Optional[torch.dtype] = None, ctas: int = 0,
                   slot_bytes: int = 0) -> torch.Tensor:
        acc = send.detach().to(torch.float32).clone()
        self._dist.all_reduce(acc, group=self._group)
        if scale is not None:
            acc.mul_(scale)
        dt = out_dtype or (recv.dtype if recv is not None else send.dtype)
        if recv is None:
            return acc.to(dt)
        recv.copy_(acc.to(dt))
        return recv

    def all_reduce_rmsnorm(self, x, weight, residual=None, *, eps: float = 1e-5, out=None, residual_out=None,
                           mode: str = "auto", ctas: int = 0):
        acc = x.detach().to(torch.float32).clone()
        self._dist.all_reduce(acc, group=self._group)
        y, pre = reference.residual_rmsnorm(acc, weight, residual, eps)
        if residual_out is not None:
            residual_out.copy_(pre.to(residual_out.dtype))
        if out is None:
            return y.to(x.dtype)
        out.copy_(y.to(out.dtype))
        return out

    def fused_linear_rmsnorm(self, x, w, norm_weight, residual=None, *, eps: float = 1e-5, out=None,
                             residual_out=None, oneshot=None, ctas: int = 0, trace=None, nvls=None):
        """Same call as Comm.fused_linear_rmsnorm: RMSNorm(residual + sum over ranks of x @ w.T) * norm_weight.
        On CPU: fp32 matmul, all-reduce, norm (the options that pick a GPU form are accepted and ignored)."""
        partial = x.detach().to(torch.float32) @ w.detach().to(torch.float32).T
        y = self.all_reduce_rmsnorm(partial, norm_weight, residual, eps=eps, residual_out=residual_out)
        if out is None:
            return y.to(x.dtype)
        out.copy_(y.to(out.dtype))
        return out

    def symm_empty(self, shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Plain host tensor: there is no symmetric heap on CPU, every buffer is as good as any other."""
        return torch.empty([shape] if isinstance(shape, int) else list(shape), dtype=dtype)

    def symm_reset(self) -> None:
        pass

    def reset(self) -> None:
        self._dist.barrier(group=self._group)

    def shard_elems(self, count: int) -> int:
        return _native.lib().yali_c_shard_elems(count, self.world)

    def reduce_scatter(self, send, recv=None, **_):
        full = self.all_reduce(send)
        s = self.shard_elems(send.numel()) if self.world > 1 else send.numel()
        out = torch.zeros(s, dtype=send.dtype) if recv is None else recv
        lo = min(self.rank * s, send.numel())
        hi = min(lo + s, send.numel())
        out[:hi - lo] = full.reshape(-1)[lo:hi]
        return out

    def all_gather(self, send, count, recv=None, **_):
        s = self.shard_elems(count) if self.world > 1 else count
        parts = [torch.empty(s, dtype=send.dtype) for _ in range(self.world)]
        self._dist.all_gather(parts, send.reshape(-1)[:s].contiguous(), group=self._group)
        full = torch.cat(parts)[:count]
        if recv is None:
            return full
        recv.copy_(full)
        return recv

    def all_reduce_host(self, src: torch.Tensor, dst: Optional[torch.Tensor] = None, *, chunk_bytes: int = 0,
                        scale: Optional[float] = None, mode: str = "auto") -> torch.Tensor:
        """Same call as Comm.all_reduce_host; on CPU the data is in host memory already."""
        return self.all_reduce(src, dst, scale=scale)

    def sync(self) -> None:
        pass

    def check(self) -> None:
        pass

    def barrier(self) -> None:
        self._dist.barrier(group=self._group)

    def close(self) -> None:
        pass


_default = None


def init_process_group(device: Optional[int] = None, heap_bytes: int = 0, want_multicast: bool = True,
                       timeout_ms: int = -1, backend: Optional[str] = None):
    """Creates the default communicator from the launcher's environment.

    With a GPU: the native communicator (one GPU per process).  Without one (or with
    backend="gloo"): torch.distributed over gloo, rendezvous on MASTER_ADDR/MASTER_PORT."""
    global _default
    if _default is not None:
        return _default
    use_gpu = torch.cuda.is_available() and backend != "gloo"
    if use_gpu:
        _default = Comm.from_env(device, heap_bytes, want_multicast, timeout_ms)
    else:
        import torch.distributed as dist
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group("gloo", rank=int(os.environ.get("RANK", "0")),
                                    world_size=int(os.environ.get("WORLD_SIZE", "1")))
        _default = GlooComm()
    return _default


def get_default_comm():
    if _default is None:
        raise RuntimeError("yali_b200.init_process_group() has not been called")
    return _default


def destroy_process_group() -> None:
    global _default
    if _default is not None:
        _default.close()
        _default = None
