"""Loading of the native parts: `libyali_b200.so` through ctypes (host-side
functions that need no GPU) and the `_C` torch extension (everything that touches
a GPU).  Both are built in-tree by `yali_b200._build`; nothing falls back to
Python silently: on a machine with a GPU a missing extension is an error."""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_ROOT = Path(__file__).resolve().parent
_LIB_PATH = _ROOT / "lib" / "libyali_b200.so"
_lib = None
_ext = None


class PlanCaps(ctypes.Structure):
    _fields_ = [("flash_cap", ctypes.c_uint64), ("ring_bytes", ctypes.c_uint64), ("nvls_cap", ctypes.c_uint64),
                ("has_multicast", ctypes.c_int), ("symmetric", ctypes.c_int), ("peer_recv", ctypes.c_int),
                ("vec_ok", ctypes.c_int), ("max_ctas", ctypes.c_uint32), ("ll_cap", ctypes.c_uint64),
                ("peer_send", ctypes.c_int), ("in_place", ctypes.c_int), ("one_gpu_per_rank", ctypes.c_int)]


class Plan(ctypes.Structure):
    _fields_ = [("variant", ctypes.c_int), ("ctas", ctypes.c_uint32), ("slot_bytes", ctypes.c_uint32),
                ("max_iters", ctypes.c_uint32), ("flags", ctypes.c_uint32), ("shard_elems", ctypes.c_uint64),
                ("stages", ctypes.c_uint32), ("smem_bytes", ctypes.c_uint32)]


class SimConfig(ctypes.Structure):
    _fields_ = [("mode", ctypes.c_int), ("world", ctypes.c_int), ("lanes", ctypes.c_int), ("calls", ctypes.c_int),
                ("count", ctypes.c_uint64), ("slot_elems", ctypes.c_uint32), ("direct_ag", ctypes.c_int),
                ("fault", ctypes.c_int), ("fault_rank", ctypes.c_int), ("fault_call", ctypes.c_int),
                ("timeout_ms", ctypes.c_int), ("seed", ctypes.c_uint64)]


class FusedSimConfig(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("ctas", ctypes.c_int), ("calls", ctypes.c_int), ("oneshot", ctypes.c_int),
                ("rows", ctypes.c_uint32), ("col_tiles", ctypes.c_uint32),
                ("fault", ctypes.c_int), ("fault_rank", ctypes.c_int), ("fault_call", ctypes.c_int),
                ("slow_rank", ctypes.c_int), ("single_parity", ctypes.c_int), ("timeout_ms", ctypes.c_int),
                ("in_switch", ctypes.c_int), ("ksplit", ctypes.c_int)]


class SimReport(ctypes.Structure):
    _fields_ = [("status", ctypes.c_int), ("mismatches", ctypes.c_uint64), ("timeouts", ctypes.c_uint64),
                ("max_outstanding_slots", ctypes.c_uint64), ("flag_writes", ctypes.c_uint64),
                ("timeout_rank", ctypes.c_int), ("timeout_peer", ctypes.c_int), ("timeout_site", ctypes.c_int)]


def _declare(lib: ctypes.CDLL) -> None:
    c = ctypes
    u64, u32, i32, f32, f64, vp, cp = c.c_uint64, c.c_uint32, c.c_int, c.c_float, c.c_double, c.c_void_p, c.c_char_p
    sig = {
        "yali_c_version": (cp, []),
        "yali_c_error_string": (cp, [i32]),
        "yali_c_bootstrap_create": (vp, [i32, i32, i32, cp, i32, cp, c.c_size_t]),
        "yali_c_bootstrap_from_env": (vp, [cp, c.c_size_t]),
        "yali_c_bootstrap_destroy": (None, [vp]),
        "yali_c_bootstrap_rank": (i32, [vp]),
        "yali_c_bootstrap_world": (i32, [vp]),
        "yali_c_bootstrap_allgather": (i32, [vp, vp, vp, c.c_size_t]),
        "yali_c_bootstrap_broadcast": (i32, [vp, vp, c.c_size_t, i32]),
        "yali_c_bootstrap_barrier": (i32, [vp]),
        "yali_c_bootstrap_allgather_fd": (i32, [vp, i32, c.POINTER(i32)]),
        "yali_c_bootstrap_broadcast_fd": (i32, [vp, c.POINTER(i32)]),
        "yali_c_bootstrap_last_error": (cp, [vp]),
        "yali_c_flash_crossover_bytes": (u64, [i32, i32]),
        "yali_c_flash_lane_preset": (i32, [u64, i32, i32]),
        "yali_c_stream_lane_preset": (i32, [u64, i32, i32]),
        "yali_c_auto_slot_bytes": (u64, [u64, i32]),
        "yali_c_clamp_slot_bytes": (u64, [u64, u64]),
        "yali_c_auto_ctas_per_lane": (i32, [i32, i32, u64, u64]),
        "yali_c_shard_elems": (u64, [u64, i32]),
        "yali_c_make_plan": (i32, [i32, u64, i32, i32, i32, i32, c.POINTER(PlanCaps), cp, c.POINTER(Plan), cp,
                                   c.c_size_t]),
        "yali_c_heap_layout": (i32, [i32, u64, c.POINTER(u64)]),
        "yali_c_flash_slice": (None, [u64, i32, u32, u32, i32, c.POINTER(u64)]),
        "yali_c_stream_piece": (None, [u64, u64, u64, u32, u32, u32, i32, c.POINTER(u64)]),
        "yali_c_stream_iters": (u32, [u64, u64, u32, u32]),
        "yali_c_philox": (None, [u64, u64, c.POINTER(u32)]),
        "yali_c_random_value": (f32, [i32, u64, u64]),
        "yali_c_fill_random": (None, [vp, u64, i32, u64, i32]),
        "yali_c_round_bf16": (f32, [f32]),
        "yali_c_round_fp16": (f32, [f32]),
        "yali_c_oracle_allreduce": (None, [vp, i32, c.c_size_t, f64, vp]),
        "yali_c_oracle_residual_rmsnorm": (None, [vp, vp, vp, c.c_size_t, c.c_size_t, f64, vp, vp]),
        "yali_c_fused_linear_counts": (None, [c.c_uint32, c.c_uint32, i32, i32, vp, vp]),
        "yali_c_fused_decode_split": (u32, [u32, u32, u32, i32, u32, u64, u32]),
        "yali_c_fused_decode_tile": (u32, [u32, u32, u32]),
        "yali_c_fused_tile_split": (u32, [u32, u32, u32, i32, u32, u64, u32]),
        "yali_c_fused_linear_oneshot_max_rows": (c.c_uint32, [i32]),
        "yali_c_fused_linear_multicast_mode": (i32, [i32, c.c_uint32]),
        "yali_c_oracle_gemm": (None, [vp, vp, c.c_size_t, c.c_size_t, c.c_size_t, vp]),
        "yali_c_verify_allreduce_sum": (i32, [vp, c.c_size_t, f32, f32, c.POINTER(c.c_size_t),
                                              c.POINTER(c.c_size_t)]),
        "yali_c_simulate": (i32, [c.POINTER(SimConfig), c.POINTER(SimReport)]),
        "yali_c_simulate_fused": (i32, [c.POINTER(FusedSimConfig), c.POINTER(SimReport)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def lib() -> ctypes.CDLL:
    """The host library; built on first use when missing."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            from . import _build
            _build.build_library(verbose=False)
        _lib = ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def ext():
    """The torch extension module (`yali_b200._C`)."""
    global _ext
    if _ext is None:
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        lib()
        try:
            from . import _C as mod
        except ImportError as first:
            if os.environ.get("YALI_NO_AUTOBUILD"):
                raise
            from . import _build
            try:
                _build.build_torch_extension(verbose=False)
                from . import _C as mod
            except Exception as second:  # noqa: BLE001
                raise ImportError(f"yali_b200._C is not built and could not be built in-tree: {first}; {second}")
        _ext = mod
    return _ext


def ext_available() -> bool:
    return (_ROOT / "_C.so").exists()
