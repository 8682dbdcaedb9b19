"""Host-only logic: enums and names, tuning functions, the planner, the heap layout,
partition arithmetic (property tests), the generator and the CPU oracles.

Reference counterparts: tests/unit/test_all_reduce_interface.cu (enum names, config
defaults), tests/unit/test_all_reduce_correctness.cu:165-208 (tuning ranges),
tests/unit/test_validation.cu:13-59 (VerifyAllReduceSum)."""
import ctypes
import json

import numpy as np
import pytest

from yali_b200 import _native
from yali_b200._native import Plan, PlanCaps

FP32, FP16, BF16 = 0, 1, 2
MiB = 1 << 20


def caps(world, **kw):
    c = PlanCaps(flash_cap=(64 if world == 2 else 16 if world <= 4 else 8) * MiB, ring_bytes=256 * MiB,
                 nvls_cap=64 * MiB, has_multicast=0, symmetric=0, peer_recv=0, vec_ok=1, max_ctas=1184, ll_cap=1 * MiB)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def make_plan(lib, world, count, in_dt=FP32, out_dt=None, epi=0, mode=0, cp=None, table=None):
    plan = Plan()
    err = ctypes.create_string_buffer(256)
    c = cp or caps(world)
    rc = lib.yali_c_make_plan(world, count, in_dt, in_dt if out_dt is None else out_dt, epi, mode, ctypes.byref(c),
                              table.encode() if table else None, ctypes.byref(plan), err, 256)
    return rc, plan, err.value.decode()


def test_version_and_errors(native_lib):
    assert b"yali" in native_lib.yali_c_version()
    names = [native_lib.yali_c_error_string(i).decode() for i in range(8)]
    assert names[0] == "Success" and "timed out" in names[5] and len(set(names)) == 8


def test_tuning_functions_sane(native_lib):
    lib = native_lib
    for world in (2, 4, 8):
        cross = lib.yali_c_flash_crossover_bytes(FP32, world)
        assert 64 * 1024 <= cross <= 64 * MiB
        prev = 0
        for shift in range(10, 32):
            b = 1 << shift
            lanes = lib.yali_c_flash_lane_preset(b, FP32, world)
            assert 1 <= lanes <= 2048
            assert lanes >= prev  # more data never means fewer CTAs
            prev = lanes
            s_lanes = lib.yali_c_stream_lane_preset(b, BF16, world)
            assert 1 <= s_lanes <= 256
            slot = lib.yali_c_auto_slot_bytes(b, world)
            assert 8 * 1024 <= slot <= 256 * 1024 and slot % 256 == 0
    assert 32 * MiB <= lib.yali_c_flash_crossover_bytes(FP32, 2) < 64 * MiB  # measured: two-shot wins from 64 MiB
    assert lib.yali_c_clamp_slot_bytes(100, 1 << 20) == 256
    assert lib.yali_c_clamp_slot_bytes(1 << 30, 1 << 16) == 1 << 16
    assert lib.yali_c_auto_ctas_per_lane(0, 16, 1 << 20, 2048) == 1
    assert 1 <= lib.yali_c_auto_ctas_per_lane(1, 16, 1 << 20, 2048) <= 32
    assert lib.yali_c_auto_ctas_per_lane(1, 16, 0, 2048) == 1


def test_shard_elems(native_lib):
    for world in range(1, 9):
        for count in (1, 7, 31, 32, 33, 1000, 262144, (1 << 29) + 3):
            s = native_lib.yali_c_shard_elems(count, world)
            assert s % 16 == 0 and s * world >= count and (s - 16) * world < count


def test_heap_layout(native_lib):
    f = (ctypes.c_uint64 * 16)()
    for world in (1, 2, 4, 8):
        assert native_lib.yali_c_heap_layout(world, 0, f) == 0
        total, flags_off, flash_off, flash_cap, ring_off, ring_bytes, nvls_off, nvls_cap, gemm_off, gemm_cap, \
            user_off, user_bytes, ll_off, ll_cap, gll_off, gll_cap = list(f)
        assert flags_off == 0 and user_off + user_bytes == total and user_bytes >= 256 * MiB
        if world > 1:
            assert flash_off >= 1 * MiB
            assert ring_off == flash_off + 2 * (world - 1) * flash_cap
            assert nvls_off == ring_off + ring_bytes
            assert gemm_off == nvls_off + 2 * nvls_cap
            assert ll_off == gemm_off + 2 * world * gemm_cap
            assert gll_off == ll_off + 2 * (world - 1) * 2 * ll_cap
            assert user_off == gll_off + 2 * world * gll_cap and gll_cap >= 64 * 4096 * 4
    assert native_lib.yali_c_heap_layout(8, 1 * MiB, f) != 0  # too small for the fixed regions
    # Every region starts on a 4 KiB boundary for every world size (vector accesses, bulk copies).
    for world in range(1, 9):
        assert native_lib.yali_c_heap_layout(world, 0, f) == 0
        total, flags_off, flash_off, flash_cap, ring_off, ring_bytes, nvls_off, nvls_cap, gemm_off, gemm_cap, \
            user_off, user_bytes, ll_off, ll_cap, gll_off, gll_cap = list(f)
        for off in (flash_off, ring_off, nvls_off, gemm_off, ll_off, gll_off, user_off, flash_cap, gemm_cap, ll_cap):
            assert off % 4096 == 0, (world, off)


def test_few_token_form_splits_k_to_eight_sources(native_lib):
    """K splits per 256-column tile of the few-token fused layer: world x splits = 8 sources where K allows,
    never more rows per split than the landing zone holds, never more work items than resident CTAs, no
    empty split."""
    f = native_lib.yali_c_fused_decode_split
    cap = 4 * MiB
    assert f(1, 4096, 2048, 2, 148, cap, 0) == 4      # TP = 2: 16 tiles x 4 splits of eight k-blocks
    assert f(16, 4096, 1024, 4, 148, cap, 0) == 2     # TP = 4
    assert f(16, 4096, 512, 8, 148, cap, 0) == 1      # TP = 8: eight sources already
    assert f(64, 4096, 2048, 2, 148, cap, 0) == 4     # 64 rows x 4096 x 4 bytes x 4 splits = 4 MiB: just fits
    assert f(64, 4096, 2048, 2, 148, 1 * MiB, 0) == 1
    assert f(1, 4096, 2048, 2, 74, cap, 0) == 4       # two emulated ranks on one GPU: 64 items on 74 CTAs
    assert f(1, 4096, 2048, 2, 37, cap, 0) == 2
    assert f(1, 4096, 128, 2, 148, cap, 0) == 1       # two k-blocks: nothing to split
    assert f(1, 4096, 2048, 2, 148, cap, 8) == 8      # forced (measurements)
    tile = native_lib.yali_c_fused_decode_tile
    assert tile(4096, 4, 148) == 128 and tile(4096, 8, 148) == 256 and tile(4096, 1, 18) == 256 and tile(1024, 2, 74) == 128
    assert f(1, 4096, 192, 2, 148, cap, 8) == 2       # three k-blocks: a third and fourth split would be empty
    for T, N, K, W in [(5, 512, 192, 3), (40, 2048, 1024, 2), (8, 128, 64, 8), (33, 4096, 4096, 2)]:
        ks = f(T, N, K, W, 148, cap, 0)
        kblocks, ntn = K // 64, -(-N // 256)
        kper = -(-kblocks // ks)
        assert ks in (1, 2, 4, 8) and T * N * 4 * ks <= cap and ntn * ks <= 148 and (ks - 1) * kper < kblocks


def test_one_shot_tile_form_splits_k(native_lib):
    """K splits per tile of a one-shot call of the tile form: only while world x splits <= 8, every split keeps
    four k-blocks, the items fit the GPU and the partial rows fit the landing zone."""
    f = native_lib.yali_c_fused_tile_split
    cap2, cap4 = 8 * MiB, 4 * MiB  # 16 MiB / world
    assert f(64, 4096, 2048, 2, 148, cap2, 0) == 4    # 16 tiles x 4 splits of eight k-blocks, 2 MiB to the peer
    assert f(128, 4096, 2048, 2, 148, cap2, 0) == 2   # four splits would send 4 MiB to the peer
    assert f(256, 4096, 2048, 2, 148, cap2, 0) == 2   # 4 MiB with two splits: still ahead of the two-shot
    assert f(128, 4096, 2048, 2, 148, cap2, 4) == 4   # forced (measurements)
    assert f(32, 4096, 1024, 4, 148, cap4, 0) == 2    # world x splits = 8
    assert f(32, 4096, 512, 8, 148, 2 * MiB, 0) == 1  # eight ranks: no room for splits
    assert f(128, 4096, 512, 2, 148, cap2, 0) == 2    # eight k-blocks: two splits of four
    assert f(128, 4096, 256, 2, 148, cap2, 0) == 1
    assert f(64, 4096, 2048, 2, 37, cap2, 0) == 2     # 16 tiles x 2 on 37 resident CTAs
    assert f(512, 4096, 2048, 2, 148, cap2, 0) == 1   # 8 MiB to the peer with two splits
    assert f(128, 4096, 2048, 2, 148, cap2, 2) == 2   # forced (measurements)


def test_plan_copy_engine_path(native_lib, monkeypatch):
    """The copy-engine path: one-shot at two ranks, two-shot over shards above, at most 64 chunks per
    rank, only for plain sums between addressable buffers of ranks that each own a GPU."""
    lib = native_lib
    ok = dict(peer_recv=1, peer_send=1, one_gpu_per_rank=1)
    rc, p, _ = make_plan(lib, 2, 32 * MiB, mode=6, cp=caps(2, **ok))  # 128 MiB
    assert rc == 0 and p.variant == 6 and p.flags & 256 and p.slot_bytes == 16 * MiB and p.stages == 3
    rc, p, _ = make_plan(lib, 2, 32 * MiB, mode=6, cp=caps(2, in_place=1, **ok))
    assert rc == 0 and p.variant == 6  # in place is handled by a per-chunk handshake
    rc, p, _ = make_plan(lib, 4, 32 * MiB, mode=6, cp=caps(4, **ok))
    assert rc == 0 and p.variant == 6 and not (p.flags & 256) and p.shard_elems == 8 * MiB and p.slot_bytes == 4 * MiB
    rc, p, _ = make_plan(lib, 2, 1 << 30, mode=6, cp=caps(2, **ok))  # 4 GiB: the chunk grows to keep 64 chunks
    assert rc == 0 and p.slot_bytes == 64 * MiB
    rc, p, _ = make_plan(lib, 2, 100001, mode=6, cp=caps(2, **ok))
    assert rc == 0 and p.slot_bytes == MiB and p.ctas >= 1
    for bad in (dict(ok, one_gpu_per_rank=0), dict(ok, peer_send=0), dict(ok, vec_ok=0)):
        rc, _, msg = make_plan(lib, 2, 32 * MiB, mode=6, cp=caps(2, **bad))
        assert rc != 0 and "cannot run" in msg
    rc, _, msg = make_plan(lib, 4, 40, mode=6, cp=caps(4, **ok))  # the last rank's shard would be empty
    assert rc != 0
    rc, _, msg = make_plan(lib, 2, 32 * MiB, out_dt=BF16, mode=6, cp=caps(2, **ok))
    assert rc != 0  # no conversion on this path
    # by size only from YALI_CE_MIN_BYTES on
    rc, p, _ = make_plan(lib, 2, 32 * MiB, cp=caps(2, **ok))
    assert rc == 0 and p.variant == 5
    monkeypatch.setenv("YALI_CE_MIN_BYTES", str(64 * MiB))
    rc, p, _ = make_plan(lib, 2, 32 * MiB, cp=caps(2, **ok))
    assert rc == 0 and p.variant == 6
    rc, p, _ = make_plan(lib, 2, 8 * MiB, cp=caps(2, **ok))
    assert rc == 0 and p.variant != 6


def test_plan_pipelined_variants_need_addressable_buffers(native_lib):
    lib = native_lib
    addressable = dict(peer_recv=1, peer_send=1)
    rc, p, _ = make_plan(lib, 2, 1 << 20, mode=4, cp=caps(2, **addressable))  # 4 MiB at two ranks, forced pull
    assert rc == 0 and p.variant == 4 and p.flags & 256 and p.stages >= 2 and p.smem_bytes == p.stages * 2 * p.slot_bytes
    assert p.smem_bytes <= 100 * 1024  # two CTAs share an SM
    rc, p, msg = make_plan(lib, 2, 1 << 20, mode=4, cp=caps(2, in_place=1, **addressable))
    assert rc != 0 and "cannot run" in msg  # the one-shot pull cannot run in place
    rc, p, _ = make_plan(lib, 2, 1 << 20, cp=caps(2, **addressable))
    assert rc == 0 and p.variant == 0  # by size the staged one-shot keeps 4 MiB (measured faster than the pull)
    rc, p, _ = make_plan(lib, 2, 32 * MiB, cp=caps(2, **addressable))  # 128 MiB: pipelined two-shot, one CTA per SM
    assert rc == 0 and p.variant == 5 and p.ctas == 148 and p.shard_elems == 16 * MiB
    assert p.slot_bytes == 32768 and p.stages == 3 and p.smem_bytes == 3 * 2 * 32768
    rc, p, _ = make_plan(lib, 2, 32 * MiB, cp=caps(2, in_place=1, **addressable))
    assert rc == 0 and p.variant == 5  # safe in place
    rc, p, _ = make_plan(lib, 2, 32 * MiB)  # plain buffers: the ring kernel
    assert rc == 0 and p.variant == 1
    rc, p, _ = make_plan(lib, 2, 1024, cp=caps(2, **addressable))
    assert rc == 0 and p.variant == 0 and p.flags & 64  # tiny messages keep the flag-in-data one-shot
    for world in (3, 5, 8):
        rc, p, _ = make_plan(lib, world, 32 * MiB, cp=caps(world, **addressable))
        assert rc == 0 and p.variant == 5 and p.stages * world * p.slot_bytes == p.smem_bytes <= 100 * 1024
    rc, p, msg = make_plan(lib, 2, 4096, mode=4)  # forced pull without addressable inputs
    assert rc != 0 and "cannot run" in msg
    rc, p, _ = make_plan(lib, 2, 4096, mode=5, cp=caps(2, vec_ok=0, **addressable))
    assert rc != 0  # 16-byte vectors into the peers' outputs need aligned buffers everywhere
    # In place on symmetric buffers the in-switch one-shot becomes the two-shot form.
    rc, p, _ = make_plan(lib, 8, 32768, cp=caps(8, has_multicast=1, symmetric=1, in_place=1))
    assert rc == 0 and p.variant == 3
    rc, p, _ = make_plan(lib, 8, 8192, mode=3, cp=caps(8, has_multicast=1, symmetric=1, in_place=1))
    assert rc == 0 and p.variant == 3


@pytest.mark.parametrize("world", [2, 4, 8])
def test_plan_of_staged_variants_ignores_local_alignment(native_lib, world):
    """With one GPU per process a rank's alignment is a local fact: two ranks must reach the same plan
    whether or not their own buffers are 16-byte aligned (symmetric buffers share their alignment)."""
    for count in (4, 1024, 65536, 1 << 20, 1 << 24, (1 << 26) + 4):
        for mc in (0, 1):
            plans = []
            for vec_ok in (0, 1):
                rc, p, _ = make_plan(native_lib, world, count, cp=caps(world, has_multicast=mc, vec_ok=vec_ok))
                assert rc == 0
                plans.append((p.variant, p.ctas, p.slot_bytes, p.shard_elems, p.stages, p.flags & ~1))
            assert plans[0] == plans[1], (count, mc, plans)


def test_plan_auto_selection(native_lib):
    lib = native_lib
    rc, p, _ = make_plan(lib, 2, 262144)  # 1 MiB fp32 at two ranks: one-shot
    assert rc == 0 and p.variant == 0 and p.ctas >= 32
    rc, p, _ = make_plan(lib, 2, 64 * MiB)  # 256 MiB: two-shot
    assert rc == 0 and p.variant == 1 and p.slot_bytes % 256 == 0 and p.max_iters >= 1
    assert p.ctas * (2 - 1) * 4 * 2 * p.slot_bytes <= 256 * MiB
    rc, p, _ = make_plan(lib, 8, 64 * MiB, cp=caps(8, has_multicast=1, symmetric=1))
    assert rc == 0 and p.variant == 3  # NVLS two-shot when multicast is there
    rc, p, _ = make_plan(lib, 8, 64 * MiB, cp=caps(8, has_multicast=1, symmetric=0))
    assert rc == 0 and p.variant == 1  # 256 MiB does not fit the NVLS staging: ring kernel
    rc, p, _ = make_plan(lib, 8, 1024)
    assert rc == 0 and p.variant == 0 and p.ctas <= 2 and p.flags & 64  # flag-in-data form for tiny messages
    rc, p, _ = make_plan(lib, 8, 32768, cp=caps(8, has_multicast=1, symmetric=1))
    assert rc == 0 and p.variant == 2  # 128 KiB at 8 ranks, symmetric buffers: in-switch one-shot
    rc, p, _ = make_plan(lib, 8, 32768, cp=caps(8, has_multicast=1, symmetric=0))
    assert rc == 0 and p.variant == 0  # plain buffers stay with the peer-to-peer one-shot
    rc, p, _ = make_plan(lib, 8, 1024, cp=caps(8, vec_ok=0))
    assert rc == 0 and p.flags & 64  # a rank's own alignment never changes the plan (its peers cannot know it)
    rc, p2, _ = make_plan(lib, 8, 1024, cp=caps(8, vec_ok=1))
    assert (p.variant, p.ctas, p.flags & ~1) == (p2.variant, p2.ctas, p2.flags & ~1)


def test_plan_forced_modes_and_errors(native_lib):
    lib = native_lib
    rc, p, _ = make_plan(lib, 4, 1 << 20, mode=2)
    assert rc == 0 and p.variant == 1
    rc, p, msg = make_plan(lib, 4, 1 << 20, mode=3)  # NVLS forced without multicast
    assert rc == 6 and "cannot run" in msg
    rc, p, msg = make_plan(lib, 2, 128 * MiB, mode=1)  # one-shot forced beyond its staging
    assert rc == 6
    rc, p, _ = make_plan(lib, 2, 4096 * 64, in_dt=BF16, epi=2)  # row-wise epilogue: one-shot only
    assert rc == 0 and p.variant == 0
    rc, p, _ = make_plan(lib, 9, 10)
    assert rc == 1


def test_plan_respects_max_ctas(native_lib):
    rc, p, _ = make_plan(native_lib, 8, 1 << 22, cp=caps(8, max_ctas=37))
    assert rc == 0 and p.ctas <= 37
    rc, p, _ = make_plan(native_lib, 8, 1 << 16, cp=caps(8, max_ctas=37))
    assert rc == 0 and p.ctas <= 37


def test_tuning_table_override(native_lib):
    table = json.dumps({"rows": [
        {"world": 2, "elem_bytes": 4, "max_bytes": 65536, "variant": "stream", "ctas": 8, "slot_bytes": 4096},
        {"world": 2, "elem_bytes": 0, "max_bytes": 1 << 40, "variant": "flash", "ctas": 77, "busbw": 123.4},
    ]})
    rc, p, _ = make_plan(native_lib, 2, 4096, table=table)  # 16 KiB fp32 -> first row
    assert rc == 0 and p.variant == 1 and p.slot_bytes == 4096 and p.ctas <= 8
    rc, p, _ = make_plan(native_lib, 2, 1 << 20, table=table)  # 4 MiB -> wildcard row
    assert rc == 0 and p.variant == 0 and p.ctas == 77
    rc, p, msg = make_plan(native_lib, 2, 4096, table='{"rows": [{"world": 2}]}')
    assert rc == 1 and "tuning table" in msg


@pytest.mark.parametrize("count", [0, 1, 7, 31, 32, 33, 4099, 262144, 1000003])
@pytest.mark.parametrize("ctas", [1, 3, 8, 37, 256])
@pytest.mark.parametrize("vec", [4, 8])
def test_flash_slices_partition_the_message(native_lib, count, ctas, vec):
    ranges = {}
    for vec_ok in (1, 0):
        covered = np.zeros(count, dtype=np.int32)
        o = (ctypes.c_uint64 * 4)()
        for cta in range(ctas):
            native_lib.yali_c_flash_slice(count, vec, ctas, cta, vec_ok, o)
            vb, ve, tb, te = list(o)
            assert vb <= ve and tb <= te
            covered[vb * vec:ve * vec] += 1
            covered[tb:te] += 1
            # CTA c of an aligned rank and CTA c of a misaligned rank cover the same elements
            # (they synchronise only with each other).
            lo = min(vb * vec, tb) if ve > vb else tb
            ranges.setdefault(cta, set()).add((lo, te))
        assert (covered == 1).all()
    assert all(len(v) == 1 for v in ranges.values())


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("count", [1, 17, 4099, 100000])
@pytest.mark.parametrize("lanes,piece", [(1, 16), (3, 64), (7, 1024)])
def test_stream_pieces_partition_the_message(native_lib, world, count, lanes, piece):
    shard = native_lib.yali_c_shard_elems(count, world)
    covered = np.zeros(count, dtype=np.int32)
    o = (ctypes.c_uint64 * 2)()
    for q in range(world):
        for lane in range(lanes):
            iters = native_lib.yali_c_stream_iters(shard, piece, lanes, lane)
            for it in range(iters):
                native_lib.yali_c_stream_piece(count, shard, piece, lanes, lane, it, q, o)
                eb, ee = list(o)
                assert eb <= ee <= count and ee - eb <= piece
                assert eb % 16 == 0 or eb == count  # vector paths start on 16-element boundaries
                covered[eb:ee] += 1
    assert (covered == 1).all()
    # every rank runs the same number of iterations per lane (the sequence numbers rely on it)
    total = sum(native_lib.yali_c_stream_iters(shard, piece, lanes, lane) for lane in range(lanes))
    assert total == -(-shard // piece)


def test_philox_reference_vector_and_determinism(native_lib):
    o = (ctypes.c_uint32 * 4)()
    # Known-answer test of Philox4x32-10 (counter 0, key 0) from the Random123 distribution.
    native_lib.yali_c_philox(0, 0, o)
    assert [hex(x) for x in o] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    a = [native_lib.yali_c_random_value(0, 1234, i) for i in range(1000)]
    b = [native_lib.yali_c_random_value(0, 1234, i) for i in range(1000)]
    c = [native_lib.yali_c_random_value(0, 1235, i) for i in range(1000)]
    assert a == b and a != c and all(-1.0 < x < 1.0 for x in a)
    n = np.array([native_lib.yali_c_random_value(1, 99, i) for i in range(20000)])
    assert abs(n.mean()) < 0.03 and abs(n.std() - 1.0) < 0.03


def test_rounding_helpers_match_torch(native_lib):
    import torch
    xs = np.concatenate([np.random.default_rng(0).normal(size=2000).astype(np.float32) * 10,
                         np.array([0.0, 1.0, -1.0, 65504.0, 1e-7, 3.1415927], dtype=np.float32)])
    t = torch.from_numpy(xs)
    bf = t.to(torch.bfloat16).to(torch.float32).numpy()
    hf = t.to(torch.float16).to(torch.float32).numpy()
    for x, eb, eh in zip(xs, bf, hf):
        assert native_lib.yali_c_round_bf16(float(x)) == eb
        assert native_lib.yali_c_round_fp16(float(x)) == eh


def test_oracles(native_lib):
    rng = np.random.default_rng(1)
    world, n = 4, 1000
    ins = [rng.normal(size=n).astype(np.float32) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[x.ctypes.data for x in ins])
    out = np.zeros(n, dtype=np.float64)
    native_lib.yali_c_oracle_allreduce(ptrs, world, n, 0.25, out.ctypes.data)
    np.testing.assert_allclose(out, 0.25 * np.sum(np.stack(ins).astype(np.float64), axis=0), rtol=1e-12)

    rows, hidden = 5, 64
    s = rng.normal(size=(rows, hidden))
    res = rng.normal(size=(rows, hidden)).astype(np.float32)
    w = rng.normal(size=hidden).astype(np.float32)
    y = np.zeros((rows, hidden))
    pre = np.zeros((rows, hidden))
    native_lib.yali_c_oracle_residual_rmsnorm(s.ctypes.data, res.ctypes.data, w.ctypes.data, rows, hidden, 1e-5,
                                              y.ctypes.data, pre.ctypes.data)
    exp_pre = s + res
    exp = exp_pre / np.sqrt((exp_pre ** 2).mean(axis=1, keepdims=True) + 1e-5) * w
    np.testing.assert_allclose(pre, exp_pre, rtol=1e-12)
    np.testing.assert_allclose(y, exp, rtol=1e-10)

    a = rng.normal(size=(3, 8)).astype(np.float32)
    b = rng.normal(size=(8, 5)).astype(np.float32)
    c = np.zeros((3, 5))
    native_lib.yali_c_oracle_gemm(a.ctypes.data, b.ctypes.data, 3, 5, 8, c.ctypes.data)
    np.testing.assert_allclose(c, a.astype(np.float64) @ b.astype(np.float64), rtol=1e-12)


def test_verify_allreduce_sum(native_lib):
    first, count = ctypes.c_size_t(), ctypes.c_size_t()
    good = np.full(100, 3.0, dtype=np.float32)
    assert native_lib.yali_c_verify_allreduce_sum(good.ctypes.data, 100, 3.0, 1e-3, ctypes.byref(first),
                                                  ctypes.byref(count)) == 1 and count.value == 0
    bad = good.copy()
    bad[17] = 2.0
    bad[50] = float("nan")
    assert native_lib.yali_c_verify_allreduce_sum(bad.ctypes.data, 100, 3.0, 1e-3, ctypes.byref(first),
                                                  ctypes.byref(count)) == 0
    assert first.value == 17 and count.value == 2
    near = np.full(10, 3.0005, dtype=np.float32)
    assert native_lib.yali_c_verify_allreduce_sum(near.ctypes.data, 10, 3.0, 1e-3, None, None) == 1
    assert native_lib.yali_c_verify_allreduce_sum(near.ctypes.data, 10, 3.0, 1e-4, None, None) == 0
    assert native_lib.yali_c_verify_allreduce_sum(None, 0, 3.0, 1e-4, None, None) == 1


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_fused_linear_counter_targets_match_the_kernels_announcements(native_lib, world):
    """The host's counter targets must equal what the kernel's announcer warp and row owners add up to:
    a mismatch would end in a bounded-wait timeout on the device."""
    import ctypes
    lib = native_lib
    BM, BN = 128, 256
    for T, N in [(t, 4096) for t in [1, 2, 7, 16, 100, 127, 128, 129, 255, 256, 300, 1000, 1024, 2047, 2048, 4099]] + \
            [(300, 128), (300, 384), (64, 2048)]:
        for oneshot in (0, 1):
            arr = (ctypes.c_uint32 * 8)()
            rows = (ctypes.c_uint32 * 8)()
            lib.yali_c_fused_linear_counts(T, N, world, oneshot, arr, rows)
            ntm, ntn = -(-T // BM), -(-N // BN)
            rs = T if oneshot else -(-T // world)
            want = [0] * world
            for mt in range(ntm):  # the announcer's rule, tile by tile (one source)
                lo, hi = mt * BM, min(T, mt * BM + BM)
                for _nt in range(ntn):
                    for q in range(world):
                        if oneshot or (q * rs < hi and (q + 1) * rs > lo):
                            want[q] += 1
            assert list(arr[:world]) == want, (T, oneshot)
            own = [0 if oneshot else max(0, min(T, q * rs + rs) - min(T, q * rs)) for q in range(world)]
            assert list(rows[:world]) == own and (oneshot or sum(own) == T)
    assert lib.yali_c_fused_linear_oneshot_max_rows(2) >= lib.yali_c_fused_linear_oneshot_max_rows(8) >= 1
    assert lib.yali_c_fused_linear_multicast_mode(2, 2048) == 0
    assert lib.yali_c_fused_linear_multicast_mode(8, 128) in (1, 2) and lib.yali_c_fused_linear_multicast_mode(8, 2048) in (1, 2)
