"""The cross-rank flag protocols of the one-shot and the two-shot ring kernel, run
by host threads on host memory (one thread per CTA): correctness of back-to-back
calls without any barrier, slot reuse (a producer that overwrites a slot before its
consumer is done is reported as an invariant violation), and fault injection on the
host: a rank that never launches must make its peers time out, not hang."""
import ctypes

import pytest

from yali_b200 import _native
from yali_b200._native import SimConfig, SimReport


def simulate(**kw):
    cfg = SimConfig(mode=1, world=2, lanes=2, calls=2, count=10000, slot_elems=64, direct_ag=0, fault=0, fault_rank=0,
                    fault_call=0, timeout_ms=5000, seed=1234)
    for k, v in kw.items():
        setattr(cfg, k, v)
    rep = SimReport()
    rc = _native.lib().yali_c_simulate(ctypes.byref(cfg), ctypes.byref(rep))
    return rc, rep


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("direct_ag", [0, 1])
def test_ring_protocol_many_iterations(world, direct_ag):
    # 50001 elements, 128-element slots, 3 lanes: dozens of iterations per lane, so every
    # slot of the 4-deep rings is reused many times and the credits matter.
    rc, rep = simulate(world=world, lanes=3, calls=3, count=50001, slot_elems=128, direct_ag=direct_ag)
    assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0
    assert rep.flag_writes > 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ring_protocol_tiny_and_ragged(world):
    for count, slot, lanes in [(1, 4, 1), (17, 4, 2), (4099, 16, 5), (1000, 1024, 4)]:
        rc, rep = simulate(world=world, lanes=lanes, calls=2, count=count, slot_elems=slot)
        assert rc == 0, (count, slot, lanes, rep.status, rep.mismatches)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_one_shot_protocol_back_to_back(world):
    rc, rep = simulate(mode=0, world=world, lanes=4, calls=6, count=4099)
    assert rc == 0 and rep.mismatches == 0


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("mode", [4, 5])
def test_pipelined_direct_protocols_back_to_back(world, mode):
    """Two-shot in place (4) and one-shot pull (5): the two per-CTA barriers of a call must keep every rank from
    rewriting its input (which all ranks read in place) or reading its output too early, over back-to-back calls
    with fresh inputs per call and chunks that interleave over the CTAs."""
    for count, lanes, chunk in [(1, 1, 4), (4099, 3, 64), (50001, 5, 128)]:
        rc, rep = simulate(mode=mode, world=world, lanes=lanes, calls=5, count=count, slot_elems=chunk)
        assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0, (count, lanes, chunk, rc, rep.mismatches)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("mode", [6, 7])
def test_copy_engine_protocol_in_place_back_to_back(world, mode):
    """One-shot (6) and two-shot (7) copy-engine path in place: two threads per rank (the caller's stream and the
    stream of the incoming copies), three staging slots, fresh inputs per call.  The stamps catch a chunk that is
    overwritten before every peer has copied it, and an input rewritten before the peers are done with it."""
    for count, chunk in [(5, 4), (4099, 64), (50001, 1024), (20000, 256)]:
        rc, rep = simulate(mode=mode, world=world, lanes=2, calls=5, count=count, slot_elems=chunk)
        assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0, (count, chunk, rc, rep.mismatches, rep.timeout_site)
        assert rep.flag_writes > 0


def test_copy_engine_model_catches_a_missing_handshake():
    # Negative control: without the wait before overwriting (and with a peer that copies slowly) a rank writes
    # its sums over a chunk that the peer has not copied yet.
    hits = 0
    for _ in range(3):
        rc, rep = simulate(mode=6, world=2, lanes=2, calls=3, count=20000, slot_elems=256, direct_ag=1)
        hits += rc == 3
    assert hits >= 1


def test_copy_engine_failures_time_out():
    rc, rep = simulate(mode=6, world=2, lanes=2, fault=1, fault_rank=1, fault_call=1, calls=3, count=5000, timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == 1 and rep.timeout_rank == 0
    rc, rep = simulate(mode=7, world=4, lanes=2, fault=1, fault_rank=3, fault_call=1, calls=3, count=5000, timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == 3 and rep.timeout_rank != 3
    rc, rep = simulate(mode=7, world=2, lanes=2, fault=2, fault_rank=0, fault_call=1, calls=3, count=5000, timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == 0  # the lost "entered" keeps rank 1 from copying
    rc, _ = simulate(mode=6, world=2, lanes=3)  # two threads per rank, no other number
    assert rc == -1


def test_rank_that_never_launches_times_out_pipelined():
    rc, rep = simulate(mode=4, world=4, lanes=2, fault=1, fault_rank=3, fault_call=1, calls=3, count=5000, timeout_ms=300)
    assert rc == 2 and rep.timeouts >= 1 and rep.timeout_peer == 3 and rep.timeout_rank != 3


def test_rank_that_never_launches_times_out_ring():
    rc, rep = simulate(world=4, fault=1, fault_rank=2, fault_call=1, calls=3, timeout_ms=300)
    assert rc == 2 and rep.timeouts >= 1 and rep.timeout_peer == 2 and rep.timeout_rank != 2
    assert rep.timeout_site in (2, 3, 4, 5)


def test_rank_that_never_launches_times_out_one_shot():
    rc, rep = simulate(mode=0, world=2, fault=1, fault_rank=0, fault_call=0, calls=1, timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == 0 and rep.timeout_site == 1


def test_dropped_flag_write_is_survived_or_times_out():
    # Counters are monotone: a lost publication is healed by the next one of the same lane;
    # when it was the last one the waiter times out.  Never a wrong result.
    for world in (2, 4):
        rc, rep = simulate(world=world, lanes=2, calls=2, count=20000, slot_elems=64, fault=2, fault_rank=1,
                           fault_call=0, timeout_ms=300)
        assert rc in (0, 2) and (rc != 0 or rep.mismatches == 0)


def test_bad_configs_are_rejected():
    assert simulate(world=1)[0] == -1
    assert simulate(world=9)[0] == -1
    assert simulate(slot_elems=6)[0] == -1
    assert simulate(count=0)[0] == -1


# ---- fused GEMM layer: pushes into landing zones, arrival / delivered-row counters, call parities ----
from yali_b200._native import FusedSimConfig  # noqa: E402


def simulate_fused(**kw):
    cfg = FusedSimConfig(world=2, ctas=3, calls=4, oneshot=0, rows=300, col_tiles=2, fault=0, fault_rank=0,
                         fault_call=0, slow_rank=-1, single_parity=0, timeout_ms=5000, in_switch=0, ksplit=0)
    for k, v in kw.items():
        setattr(cfg, k, v)
    rep = SimReport()
    rc = _native.lib().yali_c_simulate_fused(ctypes.byref(cfg), ctypes.byref(rep))
    return rc, rep


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("oneshot", [0, 1])
def test_fused_layer_protocol_back_to_back_calls(world, oneshot):
    # ragged row counts (owners without rows, tiles that span two owners), more tiles than CTAs
    for rows in (1, 7, 129, 300, 1000):
        rc, rep = simulate_fused(world=world, oneshot=oneshot, rows=rows, calls=5)
        assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0, (rows, rc, rep.mismatches, rep.timeout_site)
        assert rep.flag_writes > 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_layer_in_switch_form(world):
    # partial rows stay in the producer's image; an owner reads every rank's image (multimem.ld_reduce)
    for rows, slow in ((7, -1), (300, -1), (1000, 1), (260, 0)):
        rc, rep = simulate_fused(world=world, rows=rows, calls=6, in_switch=1, slow_rank=slow)
        assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0, (rows, rc, rep.mismatches)


@pytest.mark.parametrize("oneshot", [0, 1])
def test_fused_layer_protocol_with_a_slow_rank(oneshot):
    # The other ranks run ahead into the next calls: the two landing parities and the stream order
    # of output consumption must keep every cell intact.
    rc, rep = simulate_fused(world=4, oneshot=oneshot, rows=260, calls=8, slow_rank=2, ctas=2)
    assert rc == 0 and rep.mismatches == 0, (rc, rep.mismatches)


def test_fused_layer_model_catches_a_missing_parity():
    # Negative control: with one landing buffer instead of two, a fast rank's pushes of call n+1
    # land on cells that the slow rank has not reduced yet (one-shot: nothing makes the fast rank wait).
    hits = 0
    for _ in range(3):
        rc, rep = simulate_fused(world=2, oneshot=1, rows=64, calls=8, slow_rank=1, single_parity=1, ctas=2)
        hits += rc == 3
    assert hits >= 1


def test_fused_layer_rank_that_stops_launching_times_out_its_peers():
    rc, rep = simulate_fused(world=4, rows=300, calls=4, fault=1, fault_rank=3, fault_call=2, timeout_ms=300)
    assert rc == 2 and rep.timeouts >= 1 and rep.timeout_peer == 3 and rep.timeout_site in (1, 2)


def test_fused_layer_lost_announcement_times_out():
    rc, rep = simulate_fused(world=2, rows=300, calls=3, fault=2, fault_rank=0, fault_call=1, timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == 0 and rep.timeout_site == 1


# ---- few-token form of the fused layer: flag-in-data lines from world x ksplit sources, no counters ----
@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("ksplit", [1, 2, 4])
def test_few_token_form_protocol_back_to_back_calls(world, ksplit):
    for rows, tiles in ((1, 16), (16, 8), (64, 4)):
        rc, rep = simulate_fused(world=world, rows=rows, col_tiles=tiles, ksplit=ksplit, calls=6, ctas=4)
        assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0, (rows, rc, rep.mismatches, rep.timeout_site)
        assert rep.flag_writes == 6 * world * world * ksplit * rows * tiles  # every line to every rank, once per call


def test_few_token_form_with_a_slow_rank_needs_both_parities():
    # The fast ranks run ahead into the next call: their lines go to the other parity and wait there.
    rc, rep = simulate_fused(world=4, rows=16, col_tiles=8, ksplit=2, calls=10, slow_rank=2, ctas=3)
    assert rc == 0 and rep.mismatches == 0
    # Negative control: with one landing zone per source the next call's lines overwrite unread ones.
    hits = 0
    for _ in range(3):
        rc, rep = simulate_fused(world=2, rows=64, col_tiles=8, ksplit=4, calls=10, slow_rank=1, single_parity=1, ctas=2)
        hits += rc in (2, 3)
    assert hits >= 1


def test_few_token_form_failures_time_out():
    rc, rep = simulate_fused(world=4, rows=8, col_tiles=8, ksplit=2, calls=4, fault=1, fault_rank=3, fault_call=2,
                             timeout_ms=300)
    assert rc == 2 and rep.timeouts >= 1 and rep.timeout_peer == 3
    rc, rep = simulate_fused(world=2, rows=8, col_tiles=8, ksplit=2, calls=3, fault=2, fault_rank=0, fault_call=1,
                             timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == 0
    rc, _ = simulate_fused(world=2, rows=65, col_tiles=8, ksplit=2)  # more rows than the form takes
    assert rc == -1


# ---- flag-in-data form of the one-shot (mode 2): the call number travels inside every pushed word ----
@pytest.mark.parametrize("world", [2, 4, 8])
def test_flag_in_data_protocol_back_to_back(world):
    for count, ctas in [(1, 1), (17, 2), (4099, 3), (20000, 5)]:
        rc, rep = simulate(mode=2, world=world, lanes=ctas, calls=6, count=count)
        assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0, (count, ctas, rc, rep.mismatches)


def test_flag_in_data_lost_word_and_missing_rank_time_out():
    rc, rep = simulate(mode=2, world=2, lanes=2, calls=3, count=5000, fault=2, fault_rank=0, fault_call=1,
                       timeout_ms=300)
    assert rc == 2 and rep.timeout_rank == 1 and rep.timeout_peer == 0 and rep.timeout_site == 3
    rc, rep = simulate(mode=2, world=4, lanes=2, calls=4, count=5000, fault=1, fault_rank=2, fault_call=2,
                       timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == 2


# ---- staged two-shot through the switch (mode 3): per-CTA barriers, sums written back to every rank ----
@pytest.mark.parametrize("world", [2, 4, 8])
def test_in_switch_two_shot_protocol(world):
    for count, ctas in [(1, 1), (33, 2), (4099, 3), (20000, 4)]:
        rc, rep = simulate(mode=3, world=world, lanes=ctas, calls=5, count=count)
        assert rc == 0 and rep.mismatches == 0 and rep.timeouts == 0, (count, ctas, rc, rep.mismatches)
    rc, rep = simulate(mode=3, world=world, lanes=2, calls=4, count=3000, fault=1, fault_rank=world - 1, fault_call=1,
                       timeout_ms=300)
    assert rc == 2 and rep.timeout_peer == world - 1
