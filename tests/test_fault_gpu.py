"""Failure detection on the device without faulting it: one rank's kernel leaves at
once (as if that rank had never launched), so the flags its peers wait for are never
set.  Their waits must run out after the communicator's limit, the kernel must
return normally, the host must see a Timeout with the place of the wait, and after
reset() the communicator must work again."""
import pytest
import torch

import yali_b200 as yali
from yali_b200 import _native
from yali_b200.parallel.comm import YaliTimeout

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["flash", "stream"])
@pytest.mark.parametrize("world", [2, 4])
def test_wait_runs_out_then_reset_recovers(mode, world):
    ext = _native.ext()
    with yali.Comm.emulated(world, device=0, timeout_ms=150) as comm:
        xs = []
        for r in range(world):
            t = torch.empty(40000, dtype=torch.float32, device="cuda:0")
            ext.fill_random(t, 0, 1234 + r)
            xs.append(t)
        comm.all_reduce(xs, mode=mode)  # healthy call first
        comm.sync()
        comm.all_reduce(xs, mode=mode, _skip_rank=1)
        with pytest.raises(YaliTimeout) as info:
            comm.sync()
        assert "waiting for rank 1" in str(info.value)
        assert "waiting for rank 1" in comm.status()
        with pytest.raises(YaliTimeout):  # poisoned until reset
            comm.all_reduce(xs, mode=mode)
        comm.reset()
        assert comm.status() == ""
        outs = comm.all_reduce(xs, mode=mode)
        comm.sync()
        for o in outs:
            assert ext.validate_sum(o, torch.float32, 0, 1234, world)["mismatches"] == 0
        # the GPU context is intact
        assert torch.ones(4, device="cuda:0").sum().item() == 4.0
