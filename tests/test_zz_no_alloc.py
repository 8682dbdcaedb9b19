"""The allocation-free all-reduce entry point (`yaliAllReduceLocalNoAlloc`), called through
its exported C symbol the way a program that cannot allocate device memory would call it:
the caller passes only its own input and output buffers, the library works in its built-in
scratch array.  Results of two calls in a row are compared with the library's ordinary
entry point (a communicator's one-shot all-reduce) on the same inputs.  This file is
collected last so that a run that stops at the first failure has already run every other
test; it also passes on its own in a fresh process."""
import ctypes

import pytest
import torch

import yali_b200 as yali
from yali_b200 import _native

pytestmark = pytest.mark.gpu

MAX_BYTES = 256 * 1024


def _entry():
    lib = _native.lib()
    fn = lib.yaliAllReduceLocalNoAlloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_size_t,
                   ctypes.c_int, ctypes.c_void_p]
    lib.yaliNoAllocLastError.restype = ctypes.c_char_p
    return lib, fn


def _call(fn, sends, recvs, dtype_code):
    world = len(sends)
    s = (ctypes.c_void_p * world)(*[t.data_ptr() for t in sends])
    r = (ctypes.c_void_p * world)(*[t.data_ptr() for t in recvs])
    stream = torch.cuda.current_stream().cuda_stream
    return fn(s, r, world, sends[0].numel(), dtype_code, ctypes.c_void_p(stream))


@pytest.mark.parametrize("world", [2, 3, 4])
@pytest.mark.parametrize("dtype,code,n", [(torch.float32, 0, 65536), (torch.bfloat16, 2, 100003),
                                          (torch.float16, 1, 7)])
def test_matches_the_communicator_entry_point_twice(world, dtype, code, n):
    torch.cuda.set_device(0)
    lib, fn = _entry()
    ext = _native.ext()
    with yali.Comm.emulated(world, device=0) as comm:
        for call in range(2):  # two calls in a row share the scratch array
            sends = []
            for r in range(world):
                t = torch.empty(n, dtype=dtype, device="cuda:0")
                ext.fill_random(t, 1, 500 + 10 * call + r)
                sends.append(t)
            recvs = [torch.full((n,), float("nan"), dtype=dtype, device="cuda:0") for _ in range(world)]
            rc = _call(fn, sends, recvs, code)
            assert rc == 0, lib.yaliNoAllocLastError().decode()
            expect = comm.all_reduce(sends, mode="flash")
            comm.sync()
            torch.cuda.synchronize()
            tol = dict(rtol=0, atol=0) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2 * world)
            for got, want in zip(recvs, expect):
                torch.testing.assert_close(got.float(), want.float(), **tol)
            rep = ext.validate_sum(recvs[0], dtype, 1, 500 + 10 * call, world)
            assert rep["mismatches"] == 0, rep


@pytest.mark.parametrize("world", [2, 3])
def test_one_rank_with_unaligned_buffers(world):
    """Rank 1's buffers start one element off a 16-byte boundary, the others' do not: the ranks must still agree on
    how the message is cut (a rank that cannot use vector accesses only changes how it touches its own slice)."""
    torch.cuda.set_device(0)
    lib, fn = _entry()
    ext = _native.ext()
    for dtype, code, n in ((torch.float32, 0, 40001), (torch.bfloat16, 2, 9999)):
        for call in range(2):
            sends, recvs = [], []
            for r in range(world):
                off = 1 if r == 1 else 0
                base = torch.empty(n + 8, dtype=dtype, device="cuda:0")
                tmp = torch.empty(n, dtype=dtype, device="cuda:0")
                ext.fill_random(tmp, 1, 700 + 10 * call + r)
                base[off:off + n].copy_(tmp)
                sends.append(base[off:off + n])
                recvs.append(torch.full((n + 8,), float("nan"), dtype=dtype, device="cuda:0")[off:off + n])
            assert sends[1].data_ptr() % 16 != 0 and sends[0].data_ptr() % 16 == 0
            assert _call(fn, sends, recvs, code) == 0, lib.yaliNoAllocLastError().decode()
            torch.cuda.synchronize()
            for got in recvs:
                assert ext.validate_sum(got.clone(), dtype, 1, 700 + 10 * call, world)["mismatches"] == 0
            assert all(torch.equal(recvs[0], g) for g in recvs[1:])


def test_in_place_and_refusals():
    torch.cuda.set_device(0)
    lib, fn = _entry()
    ext = _native.ext()
    n = 4096
    xs = []
    for r in range(2):
        t = torch.empty(n, dtype=torch.float32, device="cuda:0")
        ext.fill_random(t, 0, 900 + r)
        xs.append(t)
    assert _call(fn, xs, xs, 0) == 0  # recv == send
    torch.cuda.synchronize()
    assert ext.validate_sum(xs[0], torch.float32, 0, 900, 2)["mismatches"] == 0
    assert torch.equal(xs[0], xs[1])
    big = [torch.empty(MAX_BYTES // 4 + 1, dtype=torch.float32, device="cuda:0") for _ in range(2)]
    assert _call(fn, big, big, 0) != 0 and b"larger than" in lib.yaliNoAllocLastError()
    # A count whose byte size would wrap around 64 bits is refused like any other oversized message.
    s = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in xs])
    assert fn(s, s, 2, ctypes.c_size_t(1 << 62), 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) != 0
    assert b"larger than" in lib.yaliNoAllocLastError()
    five = [torch.empty(8, dtype=torch.float32, device="cuda:0") for _ in range(5)]
    assert _call(fn, five, five, 0) != 0 and b"world" in lib.yaliNoAllocLastError()
    assert _call(fn, xs, xs, 7) != 0 and b"dtype" in lib.yaliNoAllocLastError()
    assert _call(fn, xs, xs, 0) == 0  # still usable after refusals
    torch.cuda.synchronize()
