"""Runs the C++ / CUDA test binaries, examples and a benchmark self-check (built by `make
cpptests examples bench` into build/bin) so that the C++ API is exercised by the same
pytest run as everything else.  Reference counterparts: the Bazel `unit_tests`,
`correctness_tests`, `example_tests` and `mpi_tests` suites."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "build" / "bin"


def _need(name):
    exe = BIN / name
    if not exe.exists():
        r = subprocess.run(["make", "-C", str(ROOT), f"build/bin/{name}"], capture_output=True, text=True)
        if r.returncode != 0 or not exe.exists():
            pytest.fail(f"{name} is not built and `make` failed:\n{r.stdout[-800:]}{r.stderr[-800:]}")
    return str(exe)


def _run(cmd, env=None, timeout=600):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=str(ROOT))
    assert r.returncode == 0, f"{' '.join(map(str, cmd))}\n{r.stdout[-2000:]}\n{r.stderr[-2000:]}"
    return r.stdout


def test_unit_binary():
    out = _run([_need("test_unit")])
    assert "0 failed" in out


def test_ops_binary():
    out = _run([_need("test_ops_allreduce")])
    assert "0 failed" in out


def test_benchmark_self_check_emulated():
    exe = _need("benchmark_yali")
    for mode, elems, dtype in [("flash", 262144, "fp32"), ("stream", 1 << 22, "bf16"), ("auto", 1000003, "fp16")]:
        out = _run([exe, str(elems), "20", "1", mode, "0", "cuda-events", dtype, "4"],
                   env={"YALI_EMULATE": "1", "YALI_WARMUP": "5"})
        assert "Correctness: PASSED" in out and "GB/s" in out and '"p99_us"' in out


@pytest.mark.parametrize("nranks", [2, 3])
def test_multi_process_c_abi(nranks):
    """yaliMPComm* / yaliIpc* end to end, one process per rank.  The ranks meet at host barriers only,
    so they may share a GPU (rank r uses GPU r modulo the number of GPUs)."""
    out = _run([sys.executable, "-m", "yali_b200.launch", "-np", str(nranks), _need("test_mp_cabi")])
    assert f"C ABI test on {nranks} ranks: PASSED" in out


@pytest.mark.multigpu(2)
def test_examples_and_mpi_binaries():
    assert "3.0, 3.0" in _run([_need("example_simple")])
    assert "PASSED" in _run([_need("example_multilane")], env={"YALI_ELEMS": str(1 << 20)})
    launch = [sys.executable, "-m", "yali_b200.launch", "-np", "2"]
    assert "expected 3.0" in _run(launch + [_need("example_simple_mpi")])
    assert "PASSED" in _run(launch + [_need("example_multilane_mpi")], env={"YALI_ELEMS": str(1 << 20)})
    assert "PASSED" in _run(launch + [_need("example_manual_ipc")], env={"YALI_ELEMS": str(1 << 20)})
    assert "PASSED" in _run(launch + [_need("test_ops_allreduce_mpi")])
    out = _run(launch + [_need("benchmark_yali_mpi"), "524288", "50", "1", "auto", "0", "cuda-events", "bf16"],
               env={"YALI_WARMUP": "5"})
    assert "Correctness: PASSED" in out
    out = _run([_need("benchmark_yali"), "262144", "50", "1", "auto", "0", "cuda-events", "fp32", "2"],
               env={"YALI_WARMUP": "5"})
    assert "Correctness: PASSED" in out
