"""Tooling without a GPU: statistics, report generation from sweep lines, nccl-tests log parsing, NVLink status
parsing, the launcher, and the baseline validator's version check."""
import json
import subprocess
import sys
from pathlib import Path

from yali_b200.utils import hw_info
from yali_b200.utils.stats import percentile, summarise

ROOT = Path(__file__).resolve().parent.parent


def test_stats():
    s = summarise([1.0, 2.0, 3.0, 4.0])
    assert s.mean == 2.5 and s.min == 1.0 and s.max == 4.0 and s.samples == 4
    assert abs(s.stddev - 1.2909944) < 1e-6 and abs(s.cv_pct - 51.6397779) < 1e-5
    assert s.p50 == 2.5 and percentile([1, 2, 3, 4], 100) == 4 and percentile([], 50) == 0.0
    assert summarise([]).samples == 0 and summarise([7.0]).stddev == 0.0


def test_report_from_sweep_lines(tmp_path):
    rows = []
    for size, y, n in [(4096, 0.5, 0.2), (1 << 20, 90.0, 56.0), (1 << 30, 670.0, 566.0)]:
        for var in ("auto", "flash"):
            rows.append({"impl": "yali_b200", "world": 2, "dtype": "fp32", "bytes": size, "variant": var,
                         "kernel": "flash", "ctas": 8, "slot_bytes": 0, "us": size / y / 1e3, "busbw_gbps": y,
                         "dev_p50_us": 10.0, "dev_p99_us": 10.5, "dev_max_us": 12.0, "dev_samples": 200})
        rows.append({"impl": "nccl", "world": 2, "dtype": "fp32", "bytes": size, "variant": "nccl", "us": size / n / 1e3,
                     "busbw_gbps": n})
    run = tmp_path / "run.jsonl"
    run.write_text("\n".join(json.dumps(r) for r in rows) + "\nnoise line\n")
    out = tmp_path / "rep"
    subprocess.run([sys.executable, str(ROOT / "bench" / "report.py"), "--out", str(out), str(run), str(run)], check=True)
    summary = (out / "summary.md").read_text()
    assert "| 1M | 90.0 | 90.0 | - | - | - | 56.0 | 1.61x | 12 % | 1.05 |" in summary and "## 2 ranks, fp32" in summary
    csv_text = (out / "yali_b200_w2_fp32.csv").read_text()
    assert "mean_gbps" in csv_text and ",2\n" in csv_text  # two runs per point
    # charts: bandwidth, latency, speed-up over NCCL, speed of light, run-to-run variation, device-timed tail
    for name in ("bandwidth", "latency", "speedup", "sol", "variation", "tail"):
        svg = (out / f"{name}_w2_fp32.svg").read_text()
        assert svg.startswith("<svg") and "polyline" in svg and svg.rstrip().endswith("</svg>")
    assert "![bandwidth_w2_fp32.svg]" in summary
    # the per-kernel device-time summary and the index of a campaign directory
    sys.path.insert(0, str(ROOT / "bench"))
    import run_sweep
    run_sweep.write_profiler_summary([str(run)], out)
    prof = json.loads((out / "profiler_summary.json").read_text())
    assert prof["kernels"]["flash"][f"fp32:{1 << 20}"] == {"calls": 400, "p50_us": 10.0, "p99_us": 10.5, "max_us": 12.0}

    class A:
        gpus, mode = 2, "quick"
    run_sweep.write_index(out, A, run_sweep.MODES["quick"])
    index = (out / "index.md").read_text()
    assert "[summary.md](summary.md)" in index and "profiler_summary.json" in index and ".svg" in index


def test_consolidate_eval(tmp_path):
    log = """#       size         count      type   redop    root     time   algbw   busbw #wrong     time   algbw   busbw #wrong
     1048576        262144     float     sum      -1    18.70   56.07   56.07      0    18.50   56.68   56.68      0
  1073741824     268435456     float     sum      -1   1897.1  566.00  566.00      0   1890.0  568.12  568.12      0
"""
    (tmp_path / "nccl.log").write_text(log)
    sweep = [{"impl": "yali_b200", "world": 2, "dtype": "fp32", "bytes": 1 << 20, "variant": "auto", "us": 11.9,
              "busbw_gbps": 88.1},
             {"impl": "yali_b200", "world": 2, "dtype": "fp32", "bytes": 1 << 30, "variant": "auto", "us": 1595.0,
              "busbw_gbps": 673.2}]
    (tmp_path / "s.jsonl").write_text("\n".join(json.dumps(r) for r in sweep))
    r = subprocess.run([sys.executable, str(ROOT / "bench" / "consolidate_eval.py"), "--sweep", str(tmp_path / "s.jsonl"),
                        "--nccl-log", str(tmp_path / "nccl.log"), "--out", str(tmp_path / "eval")], capture_output=True,
                       text=True, check=True)
    assert "2 sizes joined" in r.stdout and "none" in r.stdout
    assert "1.571x" in (tmp_path / "eval" / "ratio.md").read_text()


def test_nvlink_parsing_and_capability_table():
    text = "GPU 0: NVIDIA B200 (UUID: x)\n\t Link 0: 53.125 GB/s\n\t Link 1: 53.125 GB/s\nGPU 1: NVIDIA B200\n\t Link 0: 53.125 GB/s\n"
    st = hw_info.parse_nvlink_status(text)
    assert st[0]["links"] == 2 and st[1]["links"] == 1 and st[0]["gbs_per_link"] == 53.125
    b200 = hw_info.nvlink_for_capability(10)
    assert b200["links"] == 18 and b200["unidirectional_gbs"] == 900.0
    assert hw_info.measured_peaks()["source"] in ("measured", "fallback")


def test_launcher_sets_rank_environment(tmp_path):
    script = tmp_path / "p.py"
    # One write() per child: the three children share a pipe, and a line written in one system call
    # (shorter than PIPE_BUF) cannot interleave with the others.
    script.write_text("import os,sys\n"
                      "os.write(1, ('%s %s %s\\n' % (os.environ['RANK'], os.environ['WORLD_SIZE'], "
                      "os.environ['LOCAL_RANK'])).encode())\n"
                      "sys.exit(3 if os.environ['RANK']=='1' and os.environ.get('FAIL') else 0)\n")
    r = subprocess.run([sys.executable, "-m", "yali_b200.launch", "-np", "3", sys.executable, str(script)],
                       capture_output=True, text=True, cwd=str(ROOT))
    assert r.returncode == 0 and sorted(ln for ln in r.stdout.split("\n") if ln) == ["0 3 0", "1 3 1", "2 3 2"]
    r = subprocess.run([sys.executable, "-m", "yali_b200.launch", "-np", "2", sys.executable, str(script)],
                       capture_output=True, text=True, cwd=str(ROOT), env={**__import__("os").environ, "FAIL": "1"})
    assert r.returncode == 3


def test_nccl_header_matches_library():
    sys.path.insert(0, str(ROOT / "bench"))
    import validate_baselines as vb
    assert vb.header_version() == vb.library_version()


def test_baseline_validators_judge_their_inputs():
    """The checks behind `validate_baselines.py --run` (peer-copy floors, NCCL sweep sanity) on canned output."""
    sys.path.insert(0, str(ROOT / "bench"))
    import validate_baselines as vb
    good = {"copy_engine_unidirectional_gbs": 779.0, "copy_engine_bidirectional_per_direction_gbs": 774.0,
            "sm_remote_store_gbs": 714.0, "sm_remote_load_gbs": 772.0, "bulk_pull_gbs": 781.0, "bulk_push_gbs": 714.0}
    assert vb.check_p2p(good, 500.0) == []
    assert any("sm_remote_load_gbs" in m for m in vb.check_p2p({**good, "sm_remote_load_gbs": 90.0}, 500.0))
    assert vb.check_p2p({"unavailable": "needs two distinct GPUs"}, 500.0) == ["needs two distinct GPUs"]
    rows = [{"dtype": "fp32", "bytes": 4096 << i, "us": 8.0 + (4096 << i) / 450e3, "busbw_gbps": (4096 << i) / (8.0 + (4096 << i) / 450e3) / 1e3}
            for i in range(17)]  # 4 KiB .. 256 MiB
    assert vb.check_nccl_sweep(rows, 300.0) == []
    assert vb.check_nccl_sweep(rows[:5] + rows[6:], 300.0)  # a size is missing
    assert vb.check_nccl_sweep([{**r, "busbw_gbps": 100.0} if r is rows[-1] else r for r in rows], 300.0)  # too slow
    assert vb.check_nccl_sweep([], 300.0) == ["no rows"]


def test_make_tuning_table_from_sweep_lines(tmp_path):
    """bench/make_tuning_table.py: fastest forced variant per size, hysteresis against noise, merged rows; the
    planner loads the result (the committed table of the B200 runs included)."""
    import ctypes
    import importlib.util
    import json as _json
    from pathlib import Path as _Path

    from yali_b200 import _native
    root = _Path(__file__).resolve().parents[1]
    spec = importlib.util.spec_from_file_location("make_tuning_table", root / "bench" / "make_tuning_table.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    def line(size, kernel, us, world=2):
        return {"impl": "yali_b200", "world": world, "dtype": "fp32", "bytes": size, "variant": kernel[:5],
                "kernel": kernel, "us": us, "busbw_gbps": size / us / 1e3}
    rows = [line(4096, "flash", 4.0), line(4096, "stream", 10.0),
            line(8192, "flash", 5.0), line(8192, "stream", 4.95),      # 1 % better: the incumbent stays
            line(16384, "flash", 9.0), line(16384, "stream", 6.0),     # a real crossover
            line(32768, "stream", 7.0), line(32768, "flash", 12.0),
            {"impl": "nccl", "world": 2, "dtype": "fp32", "bytes": 4096, "variant": "nccl", "us": 1.0, "busbw_gbps": 1.0},
            dict(line(4096, "stream", 0.1), variant="auto")]           # auto rows never vote
    table = mod.build(rows)
    assert [(r["max_bytes"], r["variant"]) for r in table] == [(8192, "flash"), (1 << 40, "stream")]

    committed = root / "docs" / "benchmark" / "artifacts" / "2026-11-25-b200" / "tuning_b200_nvswitch.json"
    text = committed.read_text()
    assert len(_json.loads(text)["rows"]) >= 6
    # The planner follows the committed table: 64 MiB fp32 at 2 ranks is the ring kernel there.
    lib = _native.lib()
    from tests.test_core_cpu import Plan, caps  # the ctypes mirrors of the C structs
    plan, err = Plan(), ctypes.create_string_buffer(256)
    c = caps(2)
    rc = lib.yali_c_make_plan(2, (64 << 20) // 4, 0, 0, 0, 0, ctypes.byref(c), text.encode(), ctypes.byref(plan), err, 256)
    assert rc == 0 and plan.variant == 1, err.value
    rc = lib.yali_c_make_plan(2, (1 << 20) // 4, 0, 0, 0, 0, ctypes.byref(c), text.encode(), ctypes.byref(plan), err, 256)
    assert rc == 0 and plan.variant == 0


def test_fused_layer_output_buffer_is_cached_per_shape():
    """With one GPU per process the fused layer's default output comes from the symmetric heap, which is
    never freed piecemeal: one buffer per row width, grown by doubling, handed out again, forgotten by symm_reset()."""
    import torch

    from yali_b200.parallel.comm import Comm

    class FakeImpl:
        world, nlocal = 4, 1

        def __init__(self):
            self.allocs, self.calls, self.resets = 0, [], 0

        def symm_empty(self, shape, dtype):
            self.allocs += 1
            return [torch.empty(shape, dtype=dtype)]

        def fused_linear(self, xs, ws, nws, outs, res, ro, eps, oneshot, ctas, tr, nvls, decode):
            self.calls.append((outs[0], oneshot, nvls))

        def symm_reset(self):
            self.resets += 1

        def close(self):
            pass

    impl = FakeImpl()
    comm = Comm(impl)
    x, w, g = torch.zeros(6, 8, dtype=torch.bfloat16), torch.zeros(16, 8, dtype=torch.bfloat16), torch.ones(16)
    y1 = comm.fused_linear_rmsnorm(x, w, g)
    y2 = comm.fused_linear_rmsnorm(x, w, g, nvls=2)
    assert y1.data_ptr() == y2.data_ptr() and impl.allocs == 1 and tuple(y1.shape) == (6, 16)
    assert impl.calls[0][1:] == (-1, -1) and impl.calls[1][2] == 2
    y3 = comm.fused_linear_rmsnorm(torch.zeros(3, 8, dtype=torch.bfloat16), w, g)  # fewer rows: the same buffer
    assert y3.data_ptr() == y1.data_ptr() and tuple(y3.shape) == (3, 16) and impl.allocs == 1
    y5 = comm.fused_linear_rmsnorm(torch.zeros(7, 8, dtype=torch.bfloat16), w, g)  # more rows: grown by doubling
    assert tuple(y5.shape) == (7, 16) and impl.allocs == 2
    for rows in (8, 9, 12, 5, 11):  # up to 12 rows fit the doubled buffer: no further allocation
        assert tuple(comm.fused_linear_rmsnorm(torch.zeros(rows, 8, dtype=torch.bfloat16), w, g).shape) == (rows, 16)
    assert impl.allocs == 2
    mine = torch.empty(6, 16, dtype=torch.bfloat16)
    assert comm.fused_linear_rmsnorm(x, w, g, out=mine) is mine and impl.allocs == 2
    comm.symm_reset()
    assert impl.resets == 1
    y4 = comm.fused_linear_rmsnorm(x, w, g)
    assert impl.allocs == 3 and tuple(y4.shape) == (6, 16)
    comm.close()
