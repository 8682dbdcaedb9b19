"""In-tree build of the native library and the torch extension.

`python -m yali_b200._build` compiles every CUDA translation unit for sm_100a
with nvcc (cross-compiles without a GPU), links `yali_b200/lib/libyali_b200.so`
(static CUDA runtime, driver API resolved at run time) and the torch binding
`yali_b200/_C.so`.  Objects are cached under `build/` keyed by a hash of the
source, its headers and the flags.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
LIBDIR = ROOT / "yali_b200" / "lib"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default", "-Xptxas", "-v"] + ARCH_FLAGS
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function"]

LIB_SOURCES = [
    "core/core.cc",
    "comm/bootstrap.cc",
    "comm/bootstrap_mpi.cc",
    "comm/cuda_driver.cc",
    "comm/topology.cc",
    "comm/symm_heap.cc",
    "comm/communicator.cc",
    "comm/mp_comm.cc",
    "comm/copy_engine_path.cc",
    "ops/tuning.cc",
    "ops/buffer_ops.cc",
    "ops/host_oracle.cc",
    "ops/yali_api.cc",
    "sim/protocol_sim.cc",
    "sim/gemm_protocol_sim.cc",
    "ops/fused_linear.cc",
    "ops/host_pipeline.cc",
    "capi/yali_c.cc",
    "kernels/flash_oneshot.cu",
    "kernels/stream_twoshot.cu",
    "kernels/nvls.cu",
    "kernels/direct_pipeline.cu",
    "kernels/copy_engine.cu",
    "kernels/util_kernels.cu",
    "kernels/gemm_ar_rmsnorm.cu",
    "kernels/gemm_ar_decode.cu",
    "kernels/no_alloc_entry.cu",
]


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh"):
            h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str], log: Path | None = None) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    out = proc.stdout + proc.stderr
    if log is not None:
        log.write_text(" ".join(cmd) + "\n" + out)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + out)
    return out


def _extra_flags() -> list[str]:
    # YALI_BUILD_NVTX=1: NVTX ranges around the host API calls (core/nvtx.h); off by default.
    return ["-DYALI_NVTX"] if os.environ.get("YALI_BUILD_NVTX") == "1" else []


def _compile(src: Path, flags: list[str], hdr_digest: str, verbose: bool) -> Path:
    key = hashlib.sha256((src.read_text() + hdr_digest + " ".join(flags)).encode()).hexdigest()[:16]
    obj = BUILD / (src.relative_to(CSRC).as_posix().replace("/", "_") + "." + key + ".o")
    if obj.exists():
        return obj
    for old in BUILD.glob(src.relative_to(CSRC).as_posix().replace("/", "_") + ".*.o*"):
        old.unlink()
    if src.suffix == ".cu":
        cmd = [NVCC] + NVCC_FLAGS + flags + ["-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        cmd = [NVCC, "-x", "cu"] + NVCC_FLAGS + flags + ["-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        print("  nvcc", src.relative_to(ROOT), flush=True)
    _run(cmd, BUILD / (obj.name + ".log"))
    return obj


def build_library(verbose: bool = True, sources: list[str] | None = None) -> Path:
    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    hdr = _headers_digest()
    srcs = [CSRC / s for s in (sources or LIB_SOURCES) if (CSRC / s).exists()]
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: _compile(s, _extra_flags(), hdr, verbose), srcs))
    lib = LIBDIR / "libyali_b200.so"
    stamp = hashlib.sha256(" ".join(sorted(o.name for o in objs)).encode()).hexdigest()
    stamp_file = BUILD / "lib.stamp"
    if lib.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return lib
    cmd = [NVCC, "-shared", "-cudart", "static"] + ARCH_FLAGS + ["-o", str(lib)] + [str(o) for o in objs] + \
          ["-lpthread", "-ldl", "-lrt"]
    if verbose:
        print("  link", lib.relative_to(ROOT), flush=True)
    _run(cmd)
    stamp_file.write_text(stamp)
    return lib


def build_torch_extension(verbose: bool = True) -> Path:
    import torch
    from torch.utils import cpp_extension

    BUILD.mkdir(exist_ok=True)
    lib = build_library(verbose)
    src = CSRC / "torch" / "bindings.cc"
    out = ROOT / "yali_b200" / "_C.so"
    incs = cpp_extension.include_paths()
    flags = ["-std=c++17", "-O2", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_C",
             "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))]
    key = hashlib.sha256((src.read_text() + _headers_digest() + torch.__version__ + " ".join(flags)).encode()).hexdigest()
    stamp_file = BUILD / "ext.stamp"
    if out.exists() and stamp_file.exists() and stamp_file.read_text() == key and out.stat().st_mtime >= lib.stat().st_mtime:
        return out
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++"] + flags + ["-I" + str(CSRC), "-I/usr/local/cuda/include", "-I" + sysconfig.get_paths()["include"]] + \
          ["-I" + i for i in incs] + [str(src), "-o", str(out),
                                      "-L" + str(LIBDIR), "-lyali_b200", "-Wl,-rpath,$ORIGIN/lib",
                                      "-L" + str(torch_lib), "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
                                      "-Wl,-rpath," + str(torch_lib)]
    if verbose:
        print("  g++ ", src.relative_to(ROOT), flush=True)
    _run(cmd)
    stamp_file.write_text(key)
    return out


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the cached nvcc logs."""
    lines = []
    for log in sorted(BUILD.glob("*.o.log")):
        text = log.read_text()
        fn = None
        for ln in text.splitlines():
            if "Compiling entry function" in ln:
                fn = ln.split("'")[1]
            elif "Used" in ln and "registers" in ln and fn:
                lines.append(f"{log.name.split('.')[0]} {fn}: {ln.split('ptxas info    : ')[-1]}")
            elif "spill" in ln and fn and "0 bytes spill stores, 0 bytes spill loads" not in ln:
                lines.append(f"{log.name.split('.')[0]} {fn}: {ln.strip()}")
    return "\n".join(lines)


def build_binaries(verbose: bool = True) -> None:
    """The C++ benchmarks, examples and tests (build/bin).  They include the library's headers, so they are
    rebuilt whenever one of those changed (the Makefile lists the headers as prerequisites): a binary built
    against an older class layout crashes at its first call into the library."""
    import shutil
    root = CSRC.parent
    if not shutil.which("make") or not (root / "Makefile").exists():
        return
    r = subprocess.run(["make", "-j8", "bench", "examples", "cpptests"], cwd=str(root), capture_output=True, text=True)
    if verbose and r.stdout.strip():
        print("  make bench examples cpptests: " + str(len(r.stdout.strip().splitlines())) + " step(s)")
    if r.returncode != 0:
        raise RuntimeError("make bench examples cpptests failed:\n" + r.stdout[-2000:] + r.stderr[-2000:])


def build_all(verbose: bool = True) -> None:
    build_library(verbose)
    build_torch_extension(verbose)
    build_binaries(verbose)


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "lib":
        build_library()
    elif len(sys.argv) > 1 and sys.argv[1] == "ptxas":
        print(ptxas_report())
    else:
        build_all()
