#!/usr/bin/env bash
# Builds the UNMODIFIED reference (its benchmark_yali, benchmark_nccl and an
# end-to-end harness around its ops API) for sm_100 into baseline/_ref/.
# The reference is not a Python package (pip has nothing to install) and its
# Bazel build and NCCL submodule are not available offline, so the sources are
# compiled directly with nvcc.  The three NCCL-internal headers it includes are
# replaced by a shim that forwards to the system <nccl.h>.
set -euo pipefail
REF="${1:-${YALI_REFERENCE_DIR:?usage: baseline/build_reference.sh <checkout of the reference>}}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT/shim"
cat > "$OUT/shim/collectives.h" <<'EOS'
#pragma once
#include <nccl.h>
template <typename T> struct FuncSum {};
EOS
echo "#pragma once" > "$OUT/shim/device.h"
echo "#pragma once" > "$OUT/shim/primitives.h"
FLAGS=(-std=c++17 -O3 -rdc=true --expt-extended-lambda -lineinfo -gencode arch=compute_100,code=sm_100
       -I"$REF" -I"$REF/src/include" -I"$REF/src/kernels" -I"$REF/src" -I"$OUT/shim")
nvcc "${FLAGS[@]}" "$REF/bench/benchmark_yali.cu" "$REF/src/kernels/stream.cu" -o "$OUT/benchmark_yali" -lcudadevrt
nvcc "${FLAGS[@]}" "$REF/bench/benchmark_nccl.cu" -o "$OUT/benchmark_nccl" -lnccl -lcudadevrt || \
    echo "benchmark_nccl: link against the system NCCL failed" >&2
nvcc "${FLAGS[@]}" "$HERE/ref_e2e_harness.cu" "$REF/src/kernels/stream.cu" -o "$OUT/ref_e2e" -lcudadevrt
ls -la "$OUT"
