# Native build: the library, the C++ benchmarks, examples and tests.
#   make            library + torch extension (python -m yali_b200._build)
#   make bench      build/bin/benchmark_{yali,nccl}{,_mpi}
#   make examples   build/bin/example_*
#   make cpptests   build/bin/test_* (run them with `make run-cpptests` on a GPU box)
#   make reference  builds the unmodified reference into baseline/_ref/
# Reference counterparts: Makefile / BUILD.bazel targets build-*, bench, test-*.
NVCC ?= /usr/local/cuda/bin/nvcc
PY ?= python
ARCH := -gencode arch=compute_100a,code=sm_100a
NVFLAGS := -std=c++17 -O3 -lineinfo --expt-relaxed-constexpr $(ARCH) -Icsrc -Ibench
LIB := yali_b200/lib/libyali_b200.so
LINK := -Lyali_b200/lib -lyali_b200 -Xlinker -rpath -Xlinker '$$ORIGIN/../../yali_b200/lib'
BIN := build/bin
# public headers: every binary that includes them is rebuilt when one changes (class layouts)
HDRS := $(wildcard csrc/*/*.h) $(wildcard csrc/*/*.cuh)

.PHONY: all lib bench examples cpptests run-cpptests reference clean
all: lib
lib:
	$(PY) -m yali_b200._build
$(LIB):
	$(PY) -m yali_b200._build lib
$(BIN):
	mkdir -p $(BIN)

BENCH := $(BIN)/benchmark_yali $(BIN)/benchmark_yali_mpi $(BIN)/p2p_bandwidth
BENCH_NCCL := $(BIN)/benchmark_nccl $(BIN)/benchmark_nccl_mpi
bench: $(BENCH) $(BENCH_NCCL)
$(BIN)/benchmark_yali: bench/benchmark_yali.cu bench/bench_common.h $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/benchmark_yali_mpi: bench/benchmark_yali_mpi.cu bench/bench_common.h $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/p2p_bandwidth: bench/p2p_bandwidth.cu | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@
$(BIN)/benchmark_nccl: bench/benchmark_nccl.cu bench/bench_common.h $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK) -lnccl
$(BIN)/benchmark_nccl_mpi: bench/benchmark_nccl_mpi.cu bench/bench_common.h $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK) -lnccl

EXAMPLES := $(BIN)/example_simple $(BIN)/example_multilane $(BIN)/example_simple_mpi $(BIN)/example_multilane_mpi
examples: $(EXAMPLES)
$(BIN)/example_simple: examples/01_single_process/01_allreduce/simple.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/example_multilane: examples/01_single_process/01_allreduce/multilane.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/example_simple_mpi: examples/02_multi_process/01_allreduce/simple_mpi.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/example_multilane_mpi: examples/02_multi_process/01_allreduce/multilane_mpi.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)

CPPTESTS := $(patsubst tests/cpp/%.cu,$(BIN)/%,$(wildcard tests/cpp/test_*.cu))
cpptests: $(CPPTESTS)
$(BIN)/test_%: tests/cpp/test_%.cu tests/cpp/test_framework.h $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) -Itests/cpp $< -o $@ $(LINK)
run-cpptests: cpptests
	@set -e; for t in $(CPPTESTS); do echo "== $$t"; $$t; done

# make reference REFERENCE_DIR=<checkout of the reference>
reference:
	bash baseline/build_reference.sh $(REFERENCE_DIR)
clean:
	rm -rf build yali_b200/lib yali_b200/_C.so
