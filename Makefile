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

.PHONY: all lib bench examples cpptests run-cpptests reference clean test-cpu test-gpu test run-examples \
        run-examples-mp run-nccl-baseline hw-info hw-baseline sweep-quick sweep-standard sweep-full \
        quick-benchmark tp-layer ptxas format
all: lib
lib:
	$(PY) -m yali_b200._build
$(LIB):
	$(PY) -m yali_b200._build lib
$(BIN):
	mkdir -p $(BIN)

BENCH := $(BIN)/benchmark_yali $(BIN)/benchmark_yali_mpi $(BIN)/p2p_bandwidth
BENCH_NCCL := $(BIN)/benchmark_nccl $(BIN)/benchmark_nccl_mpi $(BIN)/nccl_sweep
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
$(BIN)/nccl_sweep: bench/nccl_sweep.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK) -lnccl

EXAMPLES := $(BIN)/example_simple $(BIN)/example_multilane $(BIN)/example_simple_mpi $(BIN)/example_multilane_mpi \
            $(BIN)/example_manual_ipc
examples: $(EXAMPLES)
$(BIN)/example_simple: examples/01_single_process/01_allreduce/simple.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/example_multilane: examples/01_single_process/01_allreduce/multilane.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/example_simple_mpi: examples/02_multi_process/01_allreduce/simple_mpi.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/example_multilane_mpi: examples/02_multi_process/01_allreduce/multilane_mpi.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)
$(BIN)/example_manual_ipc: examples/02_multi_process/01_allreduce/manual_ipc.cu $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) $< -o $@ $(LINK)

CPPTESTS := $(patsubst tests/cpp/%.cu,$(BIN)/%,$(wildcard tests/cpp/test_*.cu))
cpptests: $(CPPTESTS)
$(BIN)/test_%: tests/cpp/test_%.cu tests/cpp/test_framework.h $(HDRS) $(LIB) | $(BIN)
	$(NVCC) $(NVFLAGS) -Itests/cpp $< -o $@ $(LINK)
run-cpptests: cpptests
	@set -e; for t in $(CPPTESTS); do echo "== $$t"; $$t; done

# ---- tests
test-cpu:
	$(PY) -m pytest tests -q -m "not gpu"
test-gpu: lib cpptests examples bench
	$(PY) -m pytest tests -q -m gpu
test: test-cpu test-gpu

# ---- examples and baselines (GPUS=2|4|8)
GPUS ?= 2
PORT ?= 29531
TORCHRUN := $(PY) -m torch.distributed.run --nnodes=1 --nproc-per-node $(GPUS) --master-addr 127.0.0.1 --master-port $(PORT)
run-examples: examples
	$(BIN)/example_simple
	YALI_GPUS=$(GPUS) $(BIN)/example_multilane
run-examples-mp: examples
	$(PY) -m yali_b200.launch -np $(GPUS) $(BIN)/example_simple_mpi
	$(PY) -m yali_b200.launch -np $(GPUS) $(BIN)/example_multilane_mpi
	$(PY) -m yali_b200.launch -np $(GPUS) $(BIN)/example_manual_ipc
run-nccl-baseline: bench
	$(PY) bench/validate_baselines.py --run --gpus $(GPUS)
	$(PY) -m yali_b200.launch -np $(GPUS) $(BIN)/benchmark_nccl_mpi 33554432 200 0 auto 0 cuda-events fp32

# ---- hardware
hw-info:
	$(PY) -c "from yali_b200.utils import hw_info; import json; print(json.dumps(hw_info.system_info(), indent=1))"
hw-baseline: $(BIN)/p2p_bandwidth
	$(BIN)/p2p_bandwidth

# ---- sweeps (results/<mode>: raw lines, CSVs, summary.md)
sweep-quick sweep-standard sweep-full: sweep-%:
	$(PY) bench/run_sweep.py --gpus $(GPUS) --mode $* --out results/$*
quick-benchmark: bench
	$(PY) bench/quick_benchmark.py --gpus $(GPUS)
tp-layer:
	$(TORCHRUN) bench/bench_tp_layer.py --graph

# ---- developer aids
ptxas:
	$(PY) -m yali_b200._build ptxas
format:
	clang-format -i $$(git ls-files 'csrc/*' 'bench/*.cu' 'bench/*.h' 'tests/cpp/*' 'examples/*.cu' | grep -E '\.(h|cc|cu|cuh)$$')

# make reference REFERENCE_DIR=<checkout of the reference>
reference:
	bash baseline/build_reference.sh $(REFERENCE_DIR)
clean:
	rm -rf build yali_b200/lib yali_b200/_C.so
