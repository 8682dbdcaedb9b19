// benchmark_yali_mpi: all-reduce with ONE PROCESS PER GPU (yali::MPIComm style).
// Start it with the bundled launcher or torchrun:
//
//   python -m yali_b200.launch -np 8 bench/bin/benchmark_yali_mpi 524288 1000 1 auto 0 cuda-events bf16
//
// Same positional arguments as benchmark_yali (gpus is taken from the launcher).
// Buffers are pre-allocated from the symmetric heap (exported once at start-up) or,
// with symmetric=0, plain cudaMalloc buffers that go through the staged paths.
// Every call is timed on the device; per call the time is the max over ranks.
//
// Parity: bench/benchmark_yali_mpi.cu of the reference (exactly two MPI ranks, IPC
// exchange of the buffers, MPI_Allreduce(MAX) of the per-rank time).
#include <cuda_runtime.h>

#include <chrono>

#include "bench_common.h"
#include "ops/buffer_ops.h"
#include "ops/yali.h"

using namespace yali;

#define CK(x)                                                                                \
    do {                                                                                     \
        cudaError_t e_ = (x);                                                                \
        if (e_ != cudaSuccess) {                                                             \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            std::exit(1);                                                                    \
        }                                                                                    \
    } while (0)

int main(int argc, char** argv) {
    bench::Args a = bench::Parse(argc, argv);
    if (a.help) {
        bench::Usage(argv[0], "All-reduce benchmark, one process per GPU (launch with python -m yali_b200.launch).");
        return 0;
    }
    const size_t bytes = a.elements * DtypeSize(a.dtype);
    CommOptions copt;
    copt.heap_bytes = (3ull << 30) + 2 * bytes;
    MPIComm comm(&argc, &argv, copt);
    if (!comm.ok()) return 2;
    const int W = comm.world_size(), rank = comm.rank();
    a.gpus = W;
    void *send = nullptr, *recv = nullptr;
    if (a.symmetric) {
        send = comm.alloc(bytes);
        recv = comm.alloc(bytes);
        if (!send || !recv) {
            std::fprintf(stderr, "rank %d: symmetric allocation failed: %s\n", rank, comm.error().c_str());
            return 2;
        }
    } else {
        CK(cudaMalloc(&send, bytes ? bytes : 16));
        CK(cudaMalloc(&recv, bytes ? bytes : 16));
    }
    cudaStream_t st = comm.stream();
    CK(FillRandom(send, a.elements, a.dtype, kDistUniformPm1, 1234 + rank, st));
    CK(cudaStreamSynchronize(st));
    OpOptions opt;
    opt.mode = a.mode;
    opt.ctas = a.lanes;
    auto call = [&]() {
        cudaError_t e = allreduce_raw(comm, send, recv, a.elements, a.dtype, st, true, opt);
        if (e != cudaSuccess) {
            std::fprintf(stderr, "rank %d: all-reduce: %s (%s)\n", rank, cudaGetErrorString(e),
                         comm.impl()->last_error().c_str());
            std::exit(3);
        }
    };
    if (rank == 0)
        std::printf("YALI-B200 AllReduce Benchmark, one process per GPU (%s) ranks=%d %zu elements (%.2f MB) calls=%d "
                    "warmup=%d heap=%s multicast=%d buffers=%s\n",
                    DtypeName(a.dtype), W, a.elements, bytes / 1e6, a.calls, a.warmup, comm.impl()->heap_kind(),
                    comm.impl()->has_multicast() ? 1 : 0, a.symmetric ? "symmetric" : "cudaMalloc");
    for (int i = 0; i < a.warmup; ++i) call();
    CK(comm.barrier());
    Bootstrap* bs = comm.impl()->bootstrap();
    std::vector<double> per(a.calls, 0.0);
    double total_us = 0;
    bool traced = false;
    if (a.timing == bench::TimingMode::CudaEvents) {
        std::vector<cudaEvent_t> ev(a.calls + 1);
        for (auto& e : ev) CK(cudaEventCreate(&e));
        CK(cudaEventRecord(ev[0], st));
        for (int c = 0; c < a.calls; ++c) {
            call();
            CK(cudaEventRecord(ev[c + 1], st));
        }
        CK(comm.sync());
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, ev[0], ev[a.calls]));
        total_us = ms * 1e3;
        for (int c = 0; c < a.calls; ++c) {
            CK(cudaEventElapsedTime(&ms, ev[c], ev[c + 1]));
            per[c] = ms * 1e3;
        }
        // Average from a second batch with one event pair (see benchmark_yali.cu).
        CK(comm.barrier());
        cudaEvent_t b0, b1;
        CK(cudaEventCreate(&b0));
        CK(cudaEventCreate(&b1));
        CK(cudaEventRecord(b0, st));
        comm.impl()->SetTrace(true);  // kernels stamp their own start and end (no host jitter)
        for (int c = 0; c < a.calls; ++c) call();
        comm.impl()->SetTrace(false);
        traced = true;
        CK(cudaEventRecord(b1, st));
        CK(comm.sync());
        CK(cudaEventElapsedTime(&ms, b0, b1));
        total_us = ms * 1e3;
    } else if (a.timing == bench::TimingMode::Graph) {
        // All calls in one CUDA graph: no host launch work between the kernels.  Two replays, the
        // second one is timed.
        cudaGraph_t graph;
        cudaGraphExec_t exec;
        call();  // outside the capture: one-time kernel attributes
        CK(comm.sync());
        CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        comm.impl()->SetTrace(true);
        for (int c = 0; c < a.calls; ++c) call();
        comm.impl()->SetTrace(false);
        traced = true;
        CK(cudaStreamEndCapture(st, &graph));
        CK(cudaGraphInstantiate(&exec, graph, 0));
        cudaEvent_t g0, g1;
        CK(cudaEventCreate(&g0));
        CK(cudaEventCreate(&g1));
        CK(cudaGraphLaunch(exec, st));
        CK(comm.sync());
        CK(cudaEventRecord(g0, st));
        CK(cudaGraphLaunch(exec, st));
        CK(cudaEventRecord(g1, st));
        CK(comm.sync());
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, g0, g1));
        total_us = ms * 1e3;
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(graph);
    } else {
        auto t0 = std::chrono::steady_clock::now();
        for (int c = 0; c < a.calls; ++c) {
            auto s0 = std::chrono::steady_clock::now();
            call();
            if (a.timing == bench::TimingMode::Latency) {
                CK(comm.sync());
                per[c] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - s0).count();
            }
        }
        CK(comm.sync());
        total_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    }
    CK(comm.barrier());
    // Max over ranks, call by call and for the whole batch.
    if (bs && W > 1) {
        std::vector<double> mine(per);
        mine.push_back(total_us);
        std::vector<double> all(mine.size() * W);
        if (bs->allgather(mine.data(), all.data(), mine.size() * sizeof(double)) != Result::Success) return 4;
        for (size_t c = 0; c < mine.size(); ++c) {
            double m = 0;
            for (int r = 0; r < W; ++r) m = std::max(m, all[r * mine.size() + c]);
            if (c < per.size()) per[c] = m;
            else total_us = m;
        }
    }
    // Device timeline of the last batch: duration (first CTA in -> last CTA out) and cadence (end to
    // end of consecutive calls), call by call the max over ranks.
    bench::Stats dev_calls, dev_cadence;
    if (traced) {
        const int want = std::min(a.calls, 4096);
        std::vector<uint64_t> buf(static_cast<size_t>(want) * 2);
        uint64_t seen = 0;
        const int n = comm.impl()->ReadTrace(0, buf.data(), want, &seen);
        std::vector<double> mine(static_cast<size_t>(want) * 2, 0.0);
        for (int c = 0; c < n; ++c) {
            mine[c] = (buf[2 * c + 1] - buf[2 * c]) * 1e-3;
            if (c > 0) mine[want + c] = (buf[2 * c + 1] - buf[2 * c - 1]) * 1e-3;
        }
        std::vector<double> all(mine.size() * W);
        if (bs && W > 1) {
            if (bs->allgather(mine.data(), all.data(), mine.size() * sizeof(double)) != Result::Success) return 4;
        } else {
            all = mine;
        }
        std::vector<double> dur(want, 0.0), cad(want > 1 ? want - 1 : 0, 0.0);
        for (int r = 0; r < (bs && W > 1 ? W : 1); ++r)
            for (int c = 0; c < want; ++c) {
                dur[c] = std::max(dur[c], all[r * mine.size() + c]);
                if (c > 0) cad[c - 1] = std::max(cad[c - 1], all[r * mine.size() + want + c]);
            }
        if (n == want && want > 0) {
            dev_calls = bench::Summarise(dur);
            dev_cadence = bench::Summarise(cad);
        }
    }
    int ok = 1;
    if (a.verify) ok = ValidateRandomResult(recv, a.elements, a.dtype, a.dtype, kDistUniformPm1, 1234, W, 1.0f, nullptr);
    if (bs && W > 1) {
        std::vector<int> oks(W);
        bs->allgather(&ok, oks.data(), sizeof(int));
        for (int o : oks) ok &= o;
    }
    if (rank == 0) {
        bench::Stats s = (a.timing == bench::TimingMode::Throughput || a.timing == bench::TimingMode::Graph)
                             ? bench::Stats()
                             : bench::Summarise(per);
        const LastCallInfo& lc = comm.impl()->last_call();
        char extra[512];
        int len = std::snprintf(extra, sizeof(extra), "\"variant\":\"%s\",\"ctas\":%u,\"slot_bytes\":%u,\"stages\":%u,"
                                "\"symmetric\":%d,\"processes\":%d", VariantName(lc.variant), lc.ctas, lc.slot_bytes,
                                lc.stages, a.symmetric ? 1 : 0, W);
        if (dev_calls.n)
            std::snprintf(extra + len, sizeof(extra) - len,
                          ",\"dev_p50_us\":%.3f,\"dev_p99_us\":%.3f,\"dev_max_us\":%.3f,\"cadence_p50_us\":%.3f,"
                          "\"cadence_p99_us\":%.3f,\"dev_samples\":%zu",
                          dev_calls.p50, dev_calls.p99, dev_calls.max, dev_cadence.p50, dev_cadence.p99, dev_calls.n);
        const char* kname = bench::KernelLabel(lc.variant, lc.flags);
        bench::Report("YALI", kname, a, W, total_us / a.calls, &s, extra);
        if (a.verify) std::printf("Correctness: %s\n", ok ? "PASSED" : "FAILED");
    }
    if (!a.symmetric) {
        cudaFree(send);
        cudaFree(recv);
    }
    return ok ? 0 : 1;
}
