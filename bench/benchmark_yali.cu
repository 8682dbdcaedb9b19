// benchmark_yali: all-reduce over 2..8 GPUs driven by ONE process (yali::Comm style).
//
//   benchmark_yali [elements] [calls] [verify] [mode] [lanes] [timing] [dtype] [gpus] [symmetric]
//
// Inputs are U(-1,1) from seed 1234+rank.  In cuda-events mode every call is
// bracketed by events on every rank's stream; a call's time is the max over
// ranks, and the average / p50 / p99 are taken over calls.  `throughput` is wall
// clock with one sync at the end, `latency` syncs after every call.  With
// YALI_EMULATE=1 the ranks are emulated on GPU 0 (for machines with one GPU).
//
// Parity: bench/benchmark_yali.cu of the reference (same positional arguments and
// result line; two GPUs only; one event pair on GPU 0; constant fills).
#include <cuda_runtime.h>

#include <chrono>
#include <memory>

#include "bench_common.h"
#include "comm/communicator.h"
#include "ops/buffer_ops.h"

using namespace yali;

#define CK(x)                                                                                     \
    do {                                                                                          \
        cudaError_t e_ = (x);                                                                     \
        if (e_ != cudaSuccess) {                                                                  \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));      \
            std::exit(1);                                                                         \
        }                                                                                         \
    } while (0)

int main(int argc, char** argv) {
    bench::Args a = bench::Parse(argc, argv);
    if (a.help) {
        bench::Usage(argv[0], "All-reduce benchmark, one process driving all GPUs.");
        return 0;
    }
    const bool emulate = std::getenv("YALI_EMULATE") && std::atoi(std::getenv("YALI_EMULATE")) != 0;
    const int W = a.gpus;
    const size_t bytes = a.elements * DtypeSize(a.dtype);
    CommOptions copt;
    copt.heap_bytes = (3ull << 30) + 2 * bytes;
    std::unique_ptr<Communicator> comm;
    std::string err;
    Result r;
    if (emulate) {
        r = Communicator::CreateEmulated(W, 0, copt, &comm, &err);
    } else {
        std::vector<int> devs(W);
        for (int i = 0; i < W; ++i) devs[i] = i;
        r = Communicator::CreateSingleProcess(devs, copt, &comm, &err);
    }
    if (r != Result::Success) {
        std::fprintf(stderr, "communicator: %s (%s)\n", GetErrorString(r), err.c_str());
        return 2;
    }
    std::vector<void*> send(W), recv(W);
    if (a.symmetric) {
        if (comm->SymmAlloc(bytes, &send) != Result::Success || comm->SymmAlloc(bytes, &recv) != Result::Success) {
            std::fprintf(stderr, "symmetric allocation failed: %s\n", comm->last_error().c_str());
            return 2;
        }
    } else {
        for (int i = 0; i < W; ++i) {
            CK(cudaSetDevice(comm->device_of(i)));
            CK(cudaMalloc(&send[i], bytes ? bytes : 16));
            CK(cudaMalloc(&recv[i], bytes ? bytes : 16));
        }
    }
    std::vector<cudaStream_t> st(W);
    for (int i = 0; i < W; ++i) {
        CK(cudaSetDevice(comm->device_of(i)));
        st[i] = comm->default_stream(i);
        CK(FillRandom(send[i], a.elements, a.dtype, kDistUniformPm1, 1234 + i, st[i]));
        CK(cudaStreamSynchronize(st[i]));
    }
    OpOptions opt;
    opt.mode = a.mode;
    opt.ctas = a.lanes;
    std::vector<const void*> csend(send.begin(), send.end());
    auto call = [&]() {
        Result rr = comm->AllReduce(csend.data(), recv.data(), a.elements, a.dtype, a.dtype, opt, st.data());
        if (rr != Result::Success) {
            std::fprintf(stderr, "all-reduce: %s (%s)\n", GetErrorString(rr), comm->last_error().c_str());
            std::exit(3);
        }
    };
    auto sync_all = [&]() {
        if (comm->Sync(st.data()) != Result::Success) {
            std::fprintf(stderr, "sync: %s\n", comm->last_error().c_str());
            std::exit(3);
        }
    };
    std::printf("================================================================================\n");
    std::printf("YALI-B200 AllReduce Benchmark (%s)  ranks=%d%s  %zu elements (%.2f MB)  calls=%d warmup=%d\n",
                DtypeName(a.dtype), W, emulate ? " (emulated on one GPU)" : "", a.elements, bytes / 1e6, a.calls,
                a.warmup);
    std::printf("heap=%s multicast=%d buffers=%s timing=%s\n", comm->heap_kind(), comm->has_multicast() ? 1 : 0,
                a.symmetric ? "symmetric" : "cudaMalloc", bench::TimingModeName(a.timing));
    std::printf("================================================================================\n");
    for (int i = 0; i < a.warmup; ++i) call();
    sync_all();

    if (a.timing == bench::TimingMode::Graph) {
        std::fprintf(stderr, "timing 'graph' needs one graph per process: use benchmark_yali_mpi (one GPU per rank)\n");
        return 2;
    }
    double avg_us = 0;
    bench::Stats per_call, dev_calls, dev_cadence;
    const int nev = emulate ? 1 : W;
    if (a.timing == bench::TimingMode::CudaEvents) {
        std::vector<std::vector<cudaEvent_t>> ev(nev, std::vector<cudaEvent_t>(a.calls + 1));
        for (int i = 0; i < nev; ++i) {
            CK(cudaSetDevice(comm->device_of(i)));
            for (auto& e : ev[i]) CK(cudaEventCreate(&e));
            CK(cudaEventRecord(ev[i][0], st[i]));
        }
        for (int c = 0; c < a.calls; ++c) {
            call();
            for (int i = 0; i < nev; ++i) {
                CK(cudaSetDevice(comm->device_of(i)));
                CK(cudaEventRecord(ev[i][c + 1], st[i]));
            }
        }
        sync_all();
        std::vector<double> per(a.calls, 0.0);
        double total = 0;
        for (int i = 0; i < nev; ++i) {
            float ms = 0;
            CK(cudaEventElapsedTime(&ms, ev[i][0], ev[i][a.calls]));
            total = std::max(total, static_cast<double>(ms) * 1e3);
            for (int c = 0; c < a.calls; ++c) {
                CK(cudaEventElapsedTime(&ms, ev[i][c], ev[i][c + 1]));
                per[c] = std::max(per[c], static_cast<double>(ms) * 1e3);
            }
        }
        per_call = bench::Summarise(per);
        (void)total;
        // Average from a second batch with one event pair per rank (events between calls
        // keep consecutive launches from overlapping and would inflate the average).
        std::vector<cudaEvent_t> b0(nev), b1(nev);
        for (int i = 0; i < nev; ++i) {
            CK(cudaSetDevice(comm->device_of(i)));
            CK(cudaEventCreate(&b0[i]));
            CK(cudaEventCreate(&b1[i]));
            CK(cudaEventRecord(b0[i], st[i]));
        }
        comm->SetTrace(true);  // the kernels stamp their own start and end: per-call times without host jitter
        for (int c = 0; c < a.calls; ++c) call();
        comm->SetTrace(false);
        for (int i = 0; i < nev; ++i) {
            CK(cudaSetDevice(comm->device_of(i)));
            CK(cudaEventRecord(b1[i], st[i]));
        }
        sync_all();
        {
            // Device timeline: duration of call c = max over ranks of (last CTA out - first CTA in);
            // cadence = max over ranks of the distance between the ends of consecutive calls.
            const int want = std::min(a.calls, 4096);
            std::vector<double> dur(want, 0.0), cad(want > 1 ? want - 1 : 0, 0.0);
            std::vector<uint64_t> buf(static_cast<size_t>(want) * 2);
            bool ok = want > 0;
            for (int i = 0; i < nev && ok; ++i) {
                uint64_t calls_seen = 0;
                const int n = comm->ReadTrace(i, buf.data(), want, &calls_seen);
                ok = n == want;
                for (int c = 0; c < n; ++c) {
                    dur[c] = std::max(dur[c], (buf[2 * c + 1] - buf[2 * c]) * 1e-3);
                    if (c > 0) cad[c - 1] = std::max(cad[c - 1], (buf[2 * c + 1] - buf[2 * c - 1]) * 1e-3);
                }
            }
            if (ok) {
                dev_calls = bench::Summarise(dur);
                dev_cadence = bench::Summarise(cad);
            }
        }
        double batch = 0;
        for (int i = 0; i < nev; ++i) {
            float ms = 0;
            CK(cudaEventElapsedTime(&ms, b0[i], b1[i]));
            batch = std::max(batch, static_cast<double>(ms) * 1e3);
        }
        avg_us = batch / a.calls;
    } else if (a.timing == bench::TimingMode::Throughput) {
        auto t0 = std::chrono::steady_clock::now();
        for (int c = 0; c < a.calls; ++c) call();
        sync_all();
        avg_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / a.calls;
    } else {
        std::vector<double> per(a.calls);
        auto t0 = std::chrono::steady_clock::now();
        for (int c = 0; c < a.calls; ++c) {
            auto s0 = std::chrono::steady_clock::now();
            call();
            sync_all();
            per[c] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - s0).count();
        }
        avg_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / a.calls;
        per_call = bench::Summarise(per);
    }
    const LastCallInfo& lc = comm->last_call();
    char extra[512];
    int len = std::snprintf(extra, sizeof(extra), "\"variant\":\"%s\",\"ctas\":%u,\"slot_bytes\":%u,\"stages\":%u,"
                            "\"symmetric\":%d,\"emulated\":%d", VariantName(lc.variant), lc.ctas, lc.slot_bytes,
                            lc.stages, a.symmetric ? 1 : 0, emulate ? 1 : 0);
    if (dev_calls.n)
        std::snprintf(extra + len, sizeof(extra) - len,
                      ",\"dev_p50_us\":%.3f,\"dev_p99_us\":%.3f,\"dev_max_us\":%.3f,\"cadence_p50_us\":%.3f,"
                      "\"cadence_p99_us\":%.3f,\"dev_samples\":%zu",
                      dev_calls.p50, dev_calls.p99, dev_calls.max, dev_cadence.p50, dev_cadence.p99, dev_calls.n);
    const char* kname = bench::KernelLabel(lc.variant, lc.flags);
    bench::Report("YALI", kname, a, W, avg_us, &per_call, extra);
    int rc = 0;
    if (a.verify) {
        bool all_ok = true;
        for (int i = 0; i < W; ++i) {
            CK(cudaSetDevice(comm->device_of(i)));
            ValidateReport rep;
            bool ok = ValidateRandomResult(recv[i], a.elements, a.dtype, a.dtype, kDistUniformPm1, 1234, W, 1.0f, &rep);
            if (!ok) {
                std::printf("FAILED: rank %d: %llu mismatches, first at %llu, max abs err %g\n", i, rep.mismatches,
                            rep.first_mismatch, rep.max_abs_err);
                all_ok = false;
            }
        }
        std::printf("Correctness: %s\n", all_ok ? "PASSED" : "FAILED");
        rc = all_ok ? 0 : 1;
    }
    if (!a.symmetric) {
        for (int i = 0; i < W; ++i) {
            cudaSetDevice(comm->device_of(i));
            cudaFree(send[i]);
            cudaFree(recv[i]);
        }
    }
    comm.reset();
    return rc;
}
