// Shared pieces of the C++ benchmarks: argument parsing in the reference's
// positional order, timing modes, statistics and the result line.
//
// Parity: bench/benchmark_yali.cu:86-110 (dtype from env, TimingMode), :300-311
// (bus bandwidth and the result line), scripts/sweep.py:129-179 (BenchStats).
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "comm/layout.h"
#include "comm/topology.h"
#include "core/status.h"
#include "ops/tuning.h"

namespace bench {

enum class TimingMode { Throughput, Latency, CudaEvents, Graph };

inline const char* TimingModeName(TimingMode m) {
    return m == TimingMode::CudaEvents ? "cuda-events"
           : m == TimingMode::Latency  ? "latency"
           : m == TimingMode::Graph    ? "graph"
                                       : "throughput";
}

struct Args {
    size_t elements = 262144;  // 1 MiB of fp32
    int calls = 100;
    int warmup = 20;
    bool verify = false;
    yali::KernelMode mode = yali::KernelMode::Auto;
    int lanes = 0;
    TimingMode timing = TimingMode::CudaEvents;
    yali::Dtype dtype = yali::Dtype::FP32;
    int gpus = 2;
    bool symmetric = true;
    bool help = false;
};

// argv: elements calls verify mode lanes timing dtype [gpus] [symmetric]; YALI_DTYPE, YALI_GPUS, YALI_WARMUP from the environment.
inline Args Parse(int argc, char** argv) {
    Args a;
    if (const char* e = std::getenv("YALI_DTYPE")) yali::ParseDtype(e, &a.dtype);
    if (const char* e = std::getenv("YALI_GPUS")) a.gpus = std::atoi(e);
    if (const char* e = std::getenv("YALI_WARMUP")) a.warmup = std::atoi(e);
    if (argc == 2 && (!std::strcmp(argv[1], "-h") || !std::strcmp(argv[1], "--help"))) {
        a.help = true;
        return a;
    }
    if (argc > 1) a.elements = std::strtoull(argv[1], nullptr, 10);
    if (argc > 2) a.calls = std::atoi(argv[2]);
    if (argc > 3) a.verify = std::atoi(argv[3]) != 0;
    if (argc > 4) yali::ParseKernelMode(argv[4], &a.mode);
    if (argc > 5) a.lanes = std::atoi(argv[5]);
    if (argc > 6) {
        if (!std::strcmp(argv[6], "latency")) a.timing = TimingMode::Latency;
        else if (!std::strcmp(argv[6], "throughput")) a.timing = TimingMode::Throughput;
        else if (!std::strcmp(argv[6], "graph")) a.timing = TimingMode::Graph;
        else a.timing = TimingMode::CudaEvents;
    }
    if (argc > 7) yali::ParseDtype(argv[7], &a.dtype);
    if (argc > 8) a.gpus = std::atoi(argv[8]);
    if (argc > 9) a.symmetric = std::atoi(argv[9]) != 0;
    return a;
}

inline void Usage(const char* prog, const char* what) {
    std::printf("Usage: %s [elements] [calls] [verify] [mode] [lanes] [timing] [dtype] [gpus] [symmetric]\n", prog);
    std::printf("  %s\n", what);
    std::printf("  elements   number of elements per rank (default 262144 = 1 MiB of fp32)\n");
    std::printf("  calls      timed all-reduce calls (default 100; warm-up: YALI_WARMUP, default 20)\n");
    std::printf("  verify     1: check every element against the fp64 sum of the seeded inputs\n");
    std::printf("  mode       auto | flash | stream | nvls\n");
    std::printf("  lanes      CTAs (flash, nvls) or lanes (stream) per rank, 0 = tuned\n");
    std::printf("  timing     cuda-events (device time, per-call percentiles) | throughput | latency |\n");
    std::printf("             graph (all calls captured in one CUDA graph, device time of one replay; *_mpi only)\n");
    std::printf("  dtype      fp32 | fp16 | bf16 (or YALI_DTYPE)\n");
    std::printf("  gpus       ranks, one GPU each (default 2, or YALI_GPUS)\n");
    std::printf("  symmetric  1: buffers from the communicator's symmetric heap (default), 0: cudaMalloc\n");
}

// Kernel name of the result line ("YALI (Flash-fp32, ...)" in the reference's format).
inline const char* KernelLabel(yali::Variant v, uint32_t flags) {
    switch (v) {
        case yali::Variant::Flash: return (flags & yali::kFlagLowLatency) ? "FlashLL" : "Flash";
        case yali::Variant::Stream: return "Stream";
        case yali::Variant::NvlsOneShot: return "NVLS1";
        case yali::Variant::NvlsTwoShot: return "NVLS2";
        case yali::Variant::FlashPull: return "FlashPull";
        case yali::Variant::StreamDirect: return "StreamDirect";
        case yali::Variant::CopyEngine: return "CopyEngine";
    }
    return "?";
}

struct Stats {
    double mean = 0, stddev = 0, min = 0, max = 0, p50 = 0, p90 = 0, p95 = 0, p99 = 0, cv_pct = 0;
    size_t n = 0;
};

inline double Percentile(std::vector<double> v, double q) {
    if (v.empty()) return 0;
    std::sort(v.begin(), v.end());
    const double pos = q / 100.0 * (v.size() - 1);
    const size_t lo = static_cast<size_t>(pos);
    const size_t hi = std::min(v.size() - 1, lo + 1);
    return v[lo] + (v[hi] - v[lo]) * (pos - lo);
}

inline Stats Summarise(const std::vector<double>& v) {
    Stats s;
    s.n = v.size();
    if (v.empty()) return s;
    double sum = 0;
    s.min = s.max = v[0];
    for (double x : v) {
        sum += x;
        s.min = std::min(s.min, x);
        s.max = std::max(s.max, x);
    }
    s.mean = sum / v.size();
    double var = 0;
    for (double x : v) var += (x - s.mean) * (x - s.mean);
    s.stddev = v.size() > 1 ? std::sqrt(var / (v.size() - 1)) : 0;
    s.cv_pct = s.mean > 0 ? 100.0 * s.stddev / s.mean : 0;
    s.p50 = Percentile(v, 50);
    s.p90 = Percentile(v, 90);
    s.p95 = Percentile(v, 95);
    s.p99 = Percentile(v, 99);
    return s;
}

// The line the sweep scripts parse, in the reference's format, followed by one JSON line.
inline void Report(const char* impl, const char* kernel, const Args& a, int ranks, double avg_us, const Stats* per_call,
                   const char* extra_json) {
    const double bytes = static_cast<double>(a.elements) * yali::DtypeSize(a.dtype);
    const double gbps = bytes * yali::BusBwFactor(ranks) / 1e9 / (avg_us / 1e6);
    yali::NVLinkInfo nv = yali::DetectNVLinkConfig(0);
    const double peak = nv.measuredUnidirectionalGBs > 0 ? nv.measuredUnidirectionalGBs
                                                          : (nv.valid ? nv.unidirectionalGBs : 900.0);
    std::printf("%s (%s-%s, %s): %d calls, %.2f us/call avg, %.2f GB/s (%.1f%% SoL)\n", impl, kernel,
                yali::DtypeName(a.dtype), TimingModeName(a.timing), a.calls, avg_us, gbps, 100.0 * gbps / peak);
    std::printf("{\"impl\":\"%s\",\"kernel\":\"%s\",\"dtype\":\"%s\",\"timing\":\"%s\",\"ranks\":%d,\"bytes\":%.0f,"
                "\"calls\":%d,\"warmup\":%d,\"avg_us\":%.3f,\"busbw_gbps\":%.3f,\"algbw_gbps\":%.3f,\"sol_peak_gbps\":%.1f",
                impl, kernel, yali::DtypeName(a.dtype), TimingModeName(a.timing), ranks, bytes, a.calls, a.warmup,
                avg_us, gbps, bytes / 1e9 / (avg_us / 1e6), peak);
    if (per_call && per_call->n)
        std::printf(",\"p50_us\":%.3f,\"p90_us\":%.3f,\"p99_us\":%.3f,\"max_us\":%.3f,\"min_us\":%.3f,\"cv_pct\":%.3f",
                    per_call->p50, per_call->p90, per_call->p99, per_call->max, per_call->min, per_call->cv_pct);
    if (extra_json && *extra_json) std::printf(",%s", extra_json);
    std::printf("}\n");
}

}  // namespace bench
