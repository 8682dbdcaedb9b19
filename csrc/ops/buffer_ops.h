// Seeded buffer fills, conversion and validation helpers (host API), and the
// counter-based generator they share with the host-side oracles.
//
// Parity: SeedBufferSync / ZeroBuffer / AllocAndSeed (src/common/buffer_ops.cuh:26-59),
// ConvertBufferToFloat / VerifyAllReduceSum / ValidateRankResult
// (src/common/validation.cuh:28-115).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cmath>
#include <cstddef>

#include "../core/status.h"

#if defined(__CUDACC__)
#define YALI_HD __host__ __device__
#else
#define YALI_HD
#endif

namespace yali {

enum RandomDist : int { kDistUniformPm1 = 0, kDistNormal = 1 };

// Philox4x32-10 keyed by `seed`, counter = element index.  Same bits on host and device.
YALI_HD inline void Philox4x32(uint64_t seed, uint64_t index, uint32_t out[4]) {
    uint32_t c0 = static_cast<uint32_t>(index), c1 = static_cast<uint32_t>(index >> 32), c2 = 0u, c3 = 0u;
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
    for (int round = 0; round < 10; ++round) {
        const uint64_t p0 = 0xD2511F53ull * c0, p1 = 0xCD9E8D57ull * c2;
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
        c1 = static_cast<uint32_t>(p1);
        c3 = static_cast<uint32_t>(p0);
        c0 = n0;
        c2 = n2;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0;
    out[1] = c1;
    out[2] = c2;
    out[3] = c3;
}

// Element `index` of the stream `seed`: U(-1,1) or N(0,1).
YALI_HD inline float RandomValue(int dist, uint64_t seed, uint64_t index) {
    uint32_t x[4];
    Philox4x32(seed, index, x);
    const float u0 = (static_cast<float>(x[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
    if (dist == kDistUniformPm1) return 2.0f * u0 - 1.0f;
    const float u1 = static_cast<float>(x[1] >> 8) * (1.0f / 16777216.0f);  // [0,1)
    return sqrtf(-2.0f * logf(u0)) * cosf(6.28318530717958647692f * u1);
}

struct ValidateReport {
    unsigned long long mismatches;
    unsigned long long first_mismatch;  // ~0 when none
    double max_abs_err;
};

// Default tolerances for a result stored in `out` that sums `world` inputs of magnitude O(1).
inline void DefaultTolerance(Dtype out, int world, double* rtol, double* atol) {
    switch (out) {
        case Dtype::FP32: *rtol = 1e-5; *atol = 2e-6 * world; break;
        case Dtype::FP16: *rtol = 2e-3; *atol = 2e-3 * world; break;
        case Dtype::BF16: *rtol = 1e-2; *atol = 1e-2 * world; break;
    }
}

// ---- device-side operations (asynchronous on `s`, current device) ----
cudaError_t FillConstant(void* p, uint64_t n, Dtype dt, float v, cudaStream_t s);
cudaError_t FillRandom(void* p, uint64_t n, Dtype dt, int dist, uint64_t seed, cudaStream_t s);
cudaError_t ConvertToFloat(const void* src, float* dst, uint64_t n, Dtype dt, cudaStream_t s);
// Checks out[i] == scale * sum_{r<world} gen(seed_base+r, index_offset+i) (inputs rounded to in_dt);
// accumulates into *d_rep (device memory, zero it and set first_mismatch = ~0 beforehand).
cudaError_t ValidateSumAsync(const void* out, uint64_t n, uint64_t index_offset, Dtype in_dt, Dtype out_dt, int dist,
                             uint64_t seed_base, int world, float scale, double rtol, double atol,
                             ValidateReport* d_rep, cudaStream_t s);

// x[row] = RMSNorm(x[row] + residual[row]) * weight, in place; residual / residual_out may be nullptr.
cudaError_t ResidualRmsNormInPlace(void* x, const void* residual, void* residual_out, const void* weight,
                                   uint64_t rows, uint32_t hidden, float eps, Dtype dt, cudaStream_t s);

// ---- synchronous conveniences with the reference's names ----
// Fills with one value and waits (reference: SeedBufferSync).
cudaError_t SeedBufferSync(void* p, size_t n, Dtype dt, float value);
cudaError_t ZeroBuffer(void* p, size_t bytes, cudaStream_t s = nullptr);
// cudaMalloc + constant fill (reference: AllocAndSeed).
cudaError_t AllocAndSeed(void** p, size_t n, Dtype dt, float value);
// Copies a device buffer to host floats (reference: ConvertBufferToFloat).
cudaError_t ConvertBufferToFloat(const void* d_src, float* h_dst, size_t n, Dtype dt);
// Host loop: all elements within `tol` of `expected`?  Reports first mismatch and count
// (reference: VerifyAllReduceSum).
bool VerifyAllReduceSum(const float* host, size_t n, float expected, float tol, size_t* first_mismatch,
                        size_t* mismatch_count);
// Result of an all-reduce over ranks seeded with rank+1: every element == world*(world+1)/2
// (reference: ValidateRankResult).
bool ValidateRankResult(const void* d_recv, size_t n, Dtype dt, int rank, int world);
// Random-data variant: validates against the generator sum; fills *rep when given.
bool ValidateRandomResult(const void* d_recv, size_t n, Dtype in_dt, Dtype out_dt, int dist, uint64_t seed_base,
                          int world, float scale, ValidateReport* rep);

}  // namespace yali
