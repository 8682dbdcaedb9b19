// Synchronous conveniences over the fill / convert / validate kernels (see buffer_ops.h).
#include "buffer_ops.h"

#include <cmath>
#include <vector>

namespace yali {

cudaError_t SeedBufferSync(void* p, size_t n, Dtype dt, float value) {
    cudaError_t e = FillConstant(p, n, dt, value, nullptr);
    if (e != cudaSuccess) return e;
    return cudaDeviceSynchronize();
}

cudaError_t ZeroBuffer(void* p, size_t bytes, cudaStream_t s) {
    if (bytes == 0) return cudaSuccess;
    return cudaMemsetAsync(p, 0, bytes, s);
}

cudaError_t AllocAndSeed(void** p, size_t n, Dtype dt, float value) {
    *p = nullptr;
    cudaError_t e = cudaMalloc(p, (n ? n : 1) * DtypeSize(dt));
    if (e != cudaSuccess) return e;
    e = SeedBufferSync(*p, n, dt, value);
    if (e != cudaSuccess) {
        cudaFree(*p);
        *p = nullptr;
    }
    return e;
}

cudaError_t ConvertBufferToFloat(const void* d_src, float* h_dst, size_t n, Dtype dt) {
    if (n == 0) return cudaSuccess;
    if (dt == Dtype::FP32) return cudaMemcpy(h_dst, d_src, n * sizeof(float), cudaMemcpyDeviceToHost);
    float* tmp = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&tmp), n * sizeof(float));
    if (e != cudaSuccess) return e;
    e = ConvertToFloat(d_src, tmp, n, dt, nullptr);
    if (e == cudaSuccess) e = cudaMemcpy(h_dst, tmp, n * sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(tmp);
    return e;
}

bool VerifyAllReduceSum(const float* host, size_t n, float expected, float tol, size_t* first_mismatch,
                        size_t* mismatch_count) {
    size_t bad = 0, first = n;
    for (size_t i = 0; i < n; ++i) {
        if (!(std::fabs(host[i] - expected) <= tol)) {
            if (bad == 0) first = i;
            ++bad;
        }
    }
    if (first_mismatch) *first_mismatch = first;
    if (mismatch_count) *mismatch_count = bad;
    return bad == 0;
}

bool ValidateRankResult(const void* d_recv, size_t n, Dtype dt, int /*rank*/, int world) {
    std::vector<float> host(n);
    if (ConvertBufferToFloat(d_recv, host.data(), n, dt) != cudaSuccess) return false;
    const float expected = 0.5f * world * (world + 1);
    const float tol = dt == Dtype::FP32 ? 1e-3f : (dt == Dtype::FP16 ? 1e-2f : 1e-1f);
    return VerifyAllReduceSum(host.data(), n, expected, tol, nullptr, nullptr);
}

bool ValidateRandomResult(const void* d_recv, size_t n, Dtype in_dt, Dtype out_dt, int dist, uint64_t seed_base,
                          int world, float scale, ValidateReport* rep) {
    ValidateReport h = {0ull, ~0ull, 0.0};
    ValidateReport* d = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&d), sizeof(h)) != cudaSuccess) return false;
    double rtol, atol;
    DefaultTolerance(out_dt, world, &rtol, &atol);
    atol *= std::fabs(scale) > 1.f ? std::fabs(scale) : 1.f;
    bool ok = cudaMemcpy(d, &h, sizeof(h), cudaMemcpyHostToDevice) == cudaSuccess &&
              ValidateSumAsync(d_recv, n, 0, in_dt, out_dt, dist, seed_base, world, scale, rtol, atol, d, nullptr) ==
                  cudaSuccess &&
              cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost) == cudaSuccess;
    cudaFree(d);
    if (rep) *rep = h;
    return ok && h.mismatches == 0;
}

}  // namespace yali
