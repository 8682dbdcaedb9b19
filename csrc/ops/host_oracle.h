// Plain CPU restatements of every fused operation, used as test oracles and as
// the timed CPU baseline.  fp64 accumulation, inputs as fp32 arrays (callers
// round to the storage type first when they want to model 16-bit inputs).
//
// Parity: the reference's only oracle is "every element equals N(N+1)/2"
// (src/common/validation.cuh:81-82).
#pragma once

#include <cstddef>
#include <cstdint>

namespace yali {
namespace oracle {

// Rounds an fp32 value to bf16 / fp16 and back (round-to-nearest-even).
float RoundBf16(float x);
float RoundFp16(float x);

// out[i] = scale * sum_r in[r][i]
void AllReduceSum(const float* const* in, int world, size_t n, double scale, double* out);

// y[row] = RMSNorm(sum[row] + residual[row]) * weight ; residual may be null.
// pre_norm (optional) receives sum + residual.
void ResidualRmsNorm(const double* sum, const float* residual, const float* weight, size_t rows, size_t hidden,
                     double eps, double* y, double* pre_norm);

// c[m][n] = sum_k a[m][k] * b[k][n]    (row-major, fp64 accumulate)
void Gemm(const float* a, const float* b, size_t m, size_t n, size_t k, double* c);

// Partition helpers mirrored from the device code, for property tests.
// Elements [begin, end) of the message that CTA `cta` of `ctas` handles in the one-shot kernel.
void FlashSlice(uint64_t count, int vec, uint32_t ctas, uint32_t cta, bool vec_ok, uint64_t* vb, uint64_t* ve,
                uint64_t* tb, uint64_t* te);
// Element range of iteration `it` of lane `lane` inside shard `q` in the two-shot kernel.
void StreamPiece(uint64_t count, uint64_t shard_elems, uint64_t piece_elems, uint32_t lanes, uint32_t lane,
                 uint32_t it, int q, uint64_t* eb, uint64_t* ee);
uint32_t StreamIters(uint64_t shard_elems, uint64_t piece_elems, uint32_t lanes, uint32_t lane);

}  // namespace oracle
}  // namespace yali
