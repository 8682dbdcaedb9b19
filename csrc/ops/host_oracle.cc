#include "host_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace yali {
namespace oracle {

float RoundBf16(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x;  // NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
    float y;
    std::memcpy(&y, &u, 4);
    return y;
}

float RoundFp16(float x) {
    // Round to 11 significant bits with fp16's exponent range (subnormals below 2^-14).
    if (!std::isfinite(x) || x == 0.f) return x;
    const float ax = std::fabs(x);
    if (ax >= 65520.f) return std::copysign(INFINITY, x);
    int e;
    std::frexp(ax, &e);  // ax = m * 2^e, m in [0.5, 1)
    const int lsb_exp = std::max(e - 11, -24);
    const float q = std::ldexp(1.f, lsb_exp);
    return std::copysign(std::nearbyint(ax / q) * q, x);
}

void AllReduceSum(const float* const* in, int world, size_t n, double scale, double* out) {
    for (size_t i = 0; i < n; ++i) {
        double s = 0.0;
        for (int r = 0; r < world; ++r) s += static_cast<double>(in[r][i]);
        out[i] = s * scale;
    }
}

void ResidualRmsNorm(const double* sum, const float* residual, const float* weight, size_t rows, size_t hidden,
                     double eps, double* y, double* pre_norm) {
    for (size_t r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (size_t h = 0; h < hidden; ++h) {
            double v = sum[r * hidden + h] + (residual ? static_cast<double>(residual[r * hidden + h]) : 0.0);
            if (pre_norm) pre_norm[r * hidden + h] = v;
            y[r * hidden + h] = v;
            ss += v * v;
        }
        const double inv = 1.0 / std::sqrt(ss / static_cast<double>(hidden) + eps);
        for (size_t h = 0; h < hidden; ++h) y[r * hidden + h] *= inv * static_cast<double>(weight[h]);
    }
}

void Gemm(const float* a, const float* b, size_t m, size_t n, size_t k, double* c) {
    for (size_t i = 0; i < m; ++i) {
        double* ci = c + i * n;
        std::fill(ci, ci + n, 0.0);
        for (size_t p = 0; p < k; ++p) {
            const double av = a[i * k + p];
            const float* bp = b + p * n;
            for (size_t j = 0; j < n; ++j) ci[j] += av * static_cast<double>(bp[j]);
        }
    }
}

void FlashSlice(uint64_t count, int vec, uint32_t ctas, uint32_t cta, bool vec_ok, uint64_t* vb, uint64_t* ve,
                uint64_t* tb, uint64_t* te) {
    // Element range of the CTA from values all ranks share; alignment only picks the access width.
    const uint64_t nvec_all = (count + vec - 1) / vec;
    const uint64_t per_v = (nvec_all + ctas - 1) / ctas;
    const uint64_t eb = std::min<uint64_t>(count, static_cast<uint64_t>(cta) * per_v * vec);
    const uint64_t ee = std::min<uint64_t>(count, eb + per_v * vec);
    if (vec_ok) {
        *ve = ee / vec;
        *vb = std::min<uint64_t>(*ve, (eb + vec - 1) / vec);  // eb is a multiple of vec unless the slice is empty
        *tb = std::max<uint64_t>(*ve * vec, eb);
        *te = ee;
    } else {
        *vb = *ve = 0;
        *tb = eb;
        *te = ee;
    }
}

void StreamPiece(uint64_t count, uint64_t shard_elems, uint64_t piece_elems, uint32_t lanes, uint32_t lane,
                 uint32_t it, int q, uint64_t* eb, uint64_t* ee) {
    const uint64_t g = lane + static_cast<uint64_t>(it) * lanes;
    const uint64_t b = static_cast<uint64_t>(q) * shard_elems + g * piece_elems;
    const uint64_t e = std::min(b + piece_elems, static_cast<uint64_t>(q + 1) * shard_elems);
    *eb = std::min(b, count);
    *ee = std::min(e, count);
    if (*ee < *eb) *ee = *eb;
}

uint32_t StreamIters(uint64_t shard_elems, uint64_t piece_elems, uint32_t lanes, uint32_t lane) {
    const uint64_t n_pieces = (shard_elems + piece_elems - 1) / piece_elems;
    return lane < n_pieces ? static_cast<uint32_t>((n_pieces - lane + lanes - 1) / lanes) : 0u;
}

}  // namespace oracle
}  // namespace yali
