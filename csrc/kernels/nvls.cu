// NVLS: all-reduce through the NVSwitch multicast object that covers the
// symmetric heaps.  multimem.ld_reduce makes the switch fetch the same 16 bytes
// from every rank and return their sum (fp32 accumulation for 16-bit types);
// multimem.st makes it write 16 bytes to every rank.
//
//   one-shot : every rank ld_reduces the whole message into its own output.
//              Lowest latency, N times the link traffic: small messages only.
//   two-shot : rank r ld_reduces only shard r and multimem.st's the sums back to
//              all ranks.  Per rank about S(1+1/N) bytes in each direction, so the
//              bus bandwidth can exceed the one-direction link rate.
//
// User buffers outside the heap are staged: CTA c copies slice c of every shard
// into the heap first and copies the result out afterwards (the staging region
// alternates between two halves per call).  Buffers allocated from the heap are
// used in place.  CTA c synchronises only with CTA c of the other ranks, through
// the bounded per-CTA barrier.
//
// Parity: no counterpart in the reference (it has no multicast path; the survey
// of its sources lists none of cuMulticast*, multimem or NVLS).
#include "coll_common.cuh"
#include "launch.h"

namespace yali {

namespace {

template <typename T>
__device__ __forceinline__ uint4 mc_ld_reduce(const void* p);
template <>
__device__ __forceinline__ uint4 mc_ld_reduce<float>(const void* p) {
    return ptx::multimem_ld_reduce_f32x4(p);
}
template <>
__device__ __forceinline__ uint4 mc_ld_reduce<__half>(const void* p) {
    return ptx::multimem_ld_reduce_f16x8(p);
}
template <>
__device__ __forceinline__ uint4 mc_ld_reduce<__nv_bfloat16>(const void* p) {
    return ptx::multimem_ld_reduce_bf16x8(p);
}

template <typename T>
__device__ __forceinline__ uint4 scale16(const uint4& v, float s) {
    constexpr int VEC = TypeTraits<T>::kVec;
    float f[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = 0.f;
    accumulate<T>(f, v);
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] *= s;
    return pack16<T>(f);
}

// `aligned` false: the user buffer (whichever side it is) is aligned to its element type only.
template <typename T>
__device__ __forceinline__ void copy16(char* dst, const char* src, uint64_t vb, uint64_t ve, bool aligned) {
    const int tid = threadIdx.x, nt = blockDim.x;
    uint64_t v = vb + tid;
    if (!aligned) {
        constexpr int VEC = 16 / sizeof(T);
        for (; v < ve; v += nt) {
            const T* s = reinterpret_cast<const T*>(src) + v * VEC;
            T* d = reinterpret_cast<T*>(dst) + v * VEC;
#pragma unroll
            for (int i = 0; i < VEC; ++i) d[i] = s[i];
        }
        return;
    }
    for (; v + 3ull * nt < ve; v += 4ull * nt) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) x[u] = ptx::ld_cg_v4(src + (v + u * nt) * 16);
#pragma unroll
        for (int u = 0; u < 4; ++u) ptx::st_v4(dst + (v + u * nt) * 16, x[u]);
    }
    for (; v < ve; v += nt) ptx::st_v4(dst + v * 16, ptx::ld_cg_v4(src + v * 16));
}


// Vectors [vb, ve): sum over all ranks in the switch (multimem.ld_reduce), optional scale, then
// either a plain store into this rank's output or a multimem.st that writes every rank's output.
// U loads are in flight per thread before the first store.
template <typename T, int U, bool BROADCAST>
__device__ __forceinline__ void reduce_range(const char* mc_in, char* out, uint64_t vb, uint64_t ve, float scale,
                                             bool scaled, bool out_aligned = true) {
    const int tid = threadIdx.x, nt = blockDim.x;
    uint64_t v = vb + tid;
    for (; v + static_cast<uint64_t>(U - 1) * nt < ve; v += static_cast<uint64_t>(U) * nt) {
        uint4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) x[u] = mc_ld_reduce<T>(mc_in + (v + u * nt) * 16);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint4 y = scaled ? scale16<T>(x[u], scale) : x[u];
            if (BROADCAST) ptx::multimem_st_v4(out + (v + u * nt) * 16, y);
            else if (out_aligned) ptx::st_v4(out + (v + u * nt) * 16, y);
            else store16_elems<T>(out, v + u * nt, y);
        }
    }
    for (; v < ve; v += nt) {
        const uint4 x = mc_ld_reduce<T>(mc_in + v * 16);
        const uint4 y = scaled ? scale16<T>(x, scale) : x;
        if (BROADCAST) ptx::multimem_st_v4(out + v * 16, y);
        else if (out_aligned) ptx::st_v4(out + v * 16, y);
        else store16_elems<T>(out, v, y);
    }
}

// count*sizeof(T) is a multiple of 16 (the dispatcher falls back to the peer-to-peer kernels
// otherwise).  Symmetric buffers are 16-byte aligned on every rank; staged user buffers may be
// aligned to their element type only on some ranks (kFlagVecOk clear there).
template <typename T, bool TWO_SHOT>
__global__ void __launch_bounds__(kNvlsThreads, 2) nvls_kernel(const __grid_constant__ CollArgs a) {
    constexpr int VEC = TypeTraits<T>::kVec;
    if (a.flags & kFlagSkipRank) return;
    const CommView& cv = a.cv;
    const int W = cv.world, r = cv.rank;
    const int tid = threadIdx.x, nt = blockDim.x;
    const uint32_t cta = blockIdx.x, nctas = a.ctas;
    __shared__ int s_abort;
    __shared__ uint32_t s_epoch;
    if (tid == 0) s_abort = 0;
    trace_begin(cv, a.flags, cta);
    announce_plan(cv, a.plan_word, cta);
    const uint32_t epoch = load_call_word(cv, kCallBarEpoch, &s_epoch);  // barrier epochs used before this call
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;

    const bool symmetric = (a.flags & kFlagSymmetric) != 0;
    const bool aligned = (a.flags & kFlagVecOk) != 0;  // per rank: only the staging copies look at it
    const uint32_t parity = (epoch >> 1) & 1u;
    const uint64_t total_vec = a.count / VEC;
    const float scale = a.ep.scale;
    const bool scaled = scale != 1.0f;

    // Heap offsets of the data the switch reads and (two-shot) writes.
    char* heap = cv.heap[r];
    const uint64_t stage_off = cv.lay.nvls_off + static_cast<uint64_t>(parity) * cv.lay.nvls_cap;
    const uint64_t in_off = symmetric ? static_cast<uint64_t>(static_cast<const char*>(a.send) - heap) : stage_off;
    const uint64_t out_off = symmetric ? static_cast<uint64_t>(static_cast<char*>(a.recv) - heap) : stage_off;
    const char* send = static_cast<const char*>(a.send);
    char* recv = static_cast<char*>(a.recv);

    if constexpr (!TWO_SHOT) {
        const uint64_t per = (total_vec + nctas - 1) / nctas;
        const uint64_t vb = min(total_vec, cta * per), ve = min(total_vec, vb + per);
        if (!symmetric) copy16<T>(heap + stage_off, send, vb, ve, aligned);
        if (!cta_barrier_all_ranks(cv, cta, epoch + 1, deadline, &s_abort)) return;
        const char* mc_in = cv.mc_heap + in_off;
        if (a.stages == 8) reduce_range<T, 8, false>(mc_in, recv, vb, ve, scale, scaled, aligned);
        else reduce_range<T, 4, false>(mc_in, recv, vb, ve, scale, scaled, aligned);
        // In-place user buffers may be overwritten by their owner right after this
        // kernel, so nobody leaves before everybody has read.  Staged input sits in
        // the half of the staging region that is not touched again before every
        // rank has passed the first barrier of the next call.
        if (symmetric) cta_barrier_all_ranks(cv, cta, epoch + 2, deadline, &s_abort);
    } else {
        const uint64_t shard_vec = a.shard_elems / VEC;
        const uint64_t per = (shard_vec + nctas - 1) / nctas;
        // Slice c of shard q, clipped to the message.
        auto slice = [&](int q, uint64_t* vb, uint64_t* ve) {
            uint64_t b = static_cast<uint64_t>(q) * shard_vec + min(shard_vec, cta * per);
            uint64_t e = min(static_cast<uint64_t>(q) * shard_vec + min(shard_vec, cta * per + per), total_vec);
            *vb = min(b, total_vec);
            *ve = max(e, *vb);
        };
        if (!symmetric) {
            for (int k = 0; k < W; ++k) {
                uint64_t vb, ve;
                slice((r + k) % W, &vb, &ve);
                copy16<T>(heap + stage_off, send, vb, ve, aligned);
            }
        }
        if (!cta_barrier_all_ranks(cv, cta, epoch + 1, deadline, &s_abort)) return;
        {
            const char* mc_in = cv.mc_heap + in_off;
            char* mc_out = cv.mc_heap + out_off;
            if (symmetric && a.slot_bytes) {
                // Interleaved blocks: the CTAs of a rank sweep its shard together (block c, c + nctas, ...)
                // instead of each streaming through a distant slice of its own.
                const uint64_t blk = a.slot_bytes / 16;
                const uint64_t sb = min(total_vec, static_cast<uint64_t>(r) * shard_vec), se = min(total_vec, sb + shard_vec);
                for (uint64_t b = sb + cta * blk; b < se; b += static_cast<uint64_t>(nctas) * blk) {
                    if (a.stages == 8) reduce_range<T, 8, true>(mc_in, mc_out, b, min(se, b + blk), scale, scaled);
                    else reduce_range<T, 4, true>(mc_in, mc_out, b, min(se, b + blk), scale, scaled);
                }
            } else {
                uint64_t vb, ve;
                slice(r, &vb, &ve);
                if (a.stages == 8) reduce_range<T, 8, true>(mc_in, mc_out, vb, ve, scale, scaled);
                else reduce_range<T, 4, true>(mc_in, mc_out, vb, ve, scale, scaled);
            }
        }
        if (!cta_barrier_all_ranks(cv, cta, epoch + 2, deadline, &s_abort)) return;
        if (!symmetric) {
            for (int k = 0; k < W; ++k) {
                uint64_t vb, ve;
                slice((r + k) % W, &vb, &ve);
                copy16<T>(recv, heap + stage_off, vb, ve, aligned);
            }
        }
    }
    finish_call(cv, 2, kCallBarEpoch, 2, nctas, a.flags);
}

template <typename T>
const void* pick_nvls(bool two_shot) {
    return two_shot ? (const void*)nvls_kernel<T, true> : (const void*)nvls_kernel<T, false>;
}

}  // namespace

const void* NvlsKernelFor(Dtype dt, int /*world*/, bool two_shot) {
    switch (dt) {
        case Dtype::FP32: return pick_nvls<float>(two_shot);
        case Dtype::FP16: return pick_nvls<__half>(two_shot);
        case Dtype::BF16: return pick_nvls<__nv_bfloat16>(two_shot);
    }
    return nullptr;
}

}  // namespace yali
