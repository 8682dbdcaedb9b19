// Flash: the one-shot, latency-oriented all-reduce for 2..8 ranks.
//
// Every CTA owns a contiguous slice of the message.  It (1) pushes its slice of
// the local input into a staging area of every peer's heap with 16-byte remote
// stores, (2) publishes one release flag per peer, (3) waits (bounded) for the
// matching flag of every peer, (4) sums own input + the N-1 staged copies in
// fp32 in rank order, applies the epilogue and stores the result.  CTA c only
// ever talks to CTA c of the other ranks, so there is no grid-wide barrier, the
// send buffer may equal the receive buffer, and user buffers never have to be
// peer-mapped.  Staging alternates between two parities per call so that a peer
// may start call k+1 while this rank still reads call k.  The call number lives in the
// rank's heap and is advanced by the last CTA of each launch, so launches carry no per-call
// state and can be replayed from a CUDA graph.
//
// Parity: yali::FlashKernel (src/all_reduce/flash.cuh:42-184) is the 2-GPU
// counterpart: it pulls the peer's buffer with cp.async (sync loads on sm_100)
// and has no cross-GPU synchronisation at all; its launcher is
// src/all_reduce/kernels.cuh:41-55.  The epilogues (scale+cast, residual +
// RMSNorm) have no counterpart in the reference.
#include "coll_common.cuh"
#include "launch.h"

namespace yali {

namespace {

constexpr int kUnroll = 4;

template <int WORLD>
__device__ __forceinline__ int world_of(const CommView& cv) {
    return WORLD ? WORLD : cv.world;
}

// Pushes elements [vb, ve) (16-byte vectors) and [tb, te) (scalars) of `send` into
// this rank's staging area on every peer.
template <typename Tin, int WORLD>
__device__ __forceinline__ void push_slice(const CollArgs& a, uint32_t parity, uint64_t vb, uint64_t ve, uint64_t tb,
                                           uint64_t te) {
    const CommView& cv = a.cv;
    const int W = world_of<WORLD>(cv), r = cv.rank;
    const int tid = threadIdx.x, nt = blockDim.x;
    constexpr int kMaxPeers = WORLD ? WORLD - 1 : kMaxRanks - 1;
    char* dst[kMaxPeers];
#pragma unroll
    for (int k = 0; k < kMaxPeers; ++k) {
        int p = (r + 1 + k) % W;  // start with the right-hand neighbour so ranks do not gang up on one peer
        dst[k] = (k < W - 1) ? flash_stage(cv, p, r, parity) : nullptr;
    }
    const char* src = static_cast<const char*>(a.send);
    uint64_t v = vb + tid;
    for (; v + static_cast<uint64_t>(kUnroll - 1) * nt < ve; v += static_cast<uint64_t>(kUnroll) * nt) {
        uint4 x[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) x[u] = *reinterpret_cast<const uint4*>(src + (v + u * nt) * 16);
#pragma unroll
        for (int k = 0; k < kMaxPeers; ++k) {
            if (k < W - 1) {
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) ptx::st_v4(dst[k] + (v + u * nt) * 16, x[u]);
            }
        }
    }
    for (; v < ve; v += nt) {
        uint4 x = *reinterpret_cast<const uint4*>(src + v * 16);
#pragma unroll
        for (int k = 0; k < kMaxPeers; ++k)
            if (k < W - 1) ptx::st_v4(dst[k] + v * 16, x);
    }
    const Tin* s = static_cast<const Tin*>(a.send);
    for (uint64_t e = tb + tid; e < te; e += nt) {
        Tin x = s[e];
#pragma unroll
        for (int k = 0; k < kMaxPeers; ++k)
            if (k < W - 1) reinterpret_cast<Tin*>(dst[k])[e] = x;
    }
}

template <typename Tin, typename Tout, int WORLD>
__device__ __forceinline__ void flash_body(const CollArgs& a, uint32_t cta) {
    constexpr int VEC = TypeTraits<Tin>::kVec;
    if (a.flags & kFlagSkipRank) return;
    const CommView& cv = a.cv;
    const int W = world_of<WORLD>(cv), r = cv.rank;
    const int tid = threadIdx.x, nt = blockDim.x;
    __shared__ int s_abort;
    __shared__ uint32_t s_epoch;
    if (tid == 0) s_abort = 0;
    trace_begin(cv, a.flags, cta);
    announce_plan(cv, a.plan_word, cta);
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
    const uint32_t epoch = load_call_word(cv, kCallFlashEpoch, &s_epoch) + 1;  // this call's number
    const uint32_t parity = epoch & 1u;

    // Slice of this CTA: elements [eb, ee).  The boundaries depend only on `count` and the CTA
    // count, which every rank shares, never on a rank's own pointer alignment: CTA c of one
    // rank synchronises with CTA c of its peers only, so all of them must cover the same
    // elements.  Alignment (kFlagVecOk, a per-rank property) only chooses how the slice is
    // accessed: whole 16-byte vectors [vb, ve) plus a scalar remainder [tb, te), or scalars.
    const uint64_t nvec_all = (a.count + VEC - 1) / VEC;
    const uint64_t per_v = (nvec_all + a.ctas - 1) / a.ctas;
    const uint64_t eb = min(a.count, static_cast<uint64_t>(cta) * per_v * VEC), ee = min(a.count, eb + per_v * VEC);
    uint64_t vb, ve, tb, te;
    if (a.flags & kFlagVecOk) {
        ve = ee / VEC;
        vb = min(ve, (eb + VEC - 1) / VEC);  // eb is a multiple of VEC unless the slice is empty
        tb = max(ve * VEC, eb);
        te = ee;
    } else {
        vb = ve = 0;
        tb = eb;
        te = ee;
    }

    push_slice<Tin, WORLD>(a, parity, vb, ve, tb, te);
    __syncthreads();
    signal_peers(cv, kFlashFlagOff + cta * kMaxRanks, epoch);
    if (!wait_peers(cv, kFlashFlagOff + cta * kMaxRanks, epoch, deadline, kSiteFlashArrive, cta, &s_abort)) return;

    // Sum in rank order; own contribution comes from the send buffer itself.
    constexpr int kMaxW = WORLD ? WORLD : kMaxRanks;
    const char* in[kMaxW];
#pragma unroll
    for (int q = 0; q < kMaxW; ++q)
        in[q] = (q >= W) ? nullptr : (q == r ? static_cast<const char*>(a.send) : flash_stage(cv, r, q, parity));
    const EpiScale epi(a.ep);
    Tout* out = static_cast<Tout*>(a.recv);
    uint64_t v = vb + tid;
    // Two vectors per thread in flight while the inputs fit the register budget.
    for (; kMaxW <= 4 && v + nt < ve; v += 2ull * nt) {
        uint4 x0[kMaxW], x1[kMaxW];
#pragma unroll
        for (int q = 0; q < kMaxW; ++q) {
            if (q < W) {
                x0[q] = ptx::ld_cg_v4(in[q] + v * 16);
                x1[q] = ptx::ld_cg_v4(in[q] + (v + nt) * 16);
            }
        }
        float f0[VEC], f1[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) f0[i] = f1[i] = 0.f;
#pragma unroll
        for (int q = 0; q < kMaxW; ++q) {
            if (q < W) {
                accumulate<Tin>(f0, x0[q]);
                accumulate<Tin>(f1, x1[q]);
            }
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            f0[i] = epi(f0[i]);
            f1[i] = epi(f1[i]);
        }
        store_lanes<Tout, VEC>(out + v * VEC, f0);
        store_lanes<Tout, VEC>(out + (v + nt) * VEC, f1);
    }
    for (; v < ve; v += nt) {
        float f[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = 0.f;
#pragma unroll
        for (int q = 0; q < kMaxW; ++q)
            if (q < W) accumulate<Tin>(f, ptx::ld_cg_v4(in[q] + v * 16));
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = epi(f[i]);
        store_lanes<Tout, VEC>(out + v * VEC, f);
    }
    for (uint64_t e = tb + tid; e < te; e += nt) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < kMaxW; ++q)
            if (q < W) s += to_f32<Tin>(__ldcg(reinterpret_cast<const Tin*>(in[q]) + e));
        out[e] = from_f32<Tout>(epi(s));
    }
    finish_call(cv, 0, kCallFlashEpoch, 1, a.ctas, a.flags);
}

// One-shot all-reduce fused with residual-add + RMSNorm.  The message is
// [rows, hidden]; CTAs own whole rows.  Each thread keeps its part of a row in
// registers between the cross-rank sum and the normalisation.
template <typename T, int WORLD>
__device__ __forceinline__ void flash_rmsnorm_body(const CollArgs& a, uint32_t cta) {
    constexpr int VEC = TypeTraits<T>::kVec;
    constexpr int kMaxVecPerThread = 4;
    if (a.flags & kFlagSkipRank) return;
    const CommView& cv = a.cv;
    const int W = world_of<WORLD>(cv), r = cv.rank;
    const int tid = threadIdx.x, nt = blockDim.x;
    __shared__ int s_abort;
    __shared__ float s_red[32];
    __shared__ uint32_t s_epoch;
    if (tid == 0) s_abort = 0;
    trace_begin(cv, a.flags, cta);
    announce_plan(cv, a.plan_word, cta);
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
    const uint32_t epoch = load_call_word(cv, kCallFlashEpoch, &s_epoch) + 1;  // this call's number
    const uint32_t parity = epoch & 1u;

    const uint32_t H = a.ep.hidden;
    const uint32_t vec_per_row = H / VEC;
    const uint64_t rows = a.count / H;
    const uint64_t rows_per = (rows + a.ctas - 1) / a.ctas;
    const uint64_t rb = min(rows, static_cast<uint64_t>(cta) * rows_per), re = min(rows, rb + rows_per);

    push_slice<T, WORLD>(a, parity, rb * vec_per_row, re * vec_per_row, 0, 0);
    __syncthreads();
    signal_peers(cv, kFlashFlagOff + cta * kMaxRanks, epoch);
    if (!wait_peers(cv, kFlashFlagOff + cta * kMaxRanks, epoch, deadline, kSiteFlashArrive, cta, &s_abort)) return;

    constexpr int kMaxW = WORLD ? WORLD : kMaxRanks;
    const char* in[kMaxW];
#pragma unroll
    for (int q = 0; q < kMaxW; ++q)
        in[q] = (q >= W) ? nullptr : (q == r ? static_cast<const char*>(a.send) : flash_stage(cv, r, q, parity));
    const char* res = static_cast<const char*>(a.ep.residual);
    char* res_out = static_cast<char*>(a.ep.residual_out);
    const char* wgt = static_cast<const char*>(a.ep.weight);
    T* out = static_cast<T*>(a.recv);
    const float inv_h = 1.f / static_cast<float>(H);

    for (uint64_t row = rb; row < re; ++row) {
        float f[kMaxVecPerThread][VEC];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxVecPerThread; ++j) {
            const uint32_t c = tid + j * nt;
            if (c < vec_per_row) {
                const uint64_t off = (row * vec_per_row + c) * 16;
#pragma unroll
                for (int i = 0; i < VEC; ++i) f[j][i] = 0.f;
#pragma unroll
                for (int q = 0; q < kMaxW; ++q)
                    if (q < W) accumulate<T>(f[j], ptx::ld_cg_v4(in[q] + off));
                if (res) accumulate<T>(f[j], ptx::ld_cg_v4(res + off));
                if (res_out) {
                    ptx::st_v4(res_out + off, pack16<T>(f[j]));
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i) ss += f[j][i] * f[j][i];
            }
        }
        const float inv_rms = rsqrtf(block_sum(ss, s_red) * inv_h + a.ep.eps);
#pragma unroll
        for (int j = 0; j < kMaxVecPerThread; ++j) {
            const uint32_t c = tid + j * nt;
            if (c < vec_per_row) {
                float w[VEC];
#pragma unroll
                for (int i = 0; i < VEC; ++i) w[i] = 0.f;
                accumulate<T>(w, *reinterpret_cast<const uint4*>(wgt + static_cast<uint64_t>(c) * 16));
#pragma unroll
                for (int i = 0; i < VEC; ++i) f[j][i] = f[j][i] * inv_rms * w[i];
                store_lanes<T, VEC>(out + (row * vec_per_row + c) * VEC, f[j]);
            }
        }
    }
    finish_call(cv, 0, kCallFlashEpoch, 1, a.ctas, a.flags);
}

// Flag-in-data form of the one-shot all-reduce for small messages.  Every 16-byte line
// that crosses NVLink carries 8 bytes of payload and the 64-bit number of the call, split
// over its two 8-byte halves {data, call_lo} {data, call_hi}.  A receiver polls the line
// itself until both halves show this call's number, so there is no separate flag, no CTA
// barrier and no release fence between the push and the reduction: latency is one
// one-way trip.  Twice the bytes on the wire, so only small messages take this path.  Its
// staging is never written by anything else, hence stale lines always show an older call.
__device__ __forceinline__ char* ll_stage(const CommView& cv, int on_rank, int src, uint32_t parity) {
    return cv.heap[on_rank] + cv.lay.ll_off +
           (static_cast<uint64_t>(parity) * (cv.world - 1) + SrcSlot(src, on_rank)) * (2 * cv.lay.ll_cap);
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
                 : "memory");
    return v;
}

template <typename T, int WORLD>
__device__ __forceinline__ void flash_ll_body(const CollArgs& a, uint32_t cta) {
    constexpr int VEC = TypeTraits<T>::kVec;
    constexpr int kMaxW = WORLD ? WORLD : kMaxRanks;
    constexpr int kMaxPeers = kMaxW - 1;
    if (a.flags & kFlagSkipRank) return;
    const CommView& cv = a.cv;
    const int W = world_of<WORLD>(cv), r = cv.rank;
    const int tid = threadIdx.x, nt = blockDim.x;
    __shared__ uint32_t s_call[2];
    trace_begin(cv, a.flags, cta);
    announce_plan(cv, a.plan_word, cta);
    if (tid < 2)
        s_call[tid] = *reinterpret_cast<volatile uint32_t*>(flag_word(cv, r, tid == 0 ? kCallFlashEpoch : kCallFlashEpochHi));
    // The first payload vector of this thread is fetched while the call number is on its way, and kept
    // for the reduction (with one vector per thread, the common case, the input is read exactly once).
    const uint64_t nvec = a.count / VEC;  // the planner only picks this form for whole vectors
    // This rank's own buffers may be aligned to their element type only (kFlagVecOk is a per-rank
    // property here): then they are read and written element by element; the lines on the wire and
    // the CTA slices are the same either way.
    const bool aligned = (a.flags & kFlagVecOk) != 0;
    const uint64_t per = (nvec + a.ctas - 1) / a.ctas;
    const uint64_t vb = min(nvec, static_cast<uint64_t>(cta) * per), ve = min(nvec, vb + per);
    const char* src = static_cast<const char*>(a.send);
    const uint64_t v0 = vb + tid;
    uint4 x0 = make_uint4(0, 0, 0, 0);
    if (v0 < ve) x0 = aligned ? *reinterpret_cast<const uint4*>(src + v0 * 16) : load16_elems<T>(src, v0);
    __syncthreads();
    const uint32_t lo = s_call[0] + 1u;                       // this call's number (shared with the flagged form)
    const uint32_t hi = (s_call[1] + (lo == 0u ? 1u : 0u)) | 0x80000000u;  // never zero: fresh memory never matches
    const uint32_t parity = lo & 1u;
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;

    char* dst[kMaxPeers];
    const char* in[kMaxW];
#pragma unroll
    for (int k = 0; k < kMaxPeers; ++k) dst[k] = (k < W - 1) ? ll_stage(cv, (r + 1 + k) % W, r, parity) : nullptr;
#pragma unroll
    for (int q = 0; q < kMaxW; ++q) in[q] = (q < W && q != r) ? ll_stage(cv, r, q, parity) : nullptr;

    // ---- push: payload vector v becomes lines 2v and 2v+1
    for (uint64_t v = vb + tid; v < ve; v += nt) {
        const uint4 x = v == v0 ? x0 : (aligned ? *reinterpret_cast<const uint4*>(src + v * 16) : load16_elems<T>(src, v));
        const uint4 l0 = make_uint4(x.x, lo, x.y, hi), l1 = make_uint4(x.z, lo, x.w, hi);
#pragma unroll
        for (int k = 0; k < kMaxPeers; ++k) {
            if (k < W - 1) {
                ptx::st_v4(dst[k] + v * 32, l0);
                ptx::st_v4(dst[k] + v * 32 + 16, l1);
            }
        }
    }
    // ---- reduce: poll the peers' lines for the same vectors
    const EpiScale epi(a.ep);
    T* out = static_cast<T*>(a.recv);
    bool timed_out = false;
    for (uint64_t v = vb + tid; v < ve && !timed_out; v += nt) {
        float f[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = 0.f;
#pragma unroll
        for (int q = 0; q < kMaxW; ++q) {
            if (q >= W) continue;
            if (q == r) {
                accumulate<T>(f, v == v0 ? x0 : (aligned ? *reinterpret_cast<const uint4*>(src + v * 16) : load16_elems<T>(src, v)));
                continue;
            }
            uint4 l0, l1;
            uint32_t polls = 0;
            for (;;) {
                l0 = ld_volatile_v4(in[q] + v * 32);
                l1 = ld_volatile_v4(in[q] + v * 32 + 16);
                if (l0.y == lo && l0.w == hi && l1.y == lo && l1.w == hi) break;
                if ((++polls & 63u) == 0u && ptx::globaltimer() > deadline) {
                    report_timeout(cv, kSiteFlashArrive, q, cta, lo, l0.y);
                    timed_out = true;
                    break;
                }
            }
            if (timed_out) break;
            accumulate<T>(f, make_uint4(l0.x, l0.z, l1.x, l1.z));
        }
        if (timed_out) break;
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = epi(f[i]);
        if (aligned) store_lanes<T, VEC>(out + v * VEC, f);
        else store16_elems<T>(out, v, pack16<T>(f));
    }
    if (__syncthreads_or(timed_out ? 1 : 0)) return;
    if (tid == 0 && check_out_last(cv, 0, a.ctas)) {
        advance_call_word(cv, kCallFlashEpoch, 1);
        if (lo == 0u) advance_call_word(cv, kCallFlashEpochHi, 1);
        trace_end(cv, a.flags);
    }
}

// At most 128 CTAs, one per SM: no register cap (the emulated twin shares the GPU among all ranks' CTAs
// and keeps two per SM).
template <typename T, int WORLD>
__global__ void __launch_bounds__(kFlashThreads, 1) flash_ll_kernel(const __grid_constant__ CollArgs a) {
    flash_ll_body<T, WORLD>(a, blockIdx.x);
}
template <typename T, int WORLD>
__global__ void __launch_bounds__(kFlashThreads, 2) flash_ll_kernel_emu(const __grid_constant__ EmuArgs e) {
    flash_ll_body<T, WORLD>(e.r[blockIdx.y], blockIdx.x);
}
template <typename T>
const void* pick_flash_ll(int world, bool emu) {
    switch (world) {
        case 2: return emu ? (const void*)flash_ll_kernel_emu<T, 2> : (const void*)flash_ll_kernel<T, 2>;
        case 4: return emu ? (const void*)flash_ll_kernel_emu<T, 4> : (const void*)flash_ll_kernel<T, 4>;
        case 8: return emu ? (const void*)flash_ll_kernel_emu<T, 8> : (const void*)flash_ll_kernel<T, 8>;
        default: return emu ? (const void*)flash_ll_kernel_emu<T, 0> : (const void*)flash_ll_kernel<T, 0>;
    }
}

template <typename Tin, typename Tout, int WORLD>
__global__ void __launch_bounds__(kFlashThreads, 2) flash_kernel(const __grid_constant__ CollArgs a) {
    flash_body<Tin, Tout, WORLD>(a, blockIdx.x);
}
template <typename Tin, typename Tout, int WORLD>
__global__ void __launch_bounds__(kFlashThreads, 2) flash_kernel_emu(const __grid_constant__ EmuArgs e) {
    flash_body<Tin, Tout, WORLD>(e.r[blockIdx.y], blockIdx.x);
}
template <typename T, int WORLD>
__global__ void __launch_bounds__(kFlashThreads, 2) flash_rmsnorm_kernel(const __grid_constant__ CollArgs a) {
    flash_rmsnorm_body<T, WORLD>(a, blockIdx.x);
}
template <typename T, int WORLD>
__global__ void __launch_bounds__(kFlashThreads, 2) flash_rmsnorm_kernel_emu(const __grid_constant__ EmuArgs e) {
    flash_rmsnorm_body<T, WORLD>(e.r[blockIdx.y], blockIdx.x);
}

template <typename Tin, typename Tout>
const void* pick_flash(int world, bool emu) {
    switch (world) {
        case 2: return emu ? (const void*)flash_kernel_emu<Tin, Tout, 2> : (const void*)flash_kernel<Tin, Tout, 2>;
        case 4: return emu ? (const void*)flash_kernel_emu<Tin, Tout, 4> : (const void*)flash_kernel<Tin, Tout, 4>;
        case 8: return emu ? (const void*)flash_kernel_emu<Tin, Tout, 8> : (const void*)flash_kernel<Tin, Tout, 8>;
        default: return emu ? (const void*)flash_kernel_emu<Tin, Tout, 0> : (const void*)flash_kernel<Tin, Tout, 0>;
    }
}
template <typename T>
const void* pick_flash_rms(int world, bool emu) {
    switch (world) {
        case 2: return emu ? (const void*)flash_rmsnorm_kernel_emu<T, 2> : (const void*)flash_rmsnorm_kernel<T, 2>;
        case 4: return emu ? (const void*)flash_rmsnorm_kernel_emu<T, 4> : (const void*)flash_rmsnorm_kernel<T, 4>;
        case 8: return emu ? (const void*)flash_rmsnorm_kernel_emu<T, 8> : (const void*)flash_rmsnorm_kernel<T, 8>;
        default: return emu ? (const void*)flash_rmsnorm_kernel_emu<T, 0> : (const void*)flash_rmsnorm_kernel<T, 0>;
    }
}

}  // namespace

const void* FlashLLKernelFor(Dtype dt, int world, bool emu) {
    switch (dt) {
        case Dtype::FP32: return pick_flash_ll<float>(world, emu);
        case Dtype::FP16: return pick_flash_ll<__half>(world, emu);
        case Dtype::BF16: return pick_flash_ll<__nv_bfloat16>(world, emu);
    }
    return nullptr;
}

const void* FlashKernelFor(Dtype in, Dtype out, int epilogue, int world, bool emu) {
    if (epilogue == kEpiResidualRmsNorm) {
        if (in != out) return nullptr;
        switch (in) {
            case Dtype::FP32: return pick_flash_rms<float>(world, emu);
            case Dtype::FP16: return pick_flash_rms<__half>(world, emu);
            case Dtype::BF16: return pick_flash_rms<__nv_bfloat16>(world, emu);
        }
        return nullptr;
    }
    using bf16 = __nv_bfloat16;
    if (in == Dtype::FP32 && out == Dtype::FP32) return pick_flash<float, float>(world, emu);
    if (in == Dtype::FP16 && out == Dtype::FP16) return pick_flash<__half, __half>(world, emu);
    if (in == Dtype::BF16 && out == Dtype::BF16) return pick_flash<bf16, bf16>(world, emu);
    if (in == Dtype::FP32 && out == Dtype::BF16) return pick_flash<float, bf16>(world, emu);
    if (in == Dtype::FP32 && out == Dtype::FP16) return pick_flash<float, __half>(world, emu);
    if (in == Dtype::BF16 && out == Dtype::FP32) return pick_flash<bf16, float>(world, emu);
    if (in == Dtype::FP16 && out == Dtype::FP32) return pick_flash<__half, float>(world, emu);
    return nullptr;
}

}  // namespace yali
