// Pipelined direct all-reduce for buffers that every rank can address (one process
// driving all GPUs, or buffers from the symmetric heap): no staging copy, no flag
// per piece.  Each CTA runs a multi-stage asynchronous prefetch pipeline:
//
//   warp 0 (one thread)  issues cp.async.bulk copies (TMA, per CTA, no multicast) of
//                        the next chunks of EVERY rank's input (own memory and the
//                        peers' memory over NVLink) into a ring of shared-memory
//                        stages; each stage completes on an mbarrier that counts the
//                        bytes of its W sources;
//   warps 1..8           wait for a full stage, add the W copies in fp32 in rank
//                        order, apply the epilogue and store the result, then hand
//                        the stage back through a second mbarrier.
//
// Two forms share the body:
//   one-shot pull (kFlagPullOneShot)  every rank pulls and sums the whole message and
//                        writes only its own output: (W-1)*S bytes arrive per rank,
//                        nothing is pushed, so a call ends one link trip after the
//                        last load (the latency path when inputs are addressable);
//   two-shot direct      rank r pulls and sums only shard r (reduce-scatter) and
//                        stores the sums into every rank's output (all-gather by
//                        remote stores): 2(W-1)/W*S bytes per rank and direction, safe
//                        in place because every element is read and written by
//                        exactly one CTA of one rank.
// Cross-rank synchronisation is two bounded per-CTA barriers: before the first peer
// load (the peers' inputs are final and their outputs may be overwritten once their
// kernel runs) and after the last access (peers have stopped reading this rank's
// input and their stores into this rank's output are visible).
//
// Parity: yali::FlashKernel (src/all_reduce/flash.cuh:81-183) prefetches the peer's
// buffer through three cp.async stages on sm_80/90 and falls back to synchronous
// loads on sm_100; it handles two GPUs, has no cross-GPU synchronisation and is not
// safe in place.  The reference's bandwidth kernel (src/kernels/stream.cuh:71-165)
// stages everything through ring slots in the peer's memory.
#include "coll_common.cuh"
#include "launch.h"

namespace yali {

namespace {

constexpr int kConsumerWarps = kDirectThreads / 32 - 1;
constexpr int kConsumerThreads = kConsumerWarps * 32;

template <typename Tin, typename Tout, int WORLD, bool ONE_SHOT>
__device__ __forceinline__ void direct_body(const CollArgs& a, uint32_t cta) {
    constexpr int VEC = TypeTraits<Tin>::kVec;
    constexpr int kMaxW = WORLD ? WORLD : kMaxRanks;
    if (a.flags & kFlagSkipRank) return;
    const CommView& cv = a.cv;
    const int W = WORLD ? WORLD : cv.world, r = cv.rank;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t nctas = a.ctas, stages = a.stages;

    extern __shared__ __align__(128) uint8_t dsmem[];  // [stages][W sources][slot_bytes]
    __shared__ __align__(8) uint64_t full_bar[kDirectMaxStages], empty_bar[kDirectMaxStages];
    __shared__ int s_abort;
    __shared__ uint32_t s_epoch;

    trace_begin(cv, a.flags, cta);
    announce_plan(cv, a.plan_word, cta);
    if (tid == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < stages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], kConsumerWarps);
        }
        ptx::mbar_fence_init();
    }
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
    const uint32_t epoch = load_call_word(cv, kCallBarEpoch, &s_epoch);  // barrier epochs used before this call

    // Whole 16-byte vectors go through the pipeline; the last count % VEC elements are handled
    // with scalar peer loads by one CTA.
    const uint64_t nvec_total = a.count / VEC;
    const uint64_t chunk_vec = a.slot_bytes / 16;
    uint64_t range_vb, range_ve;
    if (ONE_SHOT) {
        range_vb = 0;
        range_ve = nvec_total;
    } else {
        const uint64_t shard_vec = a.shard_elems / VEC;  // shard_elems is a multiple of 16 elements
        range_vb = min(nvec_total, static_cast<uint64_t>(r) * shard_vec);
        range_ve = min(nvec_total, range_vb + shard_vec);
    }
    const uint64_t n_chunks = (range_ve - range_vb + chunk_vec - 1) / chunk_vec;

    // Nobody touches a peer's memory before that peer's kernel runs.  On a timeout nothing is in
    // flight yet and the CTA simply leaves.
    if (!cta_barrier_all_ranks(cv, cta, epoch + 1, deadline, &s_abort)) return;

    volatile int* abort_flag = &s_abort;
    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            // The barrier's acquire ordered the peers' earlier (generic-proxy) writes before this
            // thread; the bulk copies below read through the async proxy.
            ptx::fence_proxy_async();
            uint32_t it = 0;
            for (uint64_t j = cta; j < n_chunks; j += nctas, ++it) {
                const uint32_t s = it % stages;
                if (!mbar_wait_deadline(&empty_bar[s], ((it / stages) & 1u) ^ 1u, deadline, abort_flag)) {
                    if (!*abort_flag) report_timeout(cv, kSiteMbar, r, cta, 1, it);
                    *abort_flag = 1;
                    break;
                }
                const uint64_t vb = range_vb + j * chunk_vec;
                const uint32_t bytes = static_cast<uint32_t>(min(chunk_vec, range_ve - vb)) * 16u;
                ptx::mbar_expect_tx(&full_bar[s], bytes * static_cast<uint32_t>(W));
                uint8_t* stage = dsmem + static_cast<size_t>(s) * W * a.slot_bytes;
#pragma unroll
                for (int k = 0; k < kMaxW; ++k) {
                    if (k < W) {
                        const int q = (r + k) % W;  // own memory first, then the right-hand neighbour
                        ptx::bulk_g2s(stage + static_cast<size_t>(q) * a.slot_bytes,
                                      static_cast<const char*>(a.peer_send[q]) + vb * 16, bytes, &full_bar[s]);
                    }
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- consumers
        const int ctid = tid - 32;
        const EpiScale epi(a.ep);
        Tout* out_local = static_cast<Tout*>(a.recv);
        Tout* out_peer[kMaxW];
#pragma unroll
        for (int k = 1; k < kMaxW; ++k)
            out_peer[k] = (!ONE_SHOT && k < W) ? static_cast<Tout*>(a.peer_recv[(r + k) % W]) : nullptr;

        // Scalar remainder (fewer than VEC elements).  One-shot: every rank sums it for itself;
        // two-shot: the rank whose shard contains it sums it for everybody.
        const uint64_t tail_b = nvec_total * VEC;
        if (cta == 0 && tail_b + ctid < a.count && ctid < VEC) {
            bool mine = true;
            if constexpr (!ONE_SHOT) mine = static_cast<int>(tail_b / a.shard_elems) == r;
            if (mine) {
                const uint64_t e = tail_b + ctid;
                float sum = 0.f;
#pragma unroll
                for (int q = 0; q < kMaxW; ++q)
                    if (q < W) sum += to_f32<Tin>(__ldcg(static_cast<const Tin*>(a.peer_send[q]) + e));
                const Tout o = from_f32<Tout>(epi(sum));
                out_local[e] = o;
#pragma unroll
                for (int k = 1; k < kMaxW; ++k)
                    if (!ONE_SHOT && k < W) out_peer[k][e] = o;
            }
        }

        uint32_t it = 0;
        for (uint64_t j = cta; j < n_chunks; j += nctas, ++it) {
            const uint32_t s = it % stages;
            if (!mbar_wait_deadline(&full_bar[s], (it / stages) & 1u, deadline, abort_flag)) {
                if (lane == 0 && !*abort_flag) report_timeout(cv, kSiteMbar, r, cta, 2, it);
                *abort_flag = 1;
                break;
            }
            const uint64_t vb = range_vb + j * chunk_vec;
            const uint32_t nv = static_cast<uint32_t>(min(chunk_vec, range_ve - vb));
            const uint8_t* stage = dsmem + static_cast<size_t>(s) * W * a.slot_bytes;
            for (uint32_t v = ctid; v < nv; v += kConsumerThreads) {
                float f[VEC];
#pragma unroll
                for (int i = 0; i < VEC; ++i) f[i] = 0.f;
#pragma unroll
                for (int q = 0; q < kMaxW; ++q)
                    if (q < W)
                        accumulate<Tin>(f, *reinterpret_cast<const uint4*>(stage + static_cast<size_t>(q) * a.slot_bytes +
                                                                           static_cast<size_t>(v) * 16));
#pragma unroll
                for (int i = 0; i < VEC; ++i) f[i] = epi(f[i]);
                const uint64_t e = (vb + v) * VEC;
                store_lanes<Tout, VEC>(out_local + e, f);
#pragma unroll
                for (int k = 1; k < kMaxW; ++k)
                    if (!ONE_SHOT && k < W) store_lanes<Tout, VEC>(out_peer[k] + e, f);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[s]);
        }
    }
    // Every stage that was filled has been consumed here (a consumer only leaves its loop early
    // after a wait that ran out), so no bulk copy is in flight past this point.
    __syncthreads();
    if (s_abort) return;
    // Peers have read this rank's input and their stores into this rank's output are visible.
    if (!cta_barrier_all_ranks(cv, cta, epoch + 2, deadline, &s_abort)) return;
    finish_call(cv, 2, kCallBarEpoch, 2, nctas, a.flags);
}

template <typename Tin, typename Tout, int WORLD, bool ONE_SHOT>
__global__ void __launch_bounds__(kDirectThreads, 2) direct_kernel(const __grid_constant__ CollArgs a) {
    direct_body<Tin, Tout, WORLD, ONE_SHOT>(a, blockIdx.x);
}
template <typename Tin, typename Tout, int WORLD, bool ONE_SHOT>
__global__ void __launch_bounds__(kDirectThreads, 2) direct_kernel_emu(const __grid_constant__ EmuArgs e) {
    direct_body<Tin, Tout, WORLD, ONE_SHOT>(e.r[blockIdx.y], blockIdx.x);
}

template <typename Tin, typename Tout, bool ONE_SHOT>
const void* pick_direct(int world, bool emu) {
    switch (world) {
        case 2:
            return emu ? (const void*)direct_kernel_emu<Tin, Tout, 2, ONE_SHOT>
                       : (const void*)direct_kernel<Tin, Tout, 2, ONE_SHOT>;
        case 4:
            return emu ? (const void*)direct_kernel_emu<Tin, Tout, 4, ONE_SHOT>
                       : (const void*)direct_kernel<Tin, Tout, 4, ONE_SHOT>;
        case 8:
            return emu ? (const void*)direct_kernel_emu<Tin, Tout, 8, ONE_SHOT>
                       : (const void*)direct_kernel<Tin, Tout, 8, ONE_SHOT>;
        default:
            return emu ? (const void*)direct_kernel_emu<Tin, Tout, 0, ONE_SHOT>
                       : (const void*)direct_kernel<Tin, Tout, 0, ONE_SHOT>;
    }
}
template <typename Tin, typename Tout>
const void* pick_direct2(int world, bool one_shot, bool emu) {
    return one_shot ? pick_direct<Tin, Tout, true>(world, emu) : pick_direct<Tin, Tout, false>(world, emu);
}

}  // namespace

const void* DirectKernelFor(Dtype in, Dtype out, int world, bool one_shot, bool emu) {
    using bf16 = __nv_bfloat16;
    if (in == Dtype::FP32 && out == Dtype::FP32) return pick_direct2<float, float>(world, one_shot, emu);
    if (in == Dtype::FP16 && out == Dtype::FP16) return pick_direct2<__half, __half>(world, one_shot, emu);
    if (in == Dtype::BF16 && out == Dtype::BF16) return pick_direct2<bf16, bf16>(world, one_shot, emu);
    if (in == Dtype::FP32 && out == Dtype::BF16) return pick_direct2<float, bf16>(world, one_shot, emu);
    if (in == Dtype::FP32 && out == Dtype::FP16) return pick_direct2<float, __half>(world, one_shot, emu);
    if (in == Dtype::BF16 && out == Dtype::FP32) return pick_direct2<bf16, float>(world, one_shot, emu);
    if (in == Dtype::FP16 && out == Dtype::FP32) return pick_direct2<__half, float>(world, one_shot, emu);
    return nullptr;
}

}  // namespace yali
