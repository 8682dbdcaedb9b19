// Stream: the two-shot, bandwidth-oriented all-reduce for 2..8 ranks
// (reduce-scatter + all-gather) over a lane-partitioned, bounded ring of slots
// with sequence-number flow control.  ONE launch per rank; a lane is one CTA.
//
// The message is cut into `world` contiguous shards (rank q owns shard q) and
// every shard into pieces of one slot.  Lane l handles pieces l, l+L, l+2L, ...
// For its i-th piece a lane runs three stages, software-pipelined one step apart:
//   A  push this rank's part of every peer's shard piece into that peer's
//      reduce-scatter slot (remote stores), then publish rs_seq = base+i+1;
//   B  wait for the N-1 incoming reduce-scatter slots, sum them with the local
//      part in fp32 in rank order, apply the epilogue, store the result locally
//      and push it into every peer's all-gather slot (or straight into the
//      peer's output when that is peer-addressable), publish ag_seq = base+i+1;
//   C  wait for the N-1 incoming all-gather slots, copy them to the output and
//      return a credit (credit = base+i+1) to their producers.
// A producer reuses slot i % kRingCap only after every peer's credit for
// iteration i-kRingCap arrived.  All counters are monotone across calls, so
// nothing is reset between calls and back-to-back calls need no host sync.
//
// Parity: allreduce_persistent (src/kernels/stream.cuh:71-165) + entry
// (src/kernels/stream.cu:35-111) + ring helpers (src/kernels/ring.cuh:78-138):
// a 2-GPU one-shot exchange, one launch per lane per GPU on its own stream, ring
// as large as the message, remote polling of the peer's gating word, unbounded
// spins.  Reduce-scatter-only and all-gather-only modes are new.
#include "coll_common.cuh"
#include "launch.h"

namespace yali {

namespace {

template <int WORLD>
__device__ __forceinline__ int world_of(const CommView& cv) {
    return WORLD ? WORLD : cv.world;
}

// Copies n elements of T (dst, src equally aligned to 16 bytes when `vec`).
template <typename T>
__device__ __forceinline__ void copy_elems(T* dst, const T* src, uint64_t n, bool vec) {
    constexpr int VEC = TypeTraits<T>::kVec;
    const int tid = threadIdx.x, nt = blockDim.x;
    uint64_t done = 0;
    if (vec) {
        const uint64_t nv = n / VEC;
        char* d = reinterpret_cast<char*>(dst);
        const char* s = reinterpret_cast<const char*>(src);
        uint64_t v = tid;
        for (; v + 3ull * nt < nv; v += 4ull * nt) {
            uint4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) x[u] = ptx::ld_cg_v4(s + (v + u * nt) * 16);
#pragma unroll
            for (int u = 0; u < 4; ++u) ptx::st_v4(d + (v + u * nt) * 16, x[u]);
        }
        for (; v < nv; v += nt) ptx::st_v4(d + v * 16, ptx::ld_cg_v4(s + v * 16));
        done = nv * VEC;
    }
    for (uint64_t e = done + tid; e < n; e += nt) dst[e] = __ldcg(src + e);
}

template <typename Tin, typename Tout, int WORLD>
__device__ __forceinline__ void stream_body(const CollArgs& a, uint32_t lane) {
    constexpr int VEC = TypeTraits<Tin>::kVec;
    constexpr uint32_t kElemBytes = sizeof(Tin) > sizeof(Tout) ? sizeof(Tin) : sizeof(Tout);
    constexpr int kMaxW = WORLD ? WORLD : kMaxRanks;
    if (a.flags & kFlagSkipRank) return;
    const CommView& cv = a.cv;
    const int W = world_of<WORLD>(cv), r = cv.rank;
    const int tid = threadIdx.x, nt = blockDim.x;
    __shared__ int s_abort;
    __shared__ uint32_t s_seq;
    if (tid == 0) s_abort = 0;
    trace_begin(cv, a.flags, lane);
    announce_plan(cv, a.plan_word, lane);
    const uint32_t seq_base = load_call_word(cv, kCallStreamSeq, &s_seq);  // sequence numbers used before this call
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;

    const bool vec = (a.flags & kFlagVecOk) != 0;
    const bool direct = (a.flags & kFlagDirectAg) != 0;
    const bool rs_only = (a.flags & kFlagReduceScatterOnly) != 0;
    const bool ag_only = (a.flags & kFlagAllGatherOnly) != 0;
    const uint32_t nlanes = a.ctas;
    const uint64_t shard = a.shard_elems;
    const uint64_t piece = a.slot_bytes / kElemBytes;
    const uint64_t n_pieces = (shard + piece - 1) / piece;
    const uint32_t n_it = lane < n_pieces ? static_cast<uint32_t>((n_pieces - lane + nlanes - 1) / nlanes) : 0u;
    const uint32_t rs_word = kRsSeqOff + lane * kMaxRanks;
    const uint32_t ag_word = kAgSeqOff + lane * kMaxRanks;
    const uint32_t cr_word = kCreditOff + lane * kMaxRanks;

    // In the full all-reduce, send and recv hold `count` elements.  Reduce-scatter
    // only: recv holds this rank's shard.  All-gather only: send holds this rank's shard.
    const Tin* send = static_cast<const Tin*>(a.send);
    Tout* recv = static_cast<Tout*>(a.recv);
    const EpiScale epi(a.ep);

    // Element range of iteration `it` inside shard q, clipped to the message.
    auto piece_range = [&](int q, uint32_t it, uint64_t* eb, uint64_t* ee) {
        const uint64_t g = lane + static_cast<uint64_t>(it) * nlanes;
        uint64_t b = static_cast<uint64_t>(q) * shard + g * piece;
        uint64_t e = min(b + piece, static_cast<uint64_t>(q + 1) * shard);
        *eb = min(b, a.count);
        *ee = min(e, a.count);
    };

    for (uint32_t step = 0; step < n_it + 2; ++step) {
        // ---------------- stage A: reduce-scatter push of iteration `step`
        if (step < n_it && !ag_only) {
            const uint32_t i = step, slot = i % kRingCap;
            if (i >= kRingCap) {
                if (!wait_peers(cv, cr_word, seq_base + (i - kRingCap) + 1, deadline, kSiteStreamCredit, lane,
                                &s_abort))
                    return;
            }
#pragma unroll
            for (int k = 1; k < kMaxW; ++k) {
                if (k < W) {
                    const int p = (r + k) % W;
                    uint64_t eb, ee;
                    piece_range(p, i, &eb, &ee);
                    copy_elems<Tin>(reinterpret_cast<Tin*>(ring_slot(cv, p, r, lane, slot, 0, a.slot_bytes)),
                                    send + eb, ee - eb, vec);
                }
            }
            __syncthreads();
            signal_peers(cv, rs_word, seq_base + i + 1);
        }
        // ---------------- stage B: reduce iteration `step-1`, all-gather push
        if (step >= 1 && step - 1 < n_it) {
            const uint32_t i = step - 1, slot = i % kRingCap;
            if (!ag_only) {
                if (!wait_peers(cv, rs_word, seq_base + i + 1, deadline, kSiteStreamRs, lane, &s_abort)) return;
            } else if (i >= kRingCap && !direct) {
                if (!wait_peers(cv, cr_word, seq_base + (i - kRingCap) + 1, deadline, kSiteStreamCredit, lane,
                                &s_abort))
                    return;
            }
            uint64_t eb, ee;
            piece_range(r, i, &eb, &ee);
            const uint64_t n = ee - eb;
            const uint64_t shard_base = static_cast<uint64_t>(r) * shard;
            // Inputs in rank order; own part comes from the send buffer.
            const Tin* own = ag_only ? send + (eb - shard_base) : send + eb;
            const Tin* in[kMaxW];
#pragma unroll
            for (int q = 0; q < kMaxW; ++q) {
                if (q >= W) in[q] = nullptr;
                else if (q == r) in[q] = own;
                else in[q] = reinterpret_cast<const Tin*>(ring_slot(cv, r, q, lane, slot, 0, a.slot_bytes));
            }
            // Outputs: local, then every peer (slot or direct).
            Tout* out_local = rs_only ? recv + (eb - shard_base) : recv + eb;
            Tout* out_peer[kMaxW];
#pragma unroll
            for (int k = 1; k < kMaxW; ++k) {
                out_peer[k] = nullptr;
                if (k < W && !rs_only) {
                    const int p = (r + k) % W;
                    out_peer[k] = direct ? static_cast<Tout*>(a.peer_recv[p]) + eb
                                         : reinterpret_cast<Tout*>(ring_slot(cv, p, r, lane, slot, 1, a.slot_bytes));
                }
            }
            const uint64_t nv = vec ? n / VEC : 0;
            for (uint64_t v = tid; v < nv; v += nt) {
                float f[VEC];
#pragma unroll
                for (int j = 0; j < VEC; ++j) f[j] = 0.f;
                if (ag_only) {
                    accumulate<Tin>(f, ptx::ld_cg_v4(own + v * VEC));
                } else {
                    uint4 x[kMaxW];
#pragma unroll
                    for (int q = 0; q < kMaxW; ++q)
                        if (q < W) x[q] = ptx::ld_cg_v4(in[q] + v * VEC);
#pragma unroll
                    for (int q = 0; q < kMaxW; ++q)
                        if (q < W) accumulate<Tin>(f, x[q]);
                }
#pragma unroll
                for (int j = 0; j < VEC; ++j) f[j] = epi(f[j]);
                store_lanes<Tout, VEC>(out_local + v * VEC, f);
#pragma unroll
                for (int k = 1; k < kMaxW; ++k)
                    if (k < W && !rs_only) store_lanes<Tout, VEC>(out_peer[k] + v * VEC, f);
            }
            for (uint64_t e = nv * VEC + tid; e < n; e += nt) {
                float s = 0.f;
                if (ag_only) {
                    s = to_f32<Tin>(__ldcg(own + e));
                } else {
#pragma unroll
                    for (int q = 0; q < kMaxW; ++q)
                        if (q < W) s += to_f32<Tin>(__ldcg(in[q] + e));
                }
                const Tout o = from_f32<Tout>(epi(s));
                out_local[e] = o;
#pragma unroll
                for (int k = 1; k < kMaxW; ++k)
                    if (k < W && !rs_only) out_peer[k][e] = o;
            }
            __syncthreads();
            if (!rs_only) signal_peers(cv, ag_word, seq_base + i + 1);
            if ((direct || rs_only) && !ag_only) signal_peers(cv, cr_word, seq_base + i + 1);
        }
        // ---------------- stage C: all-gather consume of iteration `step-2`
        if (!direct && !rs_only && step >= 2 && step - 2 < n_it) {
            const uint32_t i = step - 2, slot = i % kRingCap;
            if (!wait_peers(cv, ag_word, seq_base + i + 1, deadline, kSiteStreamAg, lane, &s_abort)) return;
#pragma unroll
            for (int k = 1; k < kMaxW; ++k) {
                if (k < W) {
                    const int s = (r + k) % W;
                    uint64_t eb, ee;
                    piece_range(s, i, &eb, &ee);
                    copy_elems<Tout>(recv + eb,
                                     reinterpret_cast<const Tout*>(ring_slot(cv, r, s, lane, slot, 1, a.slot_bytes)),
                                     ee - eb, vec);
                }
            }
            __syncthreads();
            signal_peers(cv, cr_word, seq_base + i + 1);
        }
    }
    // Direct all-gather: peers wrote into this rank's output; leave only when all of it landed.
    if (direct && !rs_only && n_it > 0) {
        if (!wait_peers(cv, ag_word, seq_base + n_it, deadline, kSiteStreamDrain, lane, &s_abort)) return;
    }
    // In the full all-reduce a rank can only finish after every peer has read all slots this
    // rank filled (its own completion depends on their results).  The half collectives lack
    // that dependency, so they drain the credits before leaving; the next call may then
    // reuse the slots at once.
    if ((rs_only || (ag_only && !direct)) && n_it > 0) {
        if (!wait_peers(cv, cr_word, seq_base + n_it, deadline, kSiteStreamDrain, lane, &s_abort)) return;
    }
    // The next call continues after the largest sequence number any lane can have used.
    finish_call(cv, 1, kCallStreamSeq, static_cast<uint32_t>((n_pieces + nlanes - 1) / nlanes), nlanes, a.flags);
}

template <typename Tin, typename Tout, int WORLD>
__global__ void __launch_bounds__(kStreamThreads, 2) stream_kernel(const __grid_constant__ CollArgs a) {
    stream_body<Tin, Tout, WORLD>(a, blockIdx.x);
}
template <typename Tin, typename Tout, int WORLD>
__global__ void __launch_bounds__(kStreamThreads, 2) stream_kernel_emu(const __grid_constant__ EmuArgs e) {
    stream_body<Tin, Tout, WORLD>(e.r[blockIdx.y], blockIdx.x);
}

template <typename Tin, typename Tout>
const void* pick_stream(int world, bool emu) {
    switch (world) {
        case 2: return emu ? (const void*)stream_kernel_emu<Tin, Tout, 2> : (const void*)stream_kernel<Tin, Tout, 2>;
        case 4: return emu ? (const void*)stream_kernel_emu<Tin, Tout, 4> : (const void*)stream_kernel<Tin, Tout, 4>;
        case 8: return emu ? (const void*)stream_kernel_emu<Tin, Tout, 8> : (const void*)stream_kernel<Tin, Tout, 8>;
        default: return emu ? (const void*)stream_kernel_emu<Tin, Tout, 0> : (const void*)stream_kernel<Tin, Tout, 0>;
    }
}

}  // namespace

const void* StreamKernelFor(Dtype in, Dtype out, int epilogue, int world, bool emu) {
    if (epilogue == kEpiResidualRmsNorm) return nullptr;  // row-wise epilogues use the dedicated row kernel
    using bf16 = __nv_bfloat16;
    if (in == Dtype::FP32 && out == Dtype::FP32) return pick_stream<float, float>(world, emu);
    if (in == Dtype::FP16 && out == Dtype::FP16) return pick_stream<__half, __half>(world, emu);
    if (in == Dtype::BF16 && out == Dtype::BF16) return pick_stream<bf16, bf16>(world, emu);
    if (in == Dtype::FP32 && out == Dtype::BF16) return pick_stream<float, bf16>(world, emu);
    if (in == Dtype::FP32 && out == Dtype::FP16) return pick_stream<float, __half>(world, emu);
    if (in == Dtype::BF16 && out == Dtype::FP32) return pick_stream<bf16, float>(world, emu);
    if (in == Dtype::FP16 && out == Dtype::FP32) return pick_stream<__half, float>(world, emu);
    return nullptr;
}

}  // namespace yali
