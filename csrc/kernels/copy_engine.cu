// Kernels of the copy-engine all-reduce (ops/copy_engine.cc): the payload crosses NVLink in
// cudaMemcpyAsync copies issued by the host (the copy engines reach 774 GB/s per direction with
// both directions busy on this machine, SM- or TMA-issued traffic 665-707), and these kernels
// do what is left: tell the peers where this rank is (flags in the peers' heaps, written with
// release stores), wait for the peers (bounded, with the usual timeout record), and add a chunk
// of staged copies to this rank's own data.
//
// Flag words (layout.h): kCeEnterOff + src   = number of the copy-engine call `src` has entered,
//                        kCePulledOff + src  = (call << 8) | chunks `src` has copied out of this rank's input,
//                        kCeDoneOff + src    = number of the call `src` has finished with this rank
//                                              (its reads of this rank's input and its writes into this rank's output).
// The call number is a counter in this rank's own heap that the last kernel of a call advances, so the
// whole sequence can be replayed from a CUDA graph.
//
// Parity: none in the reference (its kernels move all data with SM loads and stores).
#include "coll_common.cuh"
#include "copy_engine.h"

namespace yali {

namespace {

__device__ __forceinline__ uint32_t ce_call_number(const CommView& cv) {
    return *reinterpret_cast<volatile uint32_t*>(flag_word(cv, cv.rank, kCallCeCalls)) + 1u;
}

// First kernel of a call on the caller's stream: everything queued before the call has finished,
// so this rank's input is final and its output may be written.
__global__ void ce_enter_kernel(CommView cv, uint32_t plan_word, uint32_t flags) {
    const int q = threadIdx.x;
    trace_begin(cv, flags, 0);
    announce_plan(cv, plan_word, 0);
    const uint32_t n = ce_call_number(cv);
    if (q < cv.world && q != cv.rank) ptx::st_release_sys(flag_word(cv, q, kCeEnterOff + cv.rank), n);
}

// Waits until every rank of `mask` has written this call's number at word_base + rank.
__global__ void ce_wait_kernel(CommView cv, uint32_t word_base, uint32_t mask, uint32_t site) {
    const int q = threadIdx.x;
    const uint32_t n = ce_call_number(cv);
    if (q < cv.world && q != cv.rank && (mask >> q & 1u)) {
        const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
        uint32_t seen;
        if (!ptx::wait_flag_reached(flag_word(cv, cv.rank, word_base + q), n, deadline, &seen))
            report_timeout(cv, site, q, 0, n, seen);
    }
}

// After the last copy into rank `peer`: this rank is finished with `peer` for this call.
__global__ void ce_done_kernel(CommView cv, int peer) {
    if (threadIdx.x == 0) ptx::st_release_sys(flag_word(cv, peer, kCeDoneOff + cv.rank), ce_call_number(cv));
}

// Last kernel of a call on the caller's stream.  One-shot: wait until every peer has copied all
// `chunks` chunks out of this rank's input (the caller may overwrite it afterwards).  Two-shot: wait
// for every peer's "done".  Then advance the call number.
__global__ void ce_exit_kernel(CommView cv, uint32_t chunks, uint32_t one_shot, uint32_t flags) {
    const int q = threadIdx.x;
    const uint32_t n = ce_call_number(cv);
    if (q < cv.world && q != cv.rank) {
        const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
        const uint32_t word = (one_shot ? kCePulledOff : kCeDoneOff) + q;
        const uint32_t wanted = one_shot ? ((n << 8) | chunks) : n;
        uint32_t seen;
        if (!ptx::wait_flag_reached(flag_word(cv, cv.rank, word), wanted, deadline, &seen))
            report_timeout(cv, kSiteCeExit, q, 0, wanted, seen);
    }
    __syncthreads();
    if (q == 0) {
        advance_call_word(cv, kCallCeCalls, 1);
        trace_end(cv, flags);
    }
}

// out[i] = sum over ranks, in rank order, of (rank == me ? in[i] : staged[slot(rank)][i]).
template <typename T>
__global__ void __launch_bounds__(kCeReduceThreads) ce_reduce_kernel(const __grid_constant__ CeReduceArgs a) {
    constexpr int VEC = 16 / sizeof(T);
    const CommView& cv = a.cv;
    const int W = cv.world, r = cv.rank;
    __shared__ int s_abort;
    if (a.announce_chunk) {
        // One-shot: chunk `announce_chunk - 1` of every peer's input has arrived in the staging buffers
        // (stream order), so the peers may overwrite it; in place, this rank overwrites its own chunk
        // only after every peer has said the same.
        const uint32_t n = ce_call_number(cv);
        const uint32_t word = (n << 8) | a.announce_chunk;
        const int q = threadIdx.x;
        if (blockIdx.x == 0 && q < W && q != r) ptx::st_release_sys(flag_word(cv, q, kCePulledOff + r), word);
        if (a.wait_pulled) {
            if (q == 0) s_abort = 0;
            __syncthreads();
            if (q < W && q != r) {
                const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
                uint32_t seen;
                if (!ptx::wait_flag_reached(flag_word(cv, r, kCePulledOff + q), word, deadline, &seen)) {
                    report_timeout(cv, kSiteCePulled, q, blockIdx.x, word, seen);
                    s_abort = 1;
                }
            }
            __syncthreads();
            if (s_abort) return;
        }
    }
    const uint64_t nvec = a.elems / VEC;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const char* in = static_cast<const char*>(a.in);
    char* out = static_cast<char*>(a.out);
    for (uint64_t v = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride * 2) {
        // Two vectors per thread and iteration: all loads first.
        const uint64_t v1 = v + stride;
        const bool two = v1 < nvec;
        uint4 x0[kMaxRanks], x1[kMaxRanks];
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q) {
            if (q < W) {
                const char* src = q == r ? in : static_cast<const char*>(a.staged[SrcSlot(q, r)]);
                x0[q] = ptx::ld_cg_v4(src + v * 16);
                if (two) x1[q] = ptx::ld_cg_v4(src + v1 * 16);
            }
        }
        float f0[VEC], f1[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) f0[i] = f1[i] = 0.f;
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q) {
            if (q < W) {
                accumulate<T>(f0, x0[q]);
                if (two) accumulate<T>(f1, x1[q]);
            }
        }
        ptx::st_v4(out + v * 16, pack16<T>(f0));
        if (two) ptx::st_v4(out + v1 * 16, pack16<T>(f1));
    }
    // Elements beyond the last whole vector (only the last chunk of a message has any).
    if (blockIdx.x == 0) {
        const T* tin = static_cast<const T*>(a.in);
        T* tout = static_cast<T*>(a.out);
        for (uint64_t e = nvec * VEC + threadIdx.x; e < a.elems; e += blockDim.x) {
            float acc = 0.f;
            for (int q = 0; q < W; ++q)
                acc += to_f32<T>(q == r ? tin[e] : static_cast<const T*>(a.staged[SrcSlot(q, r)])[e]);
            tout[e] = from_f32<T>(acc);
        }
    }
}

}  // namespace

cudaError_t CeLaunchEnter(const CommView& cv, uint32_t plan_word, uint32_t flags, cudaStream_t s) {
    ce_enter_kernel<<<1, 32, 0, s>>>(cv, plan_word, flags);
    return cudaGetLastError();
}
cudaError_t CeLaunchWaitEnter(const CommView& cv, uint32_t mask, cudaStream_t s) {
    ce_wait_kernel<<<1, 32, 0, s>>>(cv, kCeEnterOff, mask, kSiteCeEnter);
    return cudaGetLastError();
}
cudaError_t CeLaunchDone(const CommView& cv, int peer, cudaStream_t s) {
    ce_done_kernel<<<1, 32, 0, s>>>(cv, peer);
    return cudaGetLastError();
}
cudaError_t CeLaunchExit(const CommView& cv, uint32_t chunks, bool one_shot, uint32_t flags, cudaStream_t s) {
    ce_exit_kernel<<<1, 32, 0, s>>>(cv, chunks, one_shot ? 1u : 0u, flags);
    return cudaGetLastError();
}
cudaError_t CeLaunchReduce(const CeReduceArgs& a, Dtype dt, uint32_t ctas, cudaStream_t s) {
    switch (dt) {
        case Dtype::FP32: ce_reduce_kernel<float><<<ctas, kCeReduceThreads, 0, s>>>(a); break;
        case Dtype::FP16: ce_reduce_kernel<__half><<<ctas, kCeReduceThreads, 0, s>>>(a); break;
        case Dtype::BF16: ce_reduce_kernel<__nv_bfloat16><<<ctas, kCeReduceThreads, 0, s>>>(a); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace yali
