// Device helpers shared by the collective kernels: addressing of the heap
// regions, bounded waits that record where they gave up, and the per-CTA
// cross-rank barrier.
//
// Parity: src/kernels/ring.cuh:103-128 (wait_for_credit / wait_for_slot spin
// without limit, thread 0 only).  Here one thread per peer waits, every wait has
// a deadline, and a wait that runs out records {site, rank, peer, cta, wanted,
// observed} in the rank's status block and makes the whole CTA leave normally.
#pragma once

#include "../comm/layout.h"
#include "../core/ptx.cuh"
#include "type_ops.cuh"

namespace yali {

__device__ __forceinline__ uint32_t* flag_word(const CommView& cv, int on_rank, uint32_t word) {
    return reinterpret_cast<uint32_t*>(cv.heap[on_rank] + cv.lay.flags_off) + word;
}

// One-shot staging: where source rank `src` deposits its copy on rank `on_rank`.
__device__ __forceinline__ char* flash_stage(const CommView& cv, int on_rank, int src, uint32_t parity) {
    return cv.heap[on_rank] + cv.lay.flash_off +
           (static_cast<uint64_t>(parity) * (cv.world - 1) + SrcSlot(src, on_rank)) * cv.lay.flash_cap;
}

// Two-shot ring slot on rank `on_rank` filled by `src`: which = 0 reduce-scatter, 1 all-gather.
__device__ __forceinline__ char* ring_slot(const CommView& cv, int on_rank, int src, uint32_t lane, uint32_t slot,
                                           uint32_t which, uint32_t slot_bytes) {
    uint64_t idx = ((static_cast<uint64_t>(lane) * (cv.world - 1) + SrcSlot(src, on_rank)) * kRingCap + slot) * 2 + which;
    return cv.heap[on_rank] + cv.lay.ring_off + idx * slot_bytes;
}

// Records the first wait of this rank that gave up.  The status block is pinned
// host memory (read by the host without a copy), written with plain stores; the
// election of the first reporter uses a counter in this rank's own heap.
__device__ __forceinline__ void report_timeout(const CommView& cv, uint32_t site, uint32_t peer, uint32_t cta,
                                               uint32_t wanted, uint32_t observed) {
    volatile DeviceStatus* st = cv.status;
    if (!st) return;
    uint32_t prev = atomicAdd(flag_word(cv, cv.rank, kStatusCntOff), 1u);
    if (prev == 0) {
        st->rank = cv.rank;
        st->peer = peer;
        st->cta = cta;
        st->wanted = wanted;
        st->observed = observed;
        // Which kernels the two ranks were running: a mismatch means mismatched arguments.
        st->my_plan = *reinterpret_cast<volatile uint32_t*>(flag_word(cv, cv.rank, kCallPlanWord));
        st->peer_plan = peer < static_cast<uint32_t>(cv.world) ? ptx::ld_relaxed_sys(flag_word(cv, peer, kCallPlanWord)) : 0u;
        __threadfence_system();
        st->code = site;
        __threadfence_system();
    }
}

// Threads 0..world-1 (except `rank`) each wait for the flag that peer `tid`
// writes into this rank's heap at `word_base + tid`.  Returns, on every thread of
// the CTA, whether all flags arrived.  Contains two CTA barriers.
__device__ __forceinline__ bool wait_peers(const CommView& cv, uint32_t word_base, uint32_t wanted,
                                           uint64_t deadline_ns, uint32_t site, uint32_t cta, int* s_abort) {
    const int tid = threadIdx.x;
    if (tid < cv.world && tid != cv.rank) {
        uint32_t seen;
        if (!ptx::wait_flag_reached(flag_word(cv, cv.rank, word_base + tid), wanted, deadline_ns, &seen)) {
            report_timeout(cv, site, tid, cta, wanted, seen);
            *s_abort = 1;
        }
    }
    __syncthreads();
    return *s_abort == 0;
}

// After a CTA barrier: threads 0..world-1 (except `rank`) publish `value` into
// word `word_base + rank` of every peer's flag region with release semantics, so
// that everything the CTA wrote before the barrier is visible to whoever
// acquires the flag.
__device__ __forceinline__ void signal_peers(const CommView& cv, uint32_t word_base, uint32_t value) {
    const int tid = threadIdx.x;
    if (tid < cv.world && tid != cv.rank) ptx::st_release_sys(flag_word(cv, tid, word_base + cv.rank), value);
}

// Cross-rank barrier among the CTAs with index `cta` of all ranks.
__device__ __forceinline__ bool cta_barrier_all_ranks(const CommView& cv, uint32_t cta, uint32_t epoch,
                                                      uint64_t deadline_ns, int* s_abort) {
    __syncthreads();
    signal_peers(cv, kBarOff + cta * kMaxRanks, epoch);
    return wait_peers(cv, kBarOff + cta * kMaxRanks, epoch, deadline_ns, kSiteBarrier, cta, s_abort);
}

// Reads one of this rank's call counters (layout.h, kCall*) for the whole CTA.  The value was
// written by the last CTA of the previous launch of this kind, which stream order makes visible.
// Contains a CTA barrier.
__device__ __forceinline__ uint32_t load_call_word(const CommView& cv, uint32_t word, uint32_t* s_slot) {
    if (threadIdx.x == 0) *s_slot = *reinterpret_cast<volatile uint32_t*>(flag_word(cv, cv.rank, word));
    __syncthreads();
    return *s_slot;
}

// Every CTA that finished its part of the call normally checks out here; the last one advances
// the call counter by `inc` for the next launch.  `kind` selects the check-out word.
__device__ __forceinline__ bool check_out_last(const CommView& cv, uint32_t kind, uint32_t nctas) {
    // thread 0 only
    uint32_t* done = flag_word(cv, cv.rank, kCallDoneCtas + kind);
    __threadfence();
    if (atomicAdd(done, 1u) != nctas - 1) return false;
    *reinterpret_cast<volatile uint32_t*>(done) = 0u;
    return true;
}
__device__ __forceinline__ void advance_call_word(const CommView& cv, uint32_t word, uint32_t inc) {
    volatile uint32_t* w = flag_word(cv, cv.rank, word);
    *w = *w + inc;
}
// Device-side timeline (kFlagTrace): the first CTA stamps %globaltimer when it starts, the last CTA
// to check out stamps it again and advances the ring index.  The host reads the ring after a
// synchronisation and obtains per-call device times that contain no host jitter.
// Publishes which plan this rank runs (one store by one thread per call): read by a peer that gave up
// waiting for this rank, to tell "never arrived" from "arrived in a different kernel".
__device__ __forceinline__ void announce_plan(const CommView& cv, uint32_t plan_word, uint32_t cta) {
    if (cta == 0 && threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(flag_word(cv, cv.rank, kCallPlanWord)) = plan_word;
}

__device__ __forceinline__ void trace_begin(const CommView& cv, uint32_t flags, uint32_t cta) {
    if ((flags & kFlagTrace) && cta == 0 && threadIdx.x == 0) {
        const uint32_t idx = *reinterpret_cast<volatile uint32_t*>(flag_word(cv, cv.rank, kCallTraceIdx));
        volatile uint64_t* ring = reinterpret_cast<volatile uint64_t*>(flag_word(cv, cv.rank, kTraceOff));
        ring[(idx % kTraceCap) * 2] = ptx::globaltimer();
    }
}
__device__ __forceinline__ void trace_end(const CommView& cv, uint32_t flags) {
    // thread 0 of the last CTA only
    if (flags & kFlagTrace) {
        volatile uint32_t* iw = flag_word(cv, cv.rank, kCallTraceIdx);
        const uint32_t idx = *iw;
        volatile uint64_t* ring = reinterpret_cast<volatile uint64_t*>(flag_word(cv, cv.rank, kTraceOff));
        ring[(idx % kTraceCap) * 2 + 1] = ptx::globaltimer();
        *iw = idx + 1;
    }
}
__device__ __forceinline__ void finish_call(const CommView& cv, uint32_t kind, uint32_t word, uint32_t inc,
                                            uint32_t nctas, uint32_t flags = 0) {
    if (threadIdx.x == 0 && check_out_last(cv, kind, nctas)) {
        advance_call_word(cv, word, inc);
        trace_end(cv, flags);
    }
}

// Bounded wait on an mbarrier phase: gives up at the deadline or when another thread of the CTA
// has raised the abort flag.
__device__ __forceinline__ bool mbar_wait_deadline(uint64_t* bar, uint32_t parity, uint64_t deadline_ns,
                                                   volatile int* s_abort) {
    uint32_t tries = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if ((++tries & 15u) == 0 && (*s_abort || ptx::globaltimer() > deadline_ns)) return false;
    }
    return true;
}

// Block-wide sum of one float per thread (all threads get the result).
__device__ __forceinline__ float block_sum(float v, float* s_red /* >= 32 floats */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();  // protect s_red from the previous use
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? s_red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

}  // namespace yali
