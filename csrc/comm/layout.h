// Layout of the symmetric heap and the by-value argument blocks of the kernels.
// Shared by host and device code.
//
// Parity: the reference passes one YaliLaunchArgs per lane through a device array
// that is memcpy'd before every launch (src/include/yali_launch.h:16-58,
// src/ops/allreduce.cuh:753-761) and allocates three cudaMalloc blocks per lane
// for the ring (allreduce.cuh:388-458).  Here each rank owns ONE allocation (the
// heap) that is mapped on every peer; flags, one-shot staging, ring slots, NVLS
// staging and user-visible symmetric buffers live at fixed offsets in it, and
// kernels receive everything they need as a parameter struct.
#pragma once

#include <stdint.h>

#include "../core/status.h"

namespace yali {

// ---- control words (uint32 indices into the flag region; zero-initialised, monotone) ----
constexpr int kMaxFlashCtas = 2048;  // one flag row per CTA of the one-shot kernel
constexpr int kMaxLanes = 256;       // lanes (CTAs) of the two-shot ring kernel
constexpr int kBarSlots = 1024;      // per-CTA cross-rank barriers (NVLS and fused kernels)
constexpr int kGemmRowBlocks = 256;  // arrival counters of the fused GEMM, one per 128-row block

// Call counters of this rank, advanced by the kernels themselves (the last CTA of a launch
// bumps them), so a launch carries no per-call number and can be replayed from a CUDA graph.
constexpr uint32_t kCallFlashEpoch = 0;   // one-shot calls so far
constexpr uint32_t kCallStreamSeq = 1;    // ring sequence numbers consumed so far
constexpr uint32_t kCallBarEpoch = 2;     // per-CTA barrier epochs consumed so far
constexpr uint32_t kCallGemmEpoch = 3;    // fused GEMM calls so far
constexpr uint32_t kCallFlashEpochHi = 5;  // upper half of the one-shot call number (flag-in-data protocol)
constexpr uint32_t kCallGemmLLEpoch = 6;   // calls of the fused GEMM's few-token form so far (lower half)
constexpr uint32_t kCallGemmLLEpochHi = 7;  // upper half of that call number
constexpr uint32_t kCallGemmCnt = 4;      // arrivals (per source) this rank has been promised so far
constexpr uint32_t kCallGemmDone = 8;     // [kMaxRanks] rows each owner has been asked to deliver so far
constexpr uint32_t kCallDoneCtas = 16;    // [4] CTAs of the running launch that have finished, per kernel kind
constexpr uint32_t kCallTraceIdx = 20;    // traced calls so far (index into the kTraceOff ring)
constexpr uint32_t kCallPlanWord = 21;    // what this rank's running (or last) collective is: PlanWord() of its plan
constexpr uint32_t kCallCeCalls = 22;     // copy-engine all-reduce calls so far
constexpr uint32_t kFlashFlagOff = 32;                                       // [kMaxFlashCtas][kMaxRanks]
constexpr uint32_t kRsSeqOff = kFlashFlagOff + kMaxFlashCtas * kMaxRanks;    // [kMaxLanes][kMaxRanks]
constexpr uint32_t kAgSeqOff = kRsSeqOff + kMaxLanes * kMaxRanks;            // [kMaxLanes][kMaxRanks]
constexpr uint32_t kCreditOff = kAgSeqOff + kMaxLanes * kMaxRanks;           // [kMaxLanes][kMaxRanks]
constexpr uint32_t kBarOff = kCreditOff + kMaxLanes * kMaxRanks;             // [kBarSlots][kMaxRanks]
constexpr uint32_t kGemmCntOff = kBarOff + kBarSlots * kMaxRanks;            // [kGemmRowBlocks][kMaxRanks]
constexpr uint32_t kGemmDoneOff = kGemmCntOff + kGemmRowBlocks * kMaxRanks;  // [kGemmRowBlocks][kMaxRanks]
constexpr uint32_t kStatusCntOff = kGemmDoneOff + kGemmRowBlocks * kMaxRanks;  // [1] timeouts seen by this rank
// Device-side timeline of the collectives (kFlagTrace): call i writes %globaltimer at the entry of
// its first CTA and at the check-out of its last CTA into entry i % kTraceCap.
constexpr uint32_t kTraceCap = 4096;
constexpr uint32_t kTraceOff = kStatusCntOff + 8;              // [kTraceCap][2] uint64 = 4 words per call
// Copy-engine all-reduce (kernels/copy_engine.cu): progress words written by the peers, one per source.
constexpr uint32_t kCeEnterOff = kTraceOff + kTraceCap * 4;  // [kMaxRanks] call the source has entered
constexpr uint32_t kCePulledOff = kCeEnterOff + kMaxRanks;   // [kMaxRanks] (call << 8) | chunks the source has read here
constexpr uint32_t kCeDoneOff = kCePulledOff + kMaxRanks;    // [kMaxRanks] call the source has finished with this rank
constexpr uint32_t kFlagWords = kCeDoneOff + kMaxRanks;
constexpr uint64_t kFlagRegionBytes = 1ull << 20;
static_assert(kFlagWords * 4ull <= kFlagRegionBytes, "flag region too small");
static_assert(kTraceOff % 2 == 0, "the timeline entries are 64-bit words");

constexpr int kRingCap = 4;  // slots per (lane, source) ring
constexpr uint32_t kMaxPipelineStages = 8;  // shared-memory stages of the pipelined kernels

struct HeapLayout {
    uint64_t total_bytes;
    uint64_t flags_off;    // kFlagRegionBytes of uint32 control words
    uint64_t flash_off;    // one-shot staging: [2 parities][world-1 sources][flash_cap]
    uint64_t flash_cap;    // largest one-shot message in bytes
    uint64_t ring_off;     // two-shot rings: [lane][world-1 sources][kRingCap][2 (RS, AG)][slot]
    uint64_t ring_bytes;
    uint64_t nvls_off;     // staging for multimem kernels when user buffers are not in the heap: [2][nvls_cap]
    uint64_t nvls_cap;
    uint64_t gemm_off;     // partial-sum landing zone of the fused GEMM: [2][world][gemm_cap]
    uint64_t gemm_cap;
    uint64_t ll_off;       // staging of the flag-in-data one-shot protocol: [2 parities][world-1 sources][2 * ll_cap]
    uint64_t ll_cap;       // largest message (bytes of payload) that protocol takes
    uint64_t gemm_ll_off;  // landing zone of the fused GEMM's few-token form, flag-in-data lines: [2][world][gemm_ll_cap]
    uint64_t gemm_ll_cap;  // bytes per (parity, source): rows * N * 2 bytes of payload, doubled by the flags
    uint64_t user_off;     // symmetric allocations handed to the user
    uint64_t user_bytes;
};

// Default sizing for a world size; `requested_total` of 0 picks the default.
// Returns false when the request is too small to hold the fixed regions.
bool MakeHeapLayout(int world, uint64_t requested_total, uint64_t granularity, HeapLayout* out);

// Index of source rank `src` in the per-destination arrays that skip the owner.
__host__ __device__ inline int SrcSlot(int src, int owner) { return src < owner ? src : src - 1; }

// What a device-side wait writes when it gives up.  Lives in pinned host memory
// that the device can write, one block per rank.
enum WaitSite : uint32_t {
    kSiteNone = 0,
    kSiteFlashArrive = 1,
    kSiteStreamCredit = 2,
    kSiteStreamRs = 3,
    kSiteStreamAg = 4,
    kSiteStreamDrain = 5,
    kSiteBarrier = 6,
    kSiteGemmPartials = 7,
    kSiteGemmDone = 8,
    kSiteMbar = 9,
    kSiteCeEnter = 10,
    kSiteCePulled = 11,
    kSiteCeExit = 12,
};
struct DeviceStatus {
    uint32_t code;      // 0 = ok, otherwise a WaitSite
    uint32_t rank;
    uint32_t peer;
    uint32_t cta;
    uint32_t wanted;
    uint32_t observed;
    uint32_t my_plan;    // PlanWord of the call that gave up ...
    uint32_t peer_plan;  // ... and of what the awaited rank was running (or last ran): they differ when the
                         // ranks were given different arguments and therefore chose different kernels
};

// Identity of a plan in 32 bits: kernel (4 bits, variant + 1), CTAs (12 bits), low bits of the element count.
__host__ __device__ inline uint32_t PlanWord(int variant, uint32_t ctas, uint64_t count) {
    return (static_cast<uint32_t>(variant + 1) << 28) | ((ctas & 0xfffu) << 16) | static_cast<uint32_t>(count & 0xffffu);
}

// One rank's view of the communicator.
struct CommView {
    char* heap[kMaxRanks];  // heap base of every rank as mapped for this device
    char* mc_heap;          // multicast mapping of the heaps, nullptr without NVLS
    HeapLayout lay;
    DeviceStatus* status;
    uint64_t timeout_ns;
    int rank;
    int world;
};

enum EpilogueKind : int { kEpiIdentity = 0, kEpiScaleCast = 1, kEpiResidualRmsNorm = 2 };

struct EpilogueParams {
    float scale;            // kEpiScaleCast: out = cast(sum * scale)
    float eps;              // kEpiResidualRmsNorm
    int hidden;             // row length of the RMSNorm
    const void* residual;   // [rows, hidden], output dtype; may be nullptr
    void* residual_out;     // optional: sum + residual before normalisation
    const void* weight;     // [hidden], output dtype
};

struct CollArgs {
    CommView cv;
    const void* send;                   // this rank's input
    void* recv;                         // this rank's output
    const void* peer_send[kMaxRanks];   // inputs of all ranks when they are peer-addressable, else nullptr
    void* peer_recv[kMaxRanks];         // outputs of all ranks when they are peer-addressable, else nullptr
    uint64_t count;                     // elements
    uint32_t stages;                    // pipelined kernels: shared-memory stages per CTA
    uint32_t plan_word;                 // PlanWord(): published at kernel start, compared with the peer's after a timeout
    uint32_t ctas;                      // CTAs (one-shot, NVLS, pipelined) or lanes (two-shot ring) per rank
    uint32_t slot_bytes;                // two-shot ring slot size; pipelined kernels: bytes per source and stage
    uint64_t shard_elems;               // two-shot / NVLS: elements owned by each rank
    uint32_t flags;                     // CollFlags
    EpilogueParams ep;
};

enum CollFlags : uint32_t {
    kFlagVecOk = 1u << 0,       // pointers 16-byte aligned: vector path
    kFlagDirectAg = 1u << 1,    // all-gather writes straight into peer_recv
    kFlagSymmetric = 1u << 2,   // NVLS: send/recv live in the heap at cv offsets (zero copy)
    kFlagReduceScatterOnly = 1u << 3,
    kFlagAllGatherOnly = 1u << 4,
    kFlagLowLatency = 1u << 6,  // one-shot: flag-in-data protocol (no separate flag, no release fence)
    kFlagSkipRank = 1u << 5,    // this rank leaves at once (models a rank that never launched; tests of the timeouts)
    kFlagTrace = 1u << 7,       // stamp %globaltimer at entry and check-out into the kTraceOff ring
    kFlagPullOneShot = 1u << 8, // pipelined kernel: every rank pulls and sums the whole message (no pushes)
};

// All ranks of an emulated communicator in one launch (ranks = blockIdx.y).
struct EmuArgs {
    CollArgs r[kMaxRanks];
};

}  // namespace yali
