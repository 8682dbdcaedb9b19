// Copy-engine all-reduce: Communicator::LaunchCopyEngine.
//
// The kernels of this library move data with SM- or TMA-issued loads and stores, which on this machine
// top out at 665-707 GB/s per direction with both directions busy; the copy engines reach 774.  For
// messages of tens of MiB and more this path therefore lets cudaMemcpyAsync carry the payload and keeps
// the SMs for the additions:
//
//   one-shot (two ranks):  every rank copies the peer's WHOLE input into local staging, chunk by chunk,
//                          and a kernel adds each chunk to its own data: S bytes per direction, one phase;
//   two-shot:              rank r copies shard r of every peer into staging, adds, and copies the sums
//                          of its shard into every peer's output: 2 S (W-1)/W bytes per direction.
//
// Per rank: the caller's stream runs the enter kernel, one reduce kernel per chunk and the exit kernel;
// internal streams issue the copies: per peer a few "lanes" for the incoming copies (the first one starts
// with a kernel that waits for that peer's "entered" flag) and as many for the outgoing copies of the
// two-shot form.  Chunk c uses lane c % lanes and staging slot c % lanes, so the several microseconds a
// copy takes to start overlap with the transfer of the chunk before it.  Chunks are ordered by events:
// copy c -> reduce c -> (outgoing copy c | reuse of the staging slot by copy c + lanes).
// Every cross-rank wait is a bounded spin in a one-CTA kernel that records a timeout like all others.
//
// Parity: none in the reference.
#include <algorithm>
#include <cstring>

#include "../kernels/copy_engine.h"
#include "../ops/tuning.h"
#include "communicator.h"

namespace yali {

namespace {

#define YALI_CE_CUDA(expr)                                                                        \
    do {                                                                                          \
        cudaError_t e__ = (expr);                                                                 \
        if (e__ != cudaSuccess) {                                                                 \
            (void)cudaGetLastError();                                                             \
            return Fail(Result::CudaError, std::string("copy-engine path: " #expr ": ") + cudaGetErrorString(e__)); \
        }                                                                                         \
    } while (0)

}  // namespace

constexpr uint32_t kCeMaxLanes = 8;  // copies in flight per peer and direction (= staging slots per source)

struct Communicator::CeState {
    // A copy takes several microseconds to start, so consecutive chunks go to different streams
    // ("lanes", chunk c on lane c % lanes) and overlap their start-up with the previous chunk's transfer.
    cudaStream_t pull[kMaxRanks - 1][kCeMaxLanes] = {};
    cudaStream_t push[kMaxRanks - 1][kCeMaxLanes] = {};
    cudaEvent_t start = nullptr;
    cudaEvent_t entered[kMaxRanks - 1] = {};
    cudaEvent_t pulled[kMaxRanks - 1][kCeMaxChunks] = {};
    cudaEvent_t reduced[kCeMaxChunks] = {};
    cudaEvent_t push_lane[kMaxRanks - 1][kCeMaxLanes] = {};
    cudaEvent_t pushed[kMaxRanks - 1] = {};
    char* staging = nullptr;
    uint64_t staging_bytes = 0;
};

void Communicator::DestroyCopyEngineState() {
    for (size_t i = 0; i < ce_.size(); ++i) {
        CeState* s = ce_[i];
        if (!s) continue;
        if (nlocal() > 1) cudaSetDevice(local_[i].device);
        for (int j = 0; j < kMaxRanks - 1; ++j) {
            for (uint32_t l = 0; l < kCeMaxLanes; ++l) {
                if (s->pull[j][l]) cudaStreamDestroy(s->pull[j][l]);
                if (s->push[j][l]) cudaStreamDestroy(s->push[j][l]);
                if (s->push_lane[j][l]) cudaEventDestroy(s->push_lane[j][l]);
            }
            if (s->pushed[j]) cudaEventDestroy(s->pushed[j]);
            if (s->entered[j]) cudaEventDestroy(s->entered[j]);
            for (uint32_t c = 0; c < kCeMaxChunks; ++c)
                if (s->pulled[j][c]) cudaEventDestroy(s->pulled[j][c]);
        }
        for (uint32_t c = 0; c < kCeMaxChunks; ++c)
            if (s->reduced[c]) cudaEventDestroy(s->reduced[c]);
        if (s->start) cudaEventDestroy(s->start);
        if (s->staging) cudaFree(s->staging);
        delete s;
    }
    ce_.clear();
}

Result Communicator::LaunchCopyEngine(const Plan& plan, Dtype dt, CollArgs* args, const cudaStream_t* streams) {
    if (emulated_ || nlocal() != 1) return Fail(Result::Unsupported, "the copy-engine path needs one process and one GPU per rank");
    const bool one_shot = plan.flags & kFlagPullOneShot;
    const int W = world_;
    const uint64_t esize = DtypeSize(dt);
    const uint64_t chunk_elems = plan.slot_bytes / esize;
    const uint32_t lanes = std::min<uint32_t>(std::max<uint32_t>(2, plan.stages), kCeMaxLanes);
    if (chunk_elems == 0 || (plan.slot_bytes % 16) != 0) return Fail(Result::InvalidArg, "copy-engine chunk size");
    if (ce_.empty()) ce_.resize(local_.size(), nullptr);
    auto new_event = [](cudaEvent_t* e) {
        return *e ? cudaSuccess : cudaEventCreateWithFlags(e, cudaEventDisableTiming);
    };
    auto new_stream = [](cudaStream_t* s) {
        return *s ? cudaSuccess : cudaStreamCreateWithFlags(s, cudaStreamNonBlocking);
    };
    // The region a rank sums: everything (one-shot) or its shard.
    auto region = [&](int r, uint64_t count, uint64_t* begin, uint64_t* end) {
        *begin = one_shot ? 0 : std::min<uint64_t>(count, static_cast<uint64_t>(r) * plan.shard_elems);
        *end = one_shot ? count : std::min<uint64_t>(count, *begin + plan.shard_elems);
    };

    // First everything that allocates, for all local ranks: an allocation on one GPU can wait for kernels
    // that run on another, and the kernels launched below wait for the other ranks' kernels.
    for (int i = 0; i < nlocal(); ++i) {
        if (nlocal() > 1) YALI_CE_CUDA(cudaSetDevice(local_[i].device));
        cudaStream_t main = streams && streams[i] ? streams[i] : local_[i].stream;
        uint64_t begin, end;
        region(local_[i].rank, args[i].count, &begin, &end);
        const uint32_t chunks = static_cast<uint32_t>((end - begin + chunk_elems - 1) / chunk_elems);
        if (chunks == 0 || chunks > kCeMaxChunks)
            return Fail(Result::InvalidArg, "copy-engine path: every rank needs between 1 and 64 chunks");
        CeState*& st = ce_[i];
        if (!st) st = new CeState();
        const uint64_t need = static_cast<uint64_t>(W - 1) * lanes * plan.slot_bytes;
        if (st->staging_bytes < need) {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            YALI_CE_CUDA(cudaStreamIsCapturing(main, &cap));
            if (cap != cudaStreamCaptureStatusNone)
                return Fail(Result::Unsupported,
                            "copy-engine path: run the call once outside stream capture first (it allocates its staging then)");
            if (st->staging) {
                YALI_CE_CUDA(cudaDeviceSynchronize());
                YALI_CE_CUDA(cudaFree(st->staging));
                st->staging = nullptr;
                st->staging_bytes = 0;
            }
            YALI_CE_CUDA(cudaMalloc(reinterpret_cast<void**>(&st->staging), need));
            st->staging_bytes = need;
        }
        YALI_CE_CUDA(new_event(&st->start));
        for (int j = 0; j < W - 1; ++j) {
            for (uint32_t l = 0; l < lanes; ++l) {
                YALI_CE_CUDA(new_stream(&st->pull[j][l]));
                if (!one_shot) {
                    YALI_CE_CUDA(new_stream(&st->push[j][l]));
                    YALI_CE_CUDA(new_event(&st->push_lane[j][l]));
                }
            }
            YALI_CE_CUDA(new_event(&st->pushed[j]));
            YALI_CE_CUDA(new_event(&st->entered[j]));
            for (uint32_t c = 0; c < chunks; ++c) YALI_CE_CUDA(new_event(&st->pulled[j][c]));
        }
        for (uint32_t c = 0; c < chunks; ++c) YALI_CE_CUDA(new_event(&st->reduced[c]));
    }

    for (int i = 0; i < nlocal(); ++i) {
        const CollArgs& a = args[i];
        const int r = local_[i].rank;
        if (nlocal() > 1) YALI_CE_CUDA(cudaSetDevice(local_[i].device));
        cudaStream_t main = streams && streams[i] ? streams[i] : local_[i].stream;
        uint64_t begin, end;
        region(r, a.count, &begin, &end);
        const uint32_t chunks = static_cast<uint32_t>((end - begin + chunk_elems - 1) / chunk_elems);
        const uint32_t used = std::min(lanes, chunks);
        CeState* st = ce_[i];
        const char* send = static_cast<const char*>(a.send);
        char* recv = static_cast<char*>(a.recv);
        const bool in_place = send < recv + a.count * esize && recv < send + a.count * esize;

        YALI_CE_CUDA(CeLaunchEnter(a.cv, a.plan_word, a.flags, main));
        YALI_CE_CUDA(cudaEventRecord(st->start, main));
        last_.launches += 1;
        for (int j = 0; j < W - 1; ++j) {
            const int q = j < r ? j : j + 1;
            YALI_CE_CUDA(cudaStreamWaitEvent(st->pull[j][0], st->start, 0));
            YALI_CE_CUDA(CeLaunchWaitEnter(a.cv, 1u << q, st->pull[j][0]));
            last_.launches += 1;
            if (used > 1) YALI_CE_CUDA(cudaEventRecord(st->entered[j], st->pull[j][0]));
            for (uint32_t l = 1; l < used; ++l) YALI_CE_CUDA(cudaStreamWaitEvent(st->pull[j][l], st->entered[j], 0));
        }
        for (uint32_t c = 0; c < chunks; ++c) {
            const uint32_t l = c % lanes;
            const uint64_t e0 = begin + static_cast<uint64_t>(c) * chunk_elems;
            const uint64_t n = std::min<uint64_t>(chunk_elems, end - e0);
            CeReduceArgs ra;
            std::memset(&ra, 0, sizeof(ra));
            for (int j = 0; j < W - 1; ++j) {
                const int q = j < r ? j : j + 1;
                char* slot = st->staging + (static_cast<uint64_t>(j) * lanes + l) * plan.slot_bytes;
                // The slot is free once the reduce kernel of the chunk that used it last has run.
                if (c >= lanes) YALI_CE_CUDA(cudaStreamWaitEvent(st->pull[j][l], st->reduced[c - lanes], 0));
                YALI_CE_CUDA(cudaMemcpyAsync(slot, static_cast<const char*>(a.peer_send[q]) + e0 * esize, n * esize,
                                             cudaMemcpyDefault, st->pull[j][l]));
                YALI_CE_CUDA(cudaEventRecord(st->pulled[j][c], st->pull[j][l]));
                YALI_CE_CUDA(cudaStreamWaitEvent(main, st->pulled[j][c], 0));
                ra.staged[j] = slot;
            }
            ra.cv = a.cv;
            ra.in = send + e0 * esize;
            ra.out = recv + e0 * esize;
            ra.elems = n;
            ra.announce_chunk = one_shot ? c + 1 : 0;
            ra.wait_pulled = one_shot && in_place ? 1 : 0;
            YALI_CE_CUDA(CeLaunchReduce(ra, dt, plan.ctas, main));
            last_.launches += 1;
            if (!one_shot || c + lanes < chunks) YALI_CE_CUDA(cudaEventRecord(st->reduced[c], main));
            if (!one_shot) {
                for (int j = 0; j < W - 1; ++j) {
                    const int q = j < r ? j : j + 1;
                    YALI_CE_CUDA(cudaStreamWaitEvent(st->push[j][l], st->reduced[c], 0));
                    YALI_CE_CUDA(cudaMemcpyAsync(static_cast<char*>(a.peer_recv[q]) + e0 * esize, recv + e0 * esize, n * esize,
                                                 cudaMemcpyDefault, st->push[j][l]));
                }
            }
        }
        if (!one_shot) {
            for (int j = 0; j < W - 1; ++j) {
                const int q = j < r ? j : j + 1;
                // All outgoing copies to q, then "done" to q, then back to the caller's stream.
                for (uint32_t l = 1; l < used; ++l) {
                    YALI_CE_CUDA(cudaEventRecord(st->push_lane[j][l], st->push[j][l]));
                    YALI_CE_CUDA(cudaStreamWaitEvent(st->push[j][0], st->push_lane[j][l], 0));
                }
                YALI_CE_CUDA(CeLaunchDone(a.cv, q, st->push[j][0]));
                YALI_CE_CUDA(cudaEventRecord(st->pushed[j], st->push[j][0]));
                YALI_CE_CUDA(cudaStreamWaitEvent(main, st->pushed[j], 0));
                last_.launches += 1;
            }
        }
        YALI_CE_CUDA(CeLaunchExit(a.cv, chunks, one_shot, a.flags, main));
        last_.launches += 1;
    }
    return Result::Success;
}

}  // namespace yali
