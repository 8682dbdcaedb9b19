// Communicator: the ranks of one all-reduce group as seen from one process, their
// symmetric heaps, epochs and status blocks, and the collective entry points.
//
// A process drives `nlocal` ranks: 1 in multi-process mode (one GPU per process),
// all of them in single-process mode (one host thread launches on every GPU), or
// all of them on ONE GPU in emulated mode (one cooperative launch runs every
// rank; used to exercise the multi-rank kernels on a single device).
//
// Parity: yali::Comm (src/ops/allreduce.cuh:78-323) and yali::MPIComm
// (src/ops/allreduce_mpi.cuh:76-298) own P2P setup, per-lane rings, streams and
// IPC state; yali::allreduce (allreduce.cuh:563-810, allreduce_mpi.cuh:410-676)
// is the collective.  The thin wrappers with those names live in ops/yali.h and
// forward here.
#pragma once

#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/status.h"
#include "../ops/tuning.h"
#include "bootstrap.h"
#include "layout.h"
#include "symm_heap.h"

namespace yali {

struct CommOptions {
    uint64_t heap_bytes = 0;     // 0: YALI_HEAP_BYTES or the default for the world size
    bool want_multicast = true;  // try to set up NVLS
    int64_t timeout_ms = -1;     // -1: YALI_TIMEOUT_MS (default 2000)
};

// Per-call options.
struct OpOptions {
    KernelMode mode = KernelMode::Auto;
    int epilogue = kEpiIdentity;
    float scale = 1.0f;
    // kEpiResidualRmsNorm: per local rank pointers (nullptr entries allowed for residual*)
    int hidden = 0;
    float eps = 1e-5f;
    const void* const* residual = nullptr;
    void* const* residual_out = nullptr;
    const void* const* weight = nullptr;
    bool buffers_stable = false;  // multi-process: reuse the peer mapping of (send, recv) from an earlier call
    int ctas = 0;                 // >0 overrides the planned CTA / lane count
    int slot_bytes = 0;           // >0 overrides the planned slot size
    int skip_rank = -1;           // >=0: that rank's kernel leaves at once (timeout tests; never on a production path)
};

struct LastCallInfo {
    Variant variant = Variant::Flash;
    uint32_t ctas = 0;
    uint32_t slot_bytes = 0;
    uint32_t stages = 0;
    uint32_t flags = 0;
    uint64_t launches = 0;  // kernels launched by this process since creation
};

class Communicator {
   public:
    // One process, one rank per entry of `devices` (distinct GPUs).
    static Result CreateSingleProcess(const std::vector<int>& devices, const CommOptions& opt,
                                      std::unique_ptr<Communicator>* out, std::string* err);
    // One process, `world` ranks that all live on `device`.
    static Result CreateEmulated(int world, int device, const CommOptions& opt, std::unique_ptr<Communicator>* out,
                                 std::string* err);
    // One rank per process; collective over `bs` (ownership taken).
    static Result CreateMultiProcess(std::unique_ptr<Bootstrap> bs, int device, const CommOptions& opt,
                                     std::unique_ptr<Communicator>* out, std::string* err);
    ~Communicator();

    int world() const { return world_; }
    int nlocal() const { return static_cast<int>(local_.size()); }
    int rank_of(int local_index) const { return local_[local_index].rank; }
    int device_of(int local_index) const { return local_[local_index].device; }
    bool emulated() const { return emulated_; }
    bool has_multicast() const { return heaps_ && heaps_->mc_base() != nullptr; }
    const char* heap_kind() const { return heaps_ ? heaps_->kind() : "none"; }
    const HeapLayout& layout() const { return lay_; }
    Bootstrap* bootstrap() const { return bs_.get(); }
    cudaStream_t default_stream(int local_index) const { return local_[local_index].stream; }
    const LastCallInfo& last_call() const { return last_; }
    const std::string& last_error() const { return err_; }

    // recv[i] = epilogue(sum over all ranks of send).  Arrays have nlocal() entries;
    // streams may be nullptr (the communicator's own stream per local rank).
    Result AllReduce(const void* const* send, void* const* recv, uint64_t count, Dtype in, Dtype out,
                     const OpOptions& opt, const cudaStream_t* streams);
    // recv (ShardElems(count, world) elements, of which the valid part is used) = this rank's shard of the sum.
    Result ReduceScatter(const void* const* send, void* const* recv, uint64_t count, Dtype dt, const OpOptions& opt,
                         const cudaStream_t* streams);
    // send = this rank's shard (ShardElems elements); recv = `count` elements, all shards in rank order.
    Result AllGather(const void* const* send, void* const* recv, uint64_t count, Dtype dt, const OpOptions& opt,
                     const cudaStream_t* streams);

    // Symmetric allocation: the same offset in every rank's heap.  Returns one
    // pointer per local rank.  Collective in spirit (every process must perform
    // the same sequence of allocations); never freed individually.
    Result SymmAlloc(uint64_t bytes, std::vector<void*>* ptrs);
    void SymmReset() { user_bump_ = 0; }
    bool IsSymmetric(int local_index, const void* p, uint64_t bytes) const;

    // Waits for all work of this communicator's ranks and reports a device-side timeout.
    Result Sync(const cudaStream_t* streams = nullptr);
    // Non-blocking look at the status blocks.
    Result Check();
    // After a Timeout: host barrier (multi-process), zero all flags and epochs.  Collective.
    Result Reset();
    // Barrier across processes (multi-process) after draining the local streams.
    Result Barrier();
    // Human-readable description of the last device-side timeout, empty when none.
    std::string DescribeStatus() const;

    // Builds the argument block for one local rank without launching (used by the
    // fused GEMM and by the allocation-free entry point's tests).
    CommView View(int local_index) const;
    // Reserves epochs for an externally launched kernel that uses the per-CTA barrier.
    uint32_t TakeBarrierEpochs(uint32_t n);
    uint32_t TakeGemmEpoch() { return ++gemm_epoch_; }
    // Cumulative targets of the fused GEMM's arrival / delivered-rows counters, indexed by rank
    // (identical on every rank; cleared by Reset()).
    struct GemmCounters {
        uint32_t cnt[kMaxRanks] = {};
        uint32_t done[kMaxRanks] = {};
    };
    GemmCounters& gemm_counters() { return gemm_; }
    bool poisoned() const { return poisoned_; }
    uint32_t max_ctas() const { return max_ctas_; }
    void set_error(const std::string& e) { err_ = e; }
    void CountLaunch(uint64_t n = 1) { last_.launches += n; }

    // Device-side timeline: while enabled, every collective stamps %globaltimer when its first
    // CTA starts and when its last CTA checks out (kTraceOff ring in this rank's heap).
    void SetTrace(bool on) { trace_ = on; }
    bool trace() const { return trace_; }
    // Copies the timeline of local rank `local_index` out (after the caller has synchronised):
    // `calls` = traced calls so far; `out` receives the last min(calls, kTraceCap, max_entries)
    // {start_ns, end_ns} pairs, oldest first.  Returns the number of pairs written.
    int ReadTrace(int local_index, uint64_t* out, int max_entries, uint64_t* calls);

   private:
    struct Local {
        int rank = 0;
        int device = 0;
        cudaStream_t stream = nullptr;
        cudaEvent_t prof_start = nullptr, prof_stop = nullptr;  // YALI_PROFILE_KERNELS=1: around the last launch
        bool prof_pending = false;
        DeviceStatus* status = nullptr;  // pinned host memory, device-visible
    };
    struct PeerMap {  // multi-process registration of one user buffer
        void* peer[kMaxRanks];
        uint64_t bytes;
    };

    Communicator() = default;
    Result Init(const CommOptions& opt, std::string* err);
    Result Launch(const Plan& plan, Dtype in, Dtype out, int epilogue, CollArgs* args /*nlocal*/,
                  const cudaStream_t* streams);
    Result Collective(const void* const* send, void* const* recv, uint64_t count, Dtype in, Dtype out,
                      const OpOptions& opt, const cudaStream_t* streams, uint32_t extra_flags);
    Result ResolvePeers(const void* const* send, void* const* recv, uint64_t send_bytes, uint64_t recv_bytes,
                        bool stable, CollArgs* args, bool* peer_recv, bool* symmetric);
    Result EnsureSmemAttr(const void* fn, uint32_t smem_bytes);
    // Copy-engine all-reduce (copy_engine_path.cc): streams, events and staging per local rank, made on first use.
    struct CeState;
    Result LaunchCopyEngine(const Plan& plan, Dtype dt, CollArgs* args, const cudaStream_t* streams);
    void DestroyCopyEngineState();
    std::vector<CeState*> ce_;
    Result Fail(Result r, const std::string& what) {
        err_ = what;
        return r;
    }

    int world_ = 0;
    bool emulated_ = false;
    bool single_process_ = false;
    std::vector<Local> local_;
    std::unique_ptr<Bootstrap> bs_;
    std::unique_ptr<SymmHeapSet> heaps_;
    HeapLayout lay_{};
    uint64_t timeout_ns_ = 0;
    uint32_t max_ctas_ = 296;
    uint32_t sm_count_ = 148;
    bool trace_ = false;
    std::vector<CollArgs> args_scratch_;  // per-call argument blocks, reused (no allocation per call)
    std::vector<std::pair<const void*, int>> smem_attr_set_;  // (kernel, device) pairs with the smem limit raised
    // Epochs: identical on every rank because every rank performs the same calls.
    uint32_t flash_epoch_ = 0;
    uint32_t bar_epoch_ = 0;
    uint32_t stream_seq_ = 0;
    uint32_t gemm_epoch_ = 0;
    GemmCounters gemm_;
    uint64_t user_bump_ = 0;
    bool poisoned_ = false;
    LastCallInfo last_;
    std::string err_;
    std::unordered_map<const void*, PeerMap> ipc_cache_;
    std::vector<void*> ipc_opened_;
};

}  // namespace yali
