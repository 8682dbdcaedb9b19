#include "communicator.h"

#include "../core/nvtx.h"

#include <algorithm>
#include <cstdio>
#include <cstring>

#include "../core/env.h"
#include "../kernels/launch.h"
#include "../ops/buffer_ops.h"
#include "topology.h"

namespace yali {

namespace {
uint64_t RoundUp(uint64_t a, uint64_t b) { return (a + b - 1) / b * b; }
bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
}  // namespace

bool MakeHeapLayout(int world, uint64_t requested_total, uint64_t granularity, HeapLayout* out) {
    HeapLayout l;
    std::memset(&l, 0, sizeof(l));
    const uint64_t MiB = 1ull << 20;
    uint64_t off = 0;
    l.flags_off = off;
    off += kFlagRegionBytes;
    if (world > 1) {
        l.flash_cap = world == 2 ? 64 * MiB : (world <= 4 ? 16 * MiB : 8 * MiB);
        l.flash_off = off;
        off += 2ull * (world - 1) * l.flash_cap;
        l.ring_off = off;
        l.ring_bytes = 256 * MiB;
        off += l.ring_bytes;
        l.nvls_off = off;
        l.nvls_cap = 64 * MiB;
        off += 2 * l.nvls_cap;
        l.gemm_off = off;
        // 2048 rows of 4096 bf16 sharded over the ranks; a whole number of MiB, so that every region
        // after it stays aligned for any world size (16 MiB / 3 is not even a multiple of 16 bytes).
        l.gemm_cap = std::max<uint64_t>(4 * MiB, RoundUp(16 * MiB / world, MiB));
        off += 2ull * world * l.gemm_cap;
        l.ll_off = off;
        l.ll_cap = 1 * MiB;
        off += 2ull * (world - 1) * 2 * l.ll_cap;
        l.gemm_ll_off = off;
        l.gemm_ll_cap = 4 * MiB;  // per source rank: 64 rows of 4096 bf16 as flag-in-data lines from four K splits
        const long long ll_mib = env::GetInt("YALI_GEMM_LL_CAP_MIB", 0);  // measurements only (every rank alike)
        if (ll_mib >= 1 && ll_mib <= 64) l.gemm_ll_cap = static_cast<uint64_t>(ll_mib) * MiB;
        off += 2ull * world * l.gemm_ll_cap;
    }
    l.user_off = off;
    uint64_t total = requested_total ? requested_total : off + 256 * MiB;
    if (granularity) total = RoundUp(total, granularity);
    if (total < off + MiB) return false;
    l.user_bytes = total - off;
    l.total_bytes = total;
    *out = l;
    return true;
}

Result Communicator::CreateSingleProcess(const std::vector<int>& devices, const CommOptions& opt,
                                         std::unique_ptr<Communicator>* out, std::string* err) {
    std::vector<int> u(devices);
    std::sort(u.begin(), u.end());
    if (devices.empty() || devices.size() > static_cast<size_t>(kMaxRanks) ||
        std::adjacent_find(u.begin(), u.end()) != u.end()) {
        if (err) *err = "need 1.." + std::to_string(kMaxRanks) + " distinct GPUs";
        return Result::InvalidArg;
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || u.back() >= ndev || u.front() < 0) {
        (void)cudaGetLastError();
        if (err) *err = "GPU index out of range";
        return Result::InvalidArg;
    }
    // User buffers from cudaMalloc must be reachable from every GPU of the group.
    if (!EnableAllPairsP2P(devices)) {
        if (err) *err = "peer access could not be enabled between all GPUs";
        return Result::PeerAccessFailed;
    }
    std::unique_ptr<Communicator> c(new Communicator());
    c->world_ = static_cast<int>(devices.size());
    c->single_process_ = true;
    c->local_.resize(devices.size());
    for (size_t i = 0; i < devices.size(); ++i) {
        c->local_[i].rank = static_cast<int>(i);
        c->local_[i].device = devices[i];
    }
    Result r = c->Init(opt, err);
    if (r != Result::Success) return r;
    *out = std::move(c);
    return Result::Success;
}

Result Communicator::CreateEmulated(int world, int device, const CommOptions& opt, std::unique_ptr<Communicator>* out,
                                    std::string* err) {
    if (world < 1 || world > kMaxRanks) {
        if (err) *err = "world size out of range";
        return Result::InvalidArg;
    }
    std::unique_ptr<Communicator> c(new Communicator());
    c->world_ = world;
    c->single_process_ = true;
    c->emulated_ = true;
    c->local_.resize(world);
    for (int i = 0; i < world; ++i) {
        c->local_[i].rank = i;
        c->local_[i].device = device;
    }
    Result r = c->Init(opt, err);
    if (r != Result::Success) return r;
    *out = std::move(c);
    return Result::Success;
}

Result Communicator::CreateMultiProcess(std::unique_ptr<Bootstrap> bs, int device, const CommOptions& opt,
                                        std::unique_ptr<Communicator>* out, std::string* err) {
    if (!bs) {
        if (err) *err = "no bootstrap";
        return Result::InvalidArg;
    }
    std::unique_ptr<Communicator> c(new Communicator());
    c->world_ = bs->world();
    c->local_.resize(1);
    c->local_[0].rank = bs->rank();
    c->local_[0].device = device;
    c->bs_ = std::move(bs);
    Result r = c->Init(opt, err);
    // Whether or not this rank succeeded, all ranks must agree before anyone launches.
    char ok = r == Result::Success;
    std::vector<char> all(c->world_);
    if (c->bs_->allgather(&ok, all.data(), 1) != Result::Success) {
        if (err && r == Result::Success) *err = c->bs_->last_error();
        return r == Result::Success ? Result::BootstrapError : r;
    }
    if (r != Result::Success) return r;
    if (!std::all_of(all.begin(), all.end(), [](char x) { return x != 0; })) {
        if (err) *err = "another rank failed to create its communicator";
        return Result::BootstrapError;
    }
    *out = std::move(c);
    return Result::Success;
}

Result Communicator::Init(const CommOptions& opt, std::string* err) {
    const int dev0 = local_[0].device;
    if (cudaSetDevice(dev0) != cudaSuccess) {
        (void)cudaGetLastError();
        if (err) *err = "cudaSetDevice(" + std::to_string(dev0) + ") failed";
        return Result::CudaError;
    }
    uint64_t want = opt.heap_bytes ? opt.heap_bytes : static_cast<uint64_t>(env::HeapBytes());
    const bool want_mc = opt.want_multicast && !emulated_ && world_ > 1;
    HeapLayout probe;
    if (!MakeHeapLayout(world_, want, 0, &probe)) {
        if (err) *err = "heap size too small for the fixed regions of a " + std::to_string(world_) + "-rank group";
        return Result::InvalidArg;
    }
    Result r;
    if (bs_) {
        r = SymmHeapSet::CreateShared(*bs_, dev0, probe.total_bytes, want_mc, &heaps_, err);
    } else {
        std::vector<int> devs;
        for (const Local& l : local_) devs.push_back(l.device);
        r = SymmHeapSet::CreateLocal(devs, probe.total_bytes, want_mc, &heaps_, err);
    }
    if (r != Result::Success) return r;
    MakeHeapLayout(world_, heaps_->bytes(), 0, &lay_);

    const long long tmo = opt.timeout_ms >= 0 ? opt.timeout_ms : env::TimeoutMs();
    timeout_ns_ = static_cast<uint64_t>(std::max<long long>(tmo, 1)) * 1000000ull;

    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev0) != cudaSuccess) {
        if (err) *err = "cudaGetDeviceProperties failed";
        return Result::CudaError;
    }
    // Emulated ranks share one GPU and run in one cooperative launch: every CTA of every
    // rank must be resident (two 512-thread CTAs per SM are guaranteed by the launch bounds).
    max_ctas_ = emulated_ ? std::max(1, prop.multiProcessorCount * 2 / world_) : prop.multiProcessorCount * 8;
    sm_count_ = static_cast<uint32_t>(std::max(1, prop.multiProcessorCount));
    args_scratch_.resize(local_.size());

    for (Local& l : local_) {
        if (cudaSetDevice(l.device) != cudaSuccess || cudaStreamCreate(&l.stream) != cudaSuccess ||
            cudaHostAlloc(reinterpret_cast<void**>(&l.status), sizeof(DeviceStatus), cudaHostAllocMapped |
                                                                                         cudaHostAllocPortable) !=
                cudaSuccess) {
            (void)cudaGetLastError();
            if (err) *err = "stream / status allocation failed on GPU " + std::to_string(l.device);
            return Result::CudaError;
        }
        std::memset(l.status, 0, sizeof(DeviceStatus));
    }
    cudaSetDevice(dev0);
    if (env::DebugLevel() > 0 && local_[0].rank == 0)
        std::fprintf(stderr, "[yali] world=%d nlocal=%d heap=%s %.0f MiB multicast=%d emulated=%d\n", world_, nlocal(),
                     heaps_->kind(), lay_.total_bytes / 1048576.0, has_multicast() ? 1 : 0, emulated_ ? 1 : 0);
    return Result::Success;
}

Communicator::~Communicator() {
    for (Local& l : local_) {
        if (cudaSetDevice(l.device) == cudaSuccess) cudaDeviceSynchronize();
    }
    DestroyCopyEngineState();
    // Nobody unmaps or unbinds while a peer may still touch this rank's heap.
    if (bs_) bs_->barrier();
    for (void* p : ipc_opened_) cudaIpcCloseMemHandle(p);
    heaps_.reset();
    for (Local& l : local_) {
        if (cudaSetDevice(l.device) != cudaSuccess) continue;
        if (l.prof_start) cudaEventDestroy(l.prof_start);
        if (l.prof_stop) cudaEventDestroy(l.prof_stop);
        if (l.status) cudaFreeHost(l.status);
        if (l.stream) cudaStreamDestroy(l.stream);
    }
    (void)cudaGetLastError();
}

CommView Communicator::View(int i) const {
    CommView v;
    std::memset(&v, 0, sizeof(v));
    for (int q = 0; q < world_; ++q) v.heap[q] = heaps_->base(q);
    v.mc_heap = heaps_->mc_base();
    v.lay = lay_;
    v.status = local_[i].status;
    v.timeout_ns = timeout_ns_;
    v.rank = local_[i].rank;
    v.world = world_;
    return v;
}

uint32_t Communicator::TakeBarrierEpochs(uint32_t n) {
    uint32_t e = bar_epoch_;
    bar_epoch_ += n;
    return e;
}

bool Communicator::IsSymmetric(int i, const void* p, uint64_t bytes) const {
    const char* base = heaps_->base(local_[i].rank);
    const char* c = static_cast<const char*>(p);
    return c >= base + lay_.user_off && c + bytes <= base + lay_.total_bytes;
}

Result Communicator::SymmAlloc(uint64_t bytes, std::vector<void*>* ptrs) {
    const uint64_t need = RoundUp(std::max<uint64_t>(bytes, 1), 256);
    if (user_bump_ + need > lay_.user_bytes)
        return Fail(Result::InvalidArg, "symmetric heap exhausted: " + std::to_string(lay_.user_bytes - user_bump_) +
                                            " bytes left, " + std::to_string(need) +
                                            " requested (raise YALI_HEAP_BYTES)");
    ptrs->clear();
    for (const Local& l : local_) ptrs->push_back(heaps_->base(l.rank) + lay_.user_off + user_bump_);
    user_bump_ += need;
    return Result::Success;
}

// Fills the peer tables.  Single process: every rank's pointers are known and
// addressable.  Multi process: only heap buffers (same offset on every rank) are.
Result Communicator::ResolvePeers(const void* const* send, void* const* recv, uint64_t send_bytes, uint64_t recv_bytes,
                                  bool /*stable*/, CollArgs* args, bool* peer_recv, bool* symmetric) {
    bool all_sym = true;
    for (int i = 0; i < nlocal(); ++i) {
        if (!IsSymmetric(i, send[i], send_bytes) || !IsSymmetric(i, recv[i], recv_bytes)) all_sym = false;
    }
    if (all_sym && nlocal() > 1) {
        // Equal offsets on all local ranks?
        const uint64_t so = static_cast<const char*>(send[0]) - heaps_->base(local_[0].rank);
        const uint64_t ro = static_cast<const char*>(recv[0]) - heaps_->base(local_[0].rank);
        for (int i = 1; i < nlocal(); ++i) {
            if (static_cast<uint64_t>(static_cast<const char*>(send[i]) - heaps_->base(local_[i].rank)) != so ||
                static_cast<uint64_t>(static_cast<const char*>(recv[i]) - heaps_->base(local_[i].rank)) != ro)
                all_sym = false;
        }
    }
    *symmetric = all_sym;
    *peer_recv = false;
    for (int i = 0; i < nlocal(); ++i) {
        for (int q = 0; q < kMaxRanks; ++q) {
            args[i].peer_send[q] = nullptr;
            args[i].peer_recv[q] = nullptr;
        }
    }
    if (single_process_) {
        for (int i = 0; i < nlocal(); ++i) {
            for (int j = 0; j < nlocal(); ++j) {
                args[i].peer_send[local_[j].rank] = send[j];
                args[i].peer_recv[local_[j].rank] = recv[j];
            }
        }
        *peer_recv = true;
    } else if (all_sym) {
        const uint64_t so = static_cast<const char*>(send[0]) - heaps_->base(local_[0].rank);
        const uint64_t ro = static_cast<const char*>(recv[0]) - heaps_->base(local_[0].rank);
        for (int q = 0; q < world_; ++q) {
            args[0].peer_send[q] = heaps_->base(q) + so;
            args[0].peer_recv[q] = heaps_->base(q) + ro;
        }
        *peer_recv = true;
    }
    return Result::Success;
}

// Kernels that use more than 48 KiB of dynamic shared memory need the limit raised once per
// (kernel, device).
Result Communicator::EnsureSmemAttr(const void* fn, uint32_t smem_bytes) {
    if (smem_bytes <= 48u * 1024u) return Result::Success;
    for (int i = 0; i < nlocal(); ++i) {
        const std::pair<const void*, int> key(fn, local_[i].device);
        if (std::find(smem_attr_set_.begin(), smem_attr_set_.end(), key) != smem_attr_set_.end()) continue;
        if (nlocal() > 1 && !emulated_) cudaSetDevice(local_[i].device);
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return Fail(Result::CudaError, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
        }
        smem_attr_set_.push_back(key);
    }
    return Result::Success;
}

int Communicator::ReadTrace(int local_index, uint64_t* out, int max_entries, uint64_t* calls) {
    if (local_index < 0 || local_index >= nlocal() || !out || max_entries <= 0) return 0;
    const Local& l = local_[local_index];
    cudaSetDevice(l.device);
    const char* flags = heaps_->base(l.rank) + lay_.flags_off;
    uint32_t idx = 0;
    std::vector<uint64_t> ring(static_cast<size_t>(kTraceCap) * 2);
    if (cudaMemcpy(&idx, flags + kCallTraceIdx * 4ull, 4, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(ring.data(), flags + kTraceOff * 4ull, ring.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    if (calls) *calls = idx;
    const uint32_t n = std::min<uint32_t>(std::min<uint32_t>(idx, kTraceCap), static_cast<uint32_t>(max_entries));
    for (uint32_t k = 0; k < n; ++k) {
        const uint32_t call = idx - n + k;
        out[2 * k] = ring[(call % kTraceCap) * 2];
        out[2 * k + 1] = ring[(call % kTraceCap) * 2 + 1];
    }
    return static_cast<int>(n);
}

Result Communicator::Launch(const Plan& plan, Dtype in, Dtype out, int epilogue, CollArgs* args,
                            const cudaStream_t* streams) {
    const void* fn = nullptr;
    int threads = 0;
    switch (plan.variant) {
        case Variant::Flash:
            fn = (plan.flags & kFlagLowLatency) ? FlashLLKernelFor(in, world_, emulated_)
                                                : FlashKernelFor(in, out, epilogue, world_, emulated_);
            threads = kFlashThreads;
            break;
        case Variant::Stream:
            fn = StreamKernelFor(in, out, epilogue, world_, emulated_);
            threads = kStreamThreads;
            break;
        case Variant::NvlsOneShot:
        case Variant::NvlsTwoShot:
            if (emulated_) return Fail(Result::Unsupported, "multicast kernels cannot run on emulated ranks");
            fn = NvlsKernelFor(in, world_, plan.variant == Variant::NvlsTwoShot);
            threads = kNvlsThreads;
            {
                static const long long dev_threads = env::GetInt("YALI_DEV_THREADS", 0);  // tuning sweeps only
                if (dev_threads >= 64 && dev_threads <= kNvlsThreads) threads = static_cast<int>(dev_threads) / 32 * 32;
            }
            break;
        case Variant::CopyEngine:
            if (in != out || epilogue != kEpiIdentity) return Fail(Result::Unsupported, "the copy-engine path only sums");
            return LaunchCopyEngine(plan, in, args, streams);
        case Variant::FlashPull:
        case Variant::StreamDirect:
            fn = DirectKernelFor(in, out, world_, plan.variant == Variant::FlashPull, emulated_);
            threads = kDirectThreads;
            break;
    }
    if (!fn) return Fail(Result::Unsupported, "no kernel for this dtype / epilogue combination");
    if (epilogue == kEpiResidualRmsNorm) {
        // One thread handles up to four 16-byte vectors of a row.
        const int vec = 16 / static_cast<int>(DtypeSize(in));
        const int vec_per_row = args[0].ep.hidden / vec;
        threads = std::min(kFlashThreads, std::max(32, (vec_per_row + 31) / 32 * 32));
    }
    const uint32_t smem = plan.smem_bytes;
    if (smem > 0) {
        Result r = EnsureSmemAttr(fn, smem);
        if (r != Result::Success) return r;
    }
    if (emulated_) {
        EmuArgs e;
        std::memset(&e, 0, sizeof(e));
        for (int i = 0; i < nlocal(); ++i) e.r[local_[i].rank] = args[i];
        cudaStream_t s = streams && streams[0] ? streams[0] : local_[0].stream;
        void* params[] = {&e};
        cudaError_t ce = cudaLaunchCooperativeKernel(fn, dim3(plan.ctas, world_), dim3(threads), params, smem, s);
        if (ce != cudaSuccess) {
            (void)cudaGetLastError();
            return Fail(Result::CudaError, std::string("cooperative launch failed: ") + cudaGetErrorString(ce));
        }
        last_.launches += 1;
        return Result::Success;
    }
    for (int i = 0; i < nlocal(); ++i) {
        if (nlocal() > 1 && cudaSetDevice(local_[i].device) != cudaSuccess) {
            (void)cudaGetLastError();
            return Fail(Result::CudaError, "cudaSetDevice failed");
        }
        cudaStream_t s = streams && streams[i] ? streams[i] : local_[i].stream;
        void* params[] = {&args[i]};
        static const bool profile = env::ProfileKernels();
        Local& l = local_[i];
        if (profile) {
            if (!l.prof_start) {
                cudaEventCreate(&l.prof_start);
                cudaEventCreate(&l.prof_stop);
            }
            cudaEventRecord(l.prof_start, s);
        }
        cudaError_t ce = cudaLaunchKernel(fn, dim3(plan.ctas), dim3(threads), params, smem, s);
        if (ce != cudaSuccess) {
            (void)cudaGetLastError();
            return Fail(Result::CudaError, std::string("kernel launch failed: ") + cudaGetErrorString(ce));
        }
        if (profile) {
            cudaEventRecord(l.prof_stop, s);
            l.prof_pending = true;
        }
        last_.launches += 1;
    }
    return Result::Success;
}

Result Communicator::Collective(const void* const* send, void* const* recv, uint64_t count, Dtype in, Dtype out,
                                const OpOptions& opt, const cudaStream_t* streams, uint32_t extra_flags) {
    if (poisoned_) return Fail(Result::Timeout, "communicator is poisoned by an earlier timeout; call Reset()");
    if (!send || !recv) return Fail(Result::InvalidArg, "null buffer table");
    if (count == 0) return Result::Success;
    for (int i = 0; i < nlocal(); ++i)
        if (!send[i] || !recv[i]) return Fail(Result::InvalidArg, "null buffer");
    if (count > (1ull << 40)) return Fail(Result::InvalidArg, "count too large");

    const bool rs_only = extra_flags & kFlagReduceScatterOnly, ag_only = extra_flags & kFlagAllGatherOnly;
    const uint64_t shard = ShardElems(count, world_);
    const uint64_t send_elems = ag_only ? shard : count, recv_elems = rs_only ? shard : count;
    const uint64_t send_bytes = send_elems * DtypeSize(in), recv_bytes = recv_elems * DtypeSize(out);

    CollArgs* const args = args_scratch_.data();  // reused: no allocation on the per-call path
    std::memset(args, 0, sizeof(CollArgs) * args_scratch_.size());
    bool peer_recv = false, symmetric = false;
    Result r = ResolvePeers(send, recv, send_bytes, recv_bytes, opt.buffers_stable, args, &peer_recv, &symmetric);
    if (r != Result::Success) return r;
    bool in_place = false;
    for (int i = 0; i < nlocal(); ++i) {
        const char* s0 = static_cast<const char*>(send[i]);
        const char* r0 = static_cast<const char*>(recv[i]);
        if (s0 < r0 + recv_bytes && r0 < s0 + send_bytes) in_place = true;
    }

    PlanCaps caps;
    caps.flash_cap = lay_.flash_cap;
    caps.ring_bytes = lay_.ring_bytes;
    caps.nvls_cap = lay_.nvls_cap;
    caps.ll_cap = lay_.ll_cap;
    caps.has_multicast = has_multicast();
    caps.symmetric = symmetric;
    caps.peer_recv = peer_recv && !rs_only;
    caps.peer_send = peer_recv;  // ResolvePeers fills both tables or neither
    caps.in_place = in_place;
    // One process that drives several GPUs issues the ranks' work one after the other; the copy-engine
    // path's kernels wait for the peers' kernels, and on 2 x B200 rank 0 ran into its deadline before
    // the host got to launch rank 1.  One process per rank only.
    caps.one_gpu_per_rank = !emulated_ && nlocal() == 1;
    caps.half_collective = rs_only || ag_only;
    caps.sm_count = sm_count_;
    caps.max_ctas = max_ctas_;
    caps.force_ctas = opt.ctas > 0 ? static_cast<uint32_t>(opt.ctas) : 0u;
    caps.force_slot_bytes = opt.slot_bytes > 0 ? static_cast<uint32_t>(opt.slot_bytes) : 0u;
    caps.vec_ok = true;
    for (int i = 0; i < nlocal(); ++i) caps.vec_ok = caps.vec_ok && Aligned16(send[i]) && Aligned16(recv[i]);

    KernelMode mode = opt.mode;
    if (mode == KernelMode::Auto) mode = env::ForcedKernelMode();
    if (rs_only || ag_only) mode = KernelMode::Stream;
    Plan plan;
    std::string why;
    r = MakePlan(world_, count, in, out, opt.epilogue, mode, caps, EnvTuningTable(), &plan, &why);
    if (r != Result::Success) return Fail(r, why);
    if (world_ == 1 && plan.variant != Variant::Flash)
        return Fail(Result::Unsupported, "a single rank only runs the one-shot kernel");

    EpilogueParams ep;
    std::memset(&ep, 0, sizeof(ep));
    ep.scale = opt.epilogue == kEpiScaleCast ? opt.scale : 1.0f;
    if (opt.epilogue == kEpiResidualRmsNorm) {
        const int vec = 16 / static_cast<int>(DtypeSize(in));
        if (in != out || opt.hidden <= 0 || count % opt.hidden != 0 || opt.hidden % vec != 0 ||
            opt.hidden / vec > 4 * kFlashThreads || !opt.weight || !caps.vec_ok)
            return Fail(Result::Unsupported,
                        "fused RMSNorm needs equal in/out dtype, count a multiple of hidden, hidden a multiple of "
                        "16 bytes and at most 4*512 vectors, 16-byte aligned buffers and a weight");
        plan.ctas = static_cast<uint32_t>(std::min<uint64_t>(plan.ctas, count / opt.hidden));
        ep.eps = opt.eps;
        ep.hidden = opt.hidden;
    }

    // Call numbers (one-shot epoch, ring sequence base, barrier epoch) live in each rank's heap
    // and are advanced by the kernels; the host keeps no per-call state.
    plan.flags |= extra_flags;
    if (trace_) plan.flags |= kFlagTrace;
    // The staged kernels (one-shot incl. flag-in-data, ring without direct all-gather, staged NVLS)
    // treat alignment as a per-rank property: their partition of the message does not depend on it
    // and a rank touches nothing but its own buffers and the (aligned) staging.  The ring kernel's
    // direct all-gather and the pipelined kernels store 16-byte vectors into the peers' outputs and
    // use the flag all local ranks share.
    const bool per_rank_alignment =
        plan.variant == Variant::Flash ||
        ((plan.variant == Variant::NvlsOneShot || plan.variant == Variant::NvlsTwoShot) && !(plan.flags & kFlagSymmetric)) ||
        (plan.variant == Variant::Stream && !(plan.flags & kFlagDirectAg));
    for (int i = 0; i < nlocal(); ++i) {
        CollArgs& a = args[i];
        a.cv = View(i);
        a.send = send[i];
        a.recv = recv[i];
        a.count = count;
        a.stages = plan.stages;
        a.plan_word = PlanWord(static_cast<int>(plan.variant) * 2 + ((plan.flags & kFlagLowLatency) ? 1 : 0), plan.ctas, count);
        a.ctas = plan.ctas;
        a.slot_bytes = plan.slot_bytes;
        a.shard_elems = plan.shard_elems;
        a.flags = plan.flags;
        if (per_rank_alignment) {
            if (!(Aligned16(send[i]) && Aligned16(recv[i]))) a.flags &= ~static_cast<uint32_t>(kFlagVecOk);
            else a.flags |= kFlagVecOk;
        }
        if (opt.skip_rank >= 0 && local_[i].rank == opt.skip_rank) a.flags |= kFlagSkipRank;
        a.ep = ep;
        if (opt.epilogue == kEpiResidualRmsNorm) {
            a.ep.residual = opt.residual ? opt.residual[i] : nullptr;
            a.ep.residual_out = opt.residual_out ? opt.residual_out[i] : nullptr;
            a.ep.weight = opt.weight[i];
        }
    }
    last_.variant = plan.variant;
    last_.ctas = plan.ctas;
    last_.slot_bytes = plan.slot_bytes;
    last_.stages = plan.stages;
    last_.flags = plan.flags;
    static const int debug_level = env::DebugLevel();
    if (debug_level > 1 && local_[0].rank == 0)
        std::fprintf(stderr, "[yali] %s count=%llu ctas=%u slot=%u stages=%u flags=0x%x\n", VariantName(plan.variant),
                     static_cast<unsigned long long>(count), plan.ctas, plan.slot_bytes, plan.stages, plan.flags);
    return Launch(plan, in, out, opt.epilogue, args, streams);
}

Result Communicator::AllReduce(const void* const* send, void* const* recv, uint64_t count, Dtype in, Dtype out,
                               const OpOptions& opt, const cudaStream_t* streams) {
    YALI_NVTX_RANGE("yali::AllReduce");
    // The row-wise epilogue is fused into the one-shot kernel only.  A message beyond its
    // staging capacity is reduced by the bandwidth kernels first and normalised by a local
    // kernel afterwards (two launches per rank).
    if (opt.epilogue == kEpiResidualRmsNorm && world_ > 1 && count * DtypeSize(in) > lay_.flash_cap && in == out &&
        opt.hidden > 0 && count % opt.hidden == 0 && opt.weight) {
        OpOptions plain = opt;
        plain.epilogue = kEpiIdentity;
        if (plain.mode == KernelMode::Flash) plain.mode = KernelMode::Auto;
        Result r = Collective(send, recv, count, in, out, plain, streams, 0);
        if (r != Result::Success) return r;
        for (int i = 0; i < nlocal(); ++i) {
            if (nlocal() > 1) cudaSetDevice(local_[i].device);
            cudaStream_t s = streams && streams[i] ? streams[i] : local_[i].stream;
            if (emulated_) s = streams && streams[0] ? streams[0] : local_[0].stream;
            cudaError_t e = ResidualRmsNormInPlace(recv[i], opt.residual ? opt.residual[i] : nullptr,
                                                   opt.residual_out ? opt.residual_out[i] : nullptr, opt.weight[i],
                                                   count / opt.hidden, static_cast<uint32_t>(opt.hidden), opt.eps, out, s);
            if (e != cudaSuccess) return Fail(Result::CudaError, std::string("rmsnorm kernel: ") + cudaGetErrorString(e));
            last_.launches += 1;
        }
        return Result::Success;
    }
    return Collective(send, recv, count, in, out, opt, streams, 0);
}

Result Communicator::ReduceScatter(const void* const* send, void* const* recv, uint64_t count, Dtype dt,
                                   const OpOptions& opt, const cudaStream_t* streams) {
    YALI_NVTX_RANGE("yali::ReduceScatter");
    if (world_ == 1) return Collective(send, recv, count, dt, dt, opt, streams, 0);
    return Collective(send, recv, count, dt, dt, opt, streams, kFlagReduceScatterOnly);
}

Result Communicator::AllGather(const void* const* send, void* const* recv, uint64_t count, Dtype dt,
                               const OpOptions& opt, const cudaStream_t* streams) {
    YALI_NVTX_RANGE("yali::AllGather");
    if (world_ == 1) return Collective(send, recv, count, dt, dt, opt, streams, 0);
    return Collective(send, recv, count, dt, dt, opt, streams, kFlagAllGatherOnly);
}

Result Communicator::Check() {
    for (const Local& l : local_) {
        if (l.status && *reinterpret_cast<volatile uint32_t*>(&l.status->code) != 0) {
            poisoned_ = true;
            return Fail(Result::Timeout, DescribeStatus());
        }
    }
    return Result::Success;
}

Result Communicator::Sync(const cudaStream_t* streams) {
    YALI_NVTX_RANGE("yali::Sync");
    for (int i = 0; i < nlocal(); ++i) {
        if (nlocal() > 1) cudaSetDevice(local_[i].device);
        cudaStream_t s = streams && streams[i] ? streams[i] : local_[i].stream;
        cudaError_t e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return Fail(Result::CudaError, std::string("cudaStreamSynchronize: ") + cudaGetErrorString(e));
        }
        if (emulated_) break;  // one launch served every rank
    }
    // YALI_PROFILE_KERNELS=1: device time of the last launch, slowest rank of this process.
    float worst_ms = -1.f;
    for (Local& l : local_) {
        if (!l.prof_pending) continue;
        l.prof_pending = false;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, l.prof_start, l.prof_stop) == cudaSuccess) worst_ms = std::max(worst_ms, ms);
        else (void)cudaGetLastError();
    }
    if (worst_ms >= 0.f)
        std::fprintf(stderr, "[YALI_PROFILE] %s kernel: max_rank_ms=%.4f ctas=%u slot_bytes=%u\n",
                     VariantName(last_.variant), worst_ms, last_.ctas, last_.slot_bytes);
    return Check();
}

std::string Communicator::DescribeStatus() const {
    static const char* const sites[] = {"none",          "one-shot arrival", "ring credit", "reduce-scatter slot",
                                        "all-gather slot", "ring drain",       "CTA barrier", "GEMM partials",
                                        "GEMM done",     "mbarrier",         "copy-engine: peer entered",
                                        "copy-engine: peer read chunk", "copy-engine: peer finished"};
    for (const Local& l : local_) {
        const DeviceStatus s = *l.status;
        if (s.code == 0) continue;
        char buf[512];
        int len = std::snprintf(buf, sizeof(buf),
                                "rank %u gave up waiting for rank %u at '%s' (cta/lane %u): wanted %u, saw %u", s.rank, s.peer,
                                s.code < 13 ? sites[s.code] : "?", s.cta, s.wanted, s.observed);
        if (s.my_plan != 0 && s.peer_plan != 0 && s.my_plan != s.peer_plan) {
            static const char* const kernels[] = {"flash", "flash (flag in data)", "stream", "stream", "nvls1", "nvls1",
                                                  "nvls2", "nvls2", "flash_pull", "flash_pull", "stream_direct", "stream_direct",
                                                  "copy_engine", "copy_engine"};
            auto name = [&](uint32_t w) {
                const uint32_t k = (w >> 28) - 1;
                return k < 14 ? kernels[k] : "?";
            };
            std::snprintf(buf + len, sizeof(buf) - len,
                          "; the ranks ran different kernels (rank %u: %s on %u CTAs, rank %u: %s on %u CTAs): their "
                          "arguments differ (element count, dtype, or symmetric buffers on one rank only)",
                          s.rank, name(s.my_plan), (s.my_plan >> 16) & 0xfffu, s.peer, name(s.peer_plan),
                          (s.peer_plan >> 16) & 0xfffu);
        }
        return buf;
    }
    return "";
}

Result Communicator::Barrier() {
    YALI_NVTX_RANGE("yali::Barrier");
    for (const Local& l : local_) {
        cudaSetDevice(l.device);
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) return Fail(Result::CudaError, cudaGetErrorString(e));
    }
    if (bs_ && bs_->barrier() != Result::Success) return Fail(Result::BootstrapError, bs_->last_error());
    return Result::Success;
}

Result Communicator::Reset() {
    YALI_NVTX_RANGE("yali::Reset");
    Result r = Barrier();
    if (r != Result::Success) return r;
    for (const Local& l : local_) {
        cudaSetDevice(l.device);
        if (cudaMemset(heaps_->base(l.rank) + lay_.flags_off, 0, kFlagRegionBytes) != cudaSuccess ||
            cudaDeviceSynchronize() != cudaSuccess)
            return Fail(Result::CudaError, "clearing the flag region failed");
        std::memset(l.status, 0, sizeof(DeviceStatus));
    }
    flash_epoch_ = bar_epoch_ = stream_seq_ = gemm_epoch_ = 0;
    gemm_ = GemmCounters();
    poisoned_ = false;
    if (bs_ && bs_->barrier() != Result::Success) return Fail(Result::BootstrapError, bs_->last_error());
    return Result::Success;
}

}  // namespace yali
