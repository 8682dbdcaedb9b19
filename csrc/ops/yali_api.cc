#include <cstdio>

#include "../core/env.h"
#include "yali.h"

namespace yali {

cudaError_t ToCudaError(Result r) {
    switch (r) {
        case Result::Success: return cudaSuccess;
        case Result::InvalidArg: return cudaErrorInvalidValue;
        case Result::PeerAccessFailed: return cudaErrorPeerAccessUnsupported;
        case Result::NotInitialized: return cudaErrorInitializationError;
        case Result::Timeout: return cudaErrorTimeout;
        case Result::Unsupported: return cudaErrorNotSupported;
        case Result::BootstrapError: return cudaErrorSystemNotReady;
        case Result::CudaError: break;
    }
    return cudaErrorUnknown;
}

Comm::Comm(int gpu0, int gpu1) : Comm(std::vector<int>{gpu0, gpu1}) {}

Comm::Comm(const std::vector<int>& gpus, const CommOptions& opt) {
    Result r = Communicator::CreateSingleProcess(gpus, opt, &impl_, &err_);
    if (r != Result::Success) {
        impl_.reset();
        if (env::DebugLevel() > 0) std::fprintf(stderr, "[yali] Comm: %s (%s)\n", GetErrorString(r), err_.c_str());
    }
}

Comm Comm::Emulated(int world, int device, const CommOptions& opt) {
    Comm c;
    Result r = Communicator::CreateEmulated(world, device, opt, &c.impl_, &c.err_);
    if (r != Result::Success) c.impl_.reset();
    return c;
}

Comm::Comm(Comm&&) noexcept = default;
Comm& Comm::operator=(Comm&& o) noexcept {
    if (this != &o) {
        host_pipe_.reset();  // refers to the communicator that is about to go
        impl_ = std::move(o.impl_);
        host_pipe_ = std::move(o.host_pipe_);
        err_ = std::move(o.err_);
    }
    return *this;
}
Comm::~Comm() = default;

HostPipeline& Comm::host_pipeline() {
    if (!host_pipe_) host_pipe_ = std::make_unique<HostPipeline>(*impl_);
    return *host_pipe_;
}

cudaError_t allreduce_host_raw(Comm& comm, const void* const* send, void* const* recv, size_t count, Dtype dt,
                               const cudaStream_t* streams, bool sync, size_t chunk_bytes) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    Result r = comm.host_pipeline().AllReduce(send, recv, count, dt, OpOptions(), chunk_bytes, streams);
    if (r != Result::Success) return ToCudaError(r);
    return sync ? ToCudaError(comm.impl()->Sync(streams)) : cudaSuccess;
}

cudaError_t Comm::sync() {
    if (!impl_) return cudaErrorInitializationError;
    return ToCudaError(impl_->Sync());
}

cudaError_t allreduce_raw(Comm& comm, const void* const* send, void* const* recv, size_t count, Dtype dt,
                          const cudaStream_t* streams, bool sync, const OpOptions& opt, Dtype out_dt,
                          bool has_out_dt) {
    if (!comm.ok()) return cudaErrorInitializationError;
    Communicator* c = comm.impl();
    Result r = c->AllReduce(send, recv, count, dt, has_out_dt ? out_dt : dt, opt, streams);
    if (r != Result::Success) return ToCudaError(r);
    if (sync) return ToCudaError(c->Sync(streams));
    return cudaSuccess;
}

MPIComm::MPIComm(int* argc, char*** argv, const CommOptions& opt) {
    (void)argc;
    (void)argv;
    Result r = Result::Success;
    std::unique_ptr<Bootstrap> bs;
#ifdef YALI_MPI_SUPPORT
    bs = MakeMpiBootstrap(argc, argv, &r, &err_);
#else
    bs = MakeEnvBootstrap(&r, &err_);
#endif
    if (!bs) {
        std::fprintf(stderr, "yali::MPIComm: bootstrap failed: %s\n", err_.c_str());
        return;
    }
    rank_ = bs->rank();
    world_ = bs->world();
    local_rank_ = bs->local_rank();
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        (void)cudaGetLastError();
        err_ = "no CUDA device";
        std::fprintf(stderr, "yali::MPIComm: %s\n", err_.c_str());
        return;
    }
    r = Communicator::CreateMultiProcess(std::move(bs), local_rank_ % ndev, opt, &impl_, &err_);
    if (r != Result::Success) {
        impl_.reset();
        std::fprintf(stderr, "yali::MPIComm rank %d: %s (%s)\n", rank_, GetErrorString(r), err_.c_str());
    }
}

MPIComm::MPIComm(MPIComm&&) noexcept = default;
MPIComm& MPIComm::operator=(MPIComm&& o) noexcept {
    if (this != &o) {
        host_pipe_.reset();  // refers to the communicator that is about to go
        impl_ = std::move(o.impl_);
        host_pipe_ = std::move(o.host_pipe_);
        rank_ = o.rank_;
        world_ = o.world_;
        local_rank_ = o.local_rank_;
        err_ = std::move(o.err_);
    }
    return *this;
}
MPIComm::~MPIComm() = default;

HostPipeline& MPIComm::host_pipeline() {
    if (!host_pipe_) host_pipe_ = std::make_unique<HostPipeline>(*impl_);
    return *host_pipe_;
}

cudaError_t allreduce_host_raw(MPIComm& comm, const void* send, void* recv, size_t count, Dtype dt,
                               cudaStream_t stream, bool sync, size_t chunk_bytes) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    const void* s[1] = {send};
    void* r[1] = {recv};
    cudaStream_t st[1] = {stream};
    Result res = comm.host_pipeline().AllReduce(s, r, count, dt, OpOptions(), chunk_bytes, st);
    if (res != Result::Success) return ToCudaError(res);
    if (!sync) return cudaSuccess;
    cudaError_t e = cudaStreamSynchronize(stream ? stream : comm.stream());
    if (e != cudaSuccess) return e;
    return ToCudaError(comm.impl()->Check());
}

cudaError_t MPIComm::barrier() {
    if (!impl_) return cudaErrorInitializationError;
    return ToCudaError(impl_->Barrier());
}

cudaError_t MPIComm::sync() {
    if (!impl_) return cudaErrorInitializationError;
    return ToCudaError(impl_->Sync());
}

void* MPIComm::alloc(size_t bytes) {
    if (!impl_) return nullptr;
    std::vector<void*> p;
    if (impl_->SymmAlloc(bytes, &p) != Result::Success) {
        err_ = impl_->last_error();
        return nullptr;
    }
    return p[0];
}

cudaError_t MPIComm::exchange_buffer(const void* buf, size_t /*bytes*/) {
    if (!impl_) return cudaErrorInitializationError;
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, buf);
    if (e != cudaSuccess) return e;
    return attr.type == cudaMemoryTypeDevice ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t allreduce_raw(MPIComm& comm, const void* send, void* recv, size_t count, Dtype dt, cudaStream_t stream,
                          bool buffer_stable, const OpOptions& opt_in, Dtype out_dt, bool has_out_dt) {
    if (!comm.ok()) return cudaErrorInitializationError;
    OpOptions opt = opt_in;
    opt.buffers_stable = buffer_stable;
    const void* s[1] = {send};
    void* r[1] = {recv};
    cudaStream_t st[1] = {stream};
    return ToCudaError(comm.impl()->AllReduce(s, r, count, dt, has_out_dt ? out_dt : dt, opt, st));
}

}  // namespace yali
