// Public C++ API: yali::Comm (one process drives 2..8 GPUs), yali::MPIComm (one
// GPU per process) and yali::allreduce.
//
// Parity: yali::Comm / yali::allreduce(comm, send0, recv0, send1, recv1, count,
// stream, sync) in src/ops/allreduce.cuh:78-323,563-810 and yali::MPIComm /
// yali::allreduce(comm, send, recv, count, stream, buffer_stable) in
// src/ops/allreduce_mpi.cuh:76-298,410-676.  The 2-GPU signatures are kept as
// they are; array forms cover 4 and 8 GPUs; fused forms (scale+cast, residual +
// RMSNorm, reduce-scatter, all-gather) are additions.  Link against
// libyali_b200.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <vector>

#include "../comm/communicator.h"
#include "host_pipeline.h"
#include "../core/status.h"

namespace yali {

template <typename T>
struct DtypeOf;
template <>
struct DtypeOf<float> {
    static constexpr Dtype value = Dtype::FP32;
};
template <>
struct DtypeOf<__half> {
    static constexpr Dtype value = Dtype::FP16;
};
template <>
struct DtypeOf<__nv_bfloat16> {
    static constexpr Dtype value = Dtype::BF16;
};

// Maps a library result onto the cudaError_t the reference's API returns.
cudaError_t ToCudaError(Result r);

// ---------------------------------------------------------------- single process
class Comm {
   public:
    // Two GPUs (the reference's constructor).
    Comm(int gpu0, int gpu1);
    // 1..8 GPUs.
    explicit Comm(const std::vector<int>& gpus, const CommOptions& opt = CommOptions());
    // `world` ranks emulated on one GPU (testing aid; see Communicator).
    static Comm Emulated(int world, int device = 0, const CommOptions& opt = CommOptions());
    Comm(Comm&&) noexcept;
    Comm& operator=(Comm&&) noexcept;
    Comm(const Comm&) = delete;
    Comm& operator=(const Comm&) = delete;
    ~Comm();

    bool ok() const { return impl_ != nullptr; }
    int world_size() const { return impl_ ? impl_->world() : 0; }
    int gpu(int rank) const { return impl_->device_of(rank); }
    // Waits for all collectives issued through this communicator; reports device-side timeouts.
    cudaError_t sync();
    Result reset() { return impl_->Reset(); }
    const std::string& error() const { return err_; }
    Communicator* impl() const { return impl_.get(); }
    // Pipeline behind allreduce_host (created on first use).
    HostPipeline& host_pipeline();

   private:
    Comm() = default;
    std::unique_ptr<Communicator> impl_;
    std::unique_ptr<HostPipeline> host_pipe_;  // declared after impl_: destroyed before it
    std::string err_;
};

// Non-template cores.
cudaError_t allreduce_raw(Comm& comm, const void* const* send, void* const* recv, size_t count, Dtype dt,
                          const cudaStream_t* streams, bool sync, const OpOptions& opt = OpOptions(),
                          Dtype out_dt = Dtype::FP32, bool has_out_dt = false);

// The reference's 2-GPU form.  `stream` 0 means the communicator's own stream of
// each GPU; a non-zero stream must belong to GPU 0 and is then used for GPU 0 only.
template <typename T>
cudaError_t allreduce(Comm& comm, const T* send0, T* recv0, const T* send1, T* recv1, size_t count,
                      cudaStream_t stream = nullptr, bool sync = true) {
    if (!comm.ok() || comm.world_size() != 2) return cudaErrorInvalidValue;
    const void* s[2] = {send0, send1};
    void* r[2] = {recv0, recv1};
    cudaStream_t st[2] = {stream, nullptr};
    return allreduce_raw(comm, s, r, count, DtypeOf<T>::value, st, sync);
}

// N-GPU form: one send / recv pointer per rank, optionally one stream per rank.
template <typename T>
cudaError_t allreduce(Comm& comm, const T* const* send, T* const* recv, size_t count,
                      const cudaStream_t* streams = nullptr, bool sync = true) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    return allreduce_raw(comm, reinterpret_cast<const void* const*>(send), reinterpret_cast<void* const*>(recv), count,
                         DtypeOf<T>::value, streams, sync);
}

// Gradient form: recv = cast<Tout>(scale * sum).
template <typename Tin, typename Tout>
cudaError_t allreduce_scale_cast(Comm& comm, const Tin* const* send, Tout* const* recv, size_t count, float scale,
                                 const cudaStream_t* streams = nullptr, bool sync = true) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    OpOptions opt;
    opt.epilogue = kEpiScaleCast;
    opt.scale = scale;
    return allreduce_raw(comm, reinterpret_cast<const void* const*>(send), reinterpret_cast<void* const*>(recv), count,
                         DtypeOf<Tin>::value, streams, sync, opt, DtypeOf<Tout>::value, true);
}

// Tensor-parallel form: recv = RMSNorm(sum + residual) * weight over rows of `hidden`.
template <typename T>
cudaError_t allreduce_residual_rmsnorm(Comm& comm, const T* const* send, T* const* recv, size_t rows, int hidden,
                                       const T* const* residual, T* const* residual_out, const T* const* weight,
                                       float eps, const cudaStream_t* streams = nullptr, bool sync = true) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    OpOptions opt;
    opt.epilogue = kEpiResidualRmsNorm;
    opt.hidden = hidden;
    opt.eps = eps;
    opt.residual = reinterpret_cast<const void* const*>(residual);
    opt.residual_out = reinterpret_cast<void* const*>(residual_out);
    opt.weight = reinterpret_cast<const void* const*>(weight);
    return allreduce_raw(comm, reinterpret_cast<const void* const*>(send), reinterpret_cast<void* const*>(recv),
                         rows * static_cast<size_t>(hidden), DtypeOf<T>::value, streams, sync, opt);
}

// Host-resident data: send / recv are page-locked host buffers (one per rank).  The copies of both
// directions and the all-reduce overlap chunk by chunk (ops/host_pipeline.h); no counterpart in the
// reference, whose ops take device pointers only.
cudaError_t allreduce_host_raw(Comm& comm, const void* const* send, void* const* recv, size_t count, Dtype dt,
                               const cudaStream_t* streams, bool sync, size_t chunk_bytes);
template <typename T>
cudaError_t allreduce_host(Comm& comm, const T* const* send, T* const* recv, size_t count,
                           const cudaStream_t* streams = nullptr, bool sync = true, size_t chunk_bytes = 0) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    return allreduce_host_raw(comm, reinterpret_cast<const void* const*>(send), reinterpret_cast<void* const*>(recv),
                              count, DtypeOf<T>::value, streams, sync, chunk_bytes);
}

// ---------------------------------------------------------------- one GPU per process
class MPIComm {
   public:
    // Joins the job described by the launcher's environment (RANK / WORLD_SIZE /
    // LOCAL_RANK / MASTER_PORT from torchrun or the bundled `yalirun`; OMPI_* /
    // PMI_* / SLURM_* from an MPI launcher) or, when built with YALI_MPI_SUPPORT,
    // through MPI_Init.  argc/argv are only used by the MPI build.
    MPIComm(int* argc, char*** argv, const CommOptions& opt = CommOptions());
    MPIComm(MPIComm&&) noexcept;
    MPIComm& operator=(MPIComm&&) noexcept;
    MPIComm(const MPIComm&) = delete;
    MPIComm& operator=(const MPIComm&) = delete;
    ~MPIComm();

    bool ok() const { return impl_ != nullptr; }
    int rank() const { return rank_; }
    int world_size() const { return world_; }
    int local_rank() const { return local_rank_; }
    cudaStream_t stream() const { return impl_->default_stream(0); }
    // Drains this rank's GPU work, then a host barrier across the ranks.
    cudaError_t barrier();
    cudaError_t sync();
    Result reset() { return impl_->Reset(); }
    // Symmetric (pre-allocated, zero-copy) buffer: same offset on every rank.  Collective.
    void* alloc(size_t bytes);
    // Kept for source compatibility: buffers need no per-call exchange here.  Returns
    // success when `buf` is either a symmetric buffer or an ordinary device buffer.
    cudaError_t exchange_buffer(const void* buf, size_t bytes);
    const std::string& error() const { return err_; }
    Communicator* impl() const { return impl_.get(); }
    HostPipeline& host_pipeline();

   private:
    std::unique_ptr<Communicator> impl_;
    std::unique_ptr<HostPipeline> host_pipe_;  // declared after impl_: destroyed before it
    int rank_ = 0, world_ = 1, local_rank_ = 0;
    std::string err_;
};

cudaError_t allreduce_raw(MPIComm& comm, const void* send, void* recv, size_t count, Dtype dt, cudaStream_t stream,
                          bool buffer_stable, const OpOptions& opt = OpOptions(), Dtype out_dt = Dtype::FP32,
                          bool has_out_dt = false);

// The reference's form.  The call returns once the kernel is enqueued on `stream`
// (0: the communicator's stream) and that stream has been synchronised, as the
// reference does; use allreduce_async to keep it asynchronous.
template <typename T>
cudaError_t allreduce(MPIComm& comm, const T* send, T* recv, size_t count, cudaStream_t stream = nullptr,
                      bool buffer_stable = false) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    cudaError_t e = allreduce_raw(comm, send, recv, count, DtypeOf<T>::value, stream, buffer_stable);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream ? stream : comm.stream());
    if (e != cudaSuccess) return e;
    return ToCudaError(comm.impl()->Check());
}
cudaError_t allreduce_host_raw(MPIComm& comm, const void* send, void* recv, size_t count, Dtype dt,
                               cudaStream_t stream, bool sync, size_t chunk_bytes);
// Page-locked host buffers in and out; synchronises `stream` (0: the communicator's) unless sync is false.
template <typename T>
cudaError_t allreduce_host(MPIComm& comm, const T* send, T* recv, size_t count, cudaStream_t stream = nullptr,
                           bool sync = true, size_t chunk_bytes = 0) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    return allreduce_host_raw(comm, send, recv, count, DtypeOf<T>::value, stream, sync, chunk_bytes);
}
template <typename T>
cudaError_t allreduce_async(MPIComm& comm, const T* send, T* recv, size_t count, cudaStream_t stream = nullptr) {
    if (!comm.ok()) return cudaErrorInvalidValue;
    return allreduce_raw(comm, send, recv, count, DtypeOf<T>::value, stream, true);
}

}  // namespace yali
