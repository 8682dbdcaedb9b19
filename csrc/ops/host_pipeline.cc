#include "host_pipeline.h"

#include "../core/nvtx.h"

#include <algorithm>
#include <string>

namespace yali {

namespace {
#define YALI_HP_CUDA(call)                                                                     \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            comm_.set_error(std::string(#call) + ": " + cudaGetErrorString(e_));               \
            return Result::CudaError;                                                          \
        }                                                                                      \
    } while (0)
}  // namespace

HostPipeline::~HostPipeline() {
    for (size_t i = 0; i < loc_.size(); ++i) {
        PerLocal& l = loc_[i];
        cudaSetDevice(comm_.device_of(static_cast<int>(i)));
        for (cudaStream_t s : {l.h2d, l.comp, l.d2h})
            if (s) cudaStreamDestroy(s);
        if (l.start) cudaEventDestroy(l.start);
        for (int k = 0; k < kSlots; ++k)
            for (cudaEvent_t e : {l.copied_in[k], l.reduced[k], l.copied_out[k]})
                if (e) cudaEventDestroy(e);
    }
}

Result HostPipeline::Prepare(uint64_t chunk_bytes) {
    const int nl = comm_.nlocal();
    if (loc_.empty()) {
        loc_.resize(nl);
        for (int i = 0; i < nl; ++i) {
            PerLocal& l = loc_[i];
            YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
            YALI_HP_CUDA(cudaStreamCreateWithFlags(&l.h2d, cudaStreamNonBlocking));
            YALI_HP_CUDA(cudaStreamCreateWithFlags(&l.comp, cudaStreamNonBlocking));
            YALI_HP_CUDA(cudaStreamCreateWithFlags(&l.d2h, cudaStreamNonBlocking));
            YALI_HP_CUDA(cudaEventCreateWithFlags(&l.start, cudaEventDisableTiming));
            for (int k = 0; k < kSlots; ++k) {
                YALI_HP_CUDA(cudaEventCreateWithFlags(&l.copied_in[k], cudaEventDisableTiming));
                YALI_HP_CUDA(cudaEventCreateWithFlags(&l.reduced[k], cudaEventDisableTiming));
                YALI_HP_CUDA(cudaEventCreateWithFlags(&l.copied_out[k], cudaEventDisableTiming));
            }
        }
    }
    // Symmetric memory is never freed piecemeal, so the staging buffers are sized by bytes (any
    // dtype fits), grow in powers of two and are reused by every later call that fits: a program
    // that alternates chunk sizes or dtypes holds at most twice its largest request.
    if (chunk_bytes > slot_bytes_) {
        uint64_t cap = 1ull << 20;
        while (cap < chunk_bytes) cap <<= 1;
        for (int k = 0; k < kSlots; ++k) {
            Result r = comm_.SymmAlloc(cap, &send_[k]);
            if (r != Result::Success) return r;
            r = comm_.SymmAlloc(cap, &recv_[k]);
            if (r != Result::Success) return r;
        }
        slot_bytes_ = cap;
    }
    return Result::Success;
}

Result HostPipeline::AllReduce(const void* const* src, void* const* dst, uint64_t count, Dtype dt,
                               const OpOptions& opt, uint64_t chunk_bytes, const cudaStream_t* user_streams,
                               bool copies_only) {
    YALI_NVTX_RANGE("yali::AllReduceHost");
    if (count == 0) return Result::Success;
    const int nl = comm_.nlocal();
    const uint64_t esz = DtypeSize(dt);
    for (int i = 0; i < nl; ++i)
        if (!src[i] || !dst[i]) {
            comm_.set_error("all_reduce_host: null buffer");
            return Result::InvalidArg;
        }
    if (opt.epilogue == kEpiResidualRmsNorm) {
        comm_.set_error("all_reduce_host: the row epilogue needs whole rows on the device; use AllReduce");
        return Result::Unsupported;
    }
    // Chunks are multiples of 256 elements so that every chunk keeps the 16-byte alignment of the
    // vector paths.
    // chunk_bytes == 0: about 32 chunks per message, between 1 and 8 MiB each: the first copy in and the
    // last copy out are not overlapped with anything, so they should be a small part of the whole.
    if (chunk_bytes == 0) chunk_bytes = std::min<uint64_t>(8ull << 20, std::max<uint64_t>(1ull << 20, count * esz / 32));
    uint64_t chunk = std::max<uint64_t>(256, (std::max<uint64_t>(chunk_bytes, esz) / esz) / 256 * 256);
    chunk = std::min<uint64_t>(chunk, (count + 255) / 256 * 256);
    Result pr = Prepare(chunk * esz);
    if (pr != Result::Success) return pr;

    int prev_dev = 0;
    cudaGetDevice(&prev_dev);
    // Everything queued so far on the caller's streams comes first.
    for (int i = 0; i < nl; ++i) {
        cudaStream_t us = user_streams && user_streams[i] ? user_streams[i] : comm_.default_stream(i);
        YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
        YALI_HP_CUDA(cudaEventRecord(loc_[i].start, us));
        for (cudaStream_t s : {loc_[i].h2d, loc_[i].comp, loc_[i].d2h}) YALI_HP_CUDA(cudaStreamWaitEvent(s, loc_[i].start, 0));
    }
    const uint64_t nchunks = (count + chunk - 1) / chunk;
    std::vector<const void*> s_in(nl);
    std::vector<void*> s_out(nl);
    std::vector<cudaStream_t> comp(nl);
    for (int i = 0; i < nl; ++i) comp[i] = loc_[i].comp;
    // Several local ranks may share one launch (emulated ranks) or wait for one another inside the
    // kernels, so a stage of chunk c on any local rank waits for the previous stage on ALL of them.
    for (uint64_t c = 0; c < nchunks; ++c) {
        const uint64_t lo = c * chunk, m = std::min(chunk, count - lo);
        const int k = static_cast<int>(c % kSlots);
        for (int i = 0; i < nl; ++i) {
            YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
            if (c >= kSlots)  // the slot's previous chunk has been reduced everywhere
                for (int j = 0; j < nl; ++j) YALI_HP_CUDA(cudaStreamWaitEvent(loc_[i].h2d, loc_[j].reduced[k], 0));
            YALI_HP_CUDA(cudaMemcpyAsync(send_[k][i], static_cast<const char*>(src[i]) + lo * esz, m * esz,
                                         cudaMemcpyHostToDevice, loc_[i].h2d));
            YALI_HP_CUDA(cudaEventRecord(loc_[i].copied_in[k], loc_[i].h2d));
        }
        for (int i = 0; i < nl; ++i) {
            YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
            for (int j = 0; j < nl; ++j) {
                YALI_HP_CUDA(cudaStreamWaitEvent(loc_[i].comp, loc_[j].copied_in[k], 0));
                if (c >= kSlots) YALI_HP_CUDA(cudaStreamWaitEvent(loc_[i].comp, loc_[j].copied_out[k], 0));
            }
            s_in[i] = send_[k][i];
            s_out[i] = recv_[k][i];
        }
        if (copies_only) {
            for (int i = 0; i < nl; ++i) {
                YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
                YALI_HP_CUDA(cudaMemcpyAsync(s_out[i], s_in[i], m * esz, cudaMemcpyDeviceToDevice, loc_[i].comp));
            }
        } else {
            Result r = comm_.AllReduce(s_in.data(), s_out.data(), m, dt, dt, opt, comp.data());
            if (r != Result::Success) {
                cudaSetDevice(prev_dev);
                return r;
            }
        }
        for (int i = 0; i < nl; ++i) {
            YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
            YALI_HP_CUDA(cudaEventRecord(loc_[i].reduced[k], loc_[i].comp));
        }
        for (int i = 0; i < nl; ++i) {
            YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
            for (int j = 0; j < nl; ++j) YALI_HP_CUDA(cudaStreamWaitEvent(loc_[i].d2h, loc_[j].reduced[k], 0));
            YALI_HP_CUDA(cudaMemcpyAsync(static_cast<char*>(dst[i]) + lo * esz, recv_[k][i], m * esz,
                                         cudaMemcpyDeviceToHost, loc_[i].d2h));
            YALI_HP_CUDA(cudaEventRecord(loc_[i].copied_out[k], loc_[i].d2h));
        }
    }
    // The caller's streams continue when the last chunk has left (copies on one stream are in order).
    const int last = static_cast<int>((nchunks - 1) % kSlots);
    for (int i = 0; i < nl; ++i) {
        cudaStream_t us = user_streams && user_streams[i] ? user_streams[i] : comm_.default_stream(i);
        YALI_HP_CUDA(cudaSetDevice(comm_.device_of(i)));
        YALI_HP_CUDA(cudaStreamWaitEvent(us, loc_[i].copied_out[last], 0));
    }
    cudaSetDevice(prev_dev);
    return Result::Success;
}

}  // namespace yali
