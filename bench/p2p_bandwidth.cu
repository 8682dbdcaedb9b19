// p2p_bandwidth: device-to-device copy bandwidth between GPU pairs with the copy engines
// (cudaMemcpyPeerAsync), one direction and both directions at once, plus SM-driven remote stores
// (a kernel on the source writing into the destination), SM-driven remote loads (a kernel on the
// destination reading the source), the same through a pipeline of bulk-async copies into shared memory
// (cp.async.bulk + mbarrier, the access pattern of the pipelined all-reduce kernels), each in one
// direction and in both directions at once, and the two-shot mix (each GPU pulls one half and pushes
// the other).  These are the speed-of-light denominators the all-reduce results are compared against
// on the same box, and what decides between pulling and pushing in the planner.
//
//   p2p_bandwidth [bytes=1073741824] [iters=10] [gpu_a=0] [gpu_b=1]
//
// Reference counterpart: the nvbandwidth runs of `make hw-baseline` (device_to_device_memcpy_read_ce,
// device_to_device_bidirectional_memcpy_*), which need the nvbandwidth submodule.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#define CK(x)                                                                                \
    do {                                                                                     \
        cudaError_t e_ = (x);                                                                \
        if (e_ != cudaSuccess) {                                                             \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            std::exit(1);                                                                    \
        }                                                                                    \
    } while (0)

__global__ void remote_store_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n) {
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (; i + 3 * stride < n; i += 4 * stride) {
        uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
        dst[i] = a;
        dst[i + stride] = b;
        dst[i + 2 * stride] = c;
        dst[i + 3 * stride] = d;
    }
    for (; i < n; i += stride) dst[i] = src[i];
}

// Bulk-async pull: one thread per CTA keeps `kStages` copies of `kChunk` bytes in flight from `src`
// (any GPU) into shared memory; eight warps move every arrived chunk on to `dst` with 16-byte stores.
constexpr int kStages = 6, kChunk = 8192, kTmaThreads = 288;
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i)  // bounded: gives up instead of spinning for ever
        if (mbar_try(bar, parity)) return true;
    return false;
}
__global__ void __launch_bounds__(kTmaThreads, 2) bulk_pull_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                                    size_t nvec) {
    extern __shared__ __align__(128) unsigned char stage[];
    __shared__ __align__(8) uint64_t full[kStages], empty[kStages];
    __shared__ int failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        failed = 0;
        for (int s = 0; s < kStages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full[s])), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&empty[s])), "r"(8) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const size_t chunk_vec = kChunk / 16, n_chunks = (nvec + chunk_vec - 1) / chunk_vec;
    volatile int* vfailed = &failed;
    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (size_t j = blockIdx.x; j < n_chunks; j += gridDim.x, ++it) {
                const int s = it % kStages;
                if (!mbar_wait(&empty[s], ((it / kStages) & 1u) ^ 1u)) { *vfailed = 1; break; }
                const size_t vb = j * chunk_vec;
                const uint32_t bytes = static_cast<uint32_t>((nvec - vb < chunk_vec ? nvec - vb : chunk_vec) * 16);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&full[s])), "r"(bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 smem_u32(stage + s * kChunk)), "l"(src + vb), "r"(bytes), "r"(smem_u32(&full[s])) : "memory");
            }
        }
    } else {
        uint32_t it = 0;
        for (size_t j = blockIdx.x; j < n_chunks; j += gridDim.x, ++it) {
            const int s = it % kStages;
            if (*vfailed || !mbar_wait(&full[s], (it / kStages) & 1u)) { *vfailed = 1; break; }
            const size_t vb = j * chunk_vec;
            const uint32_t nv = static_cast<uint32_t>(nvec - vb < chunk_vec ? nvec - vb : chunk_vec);
            for (uint32_t v = tid - 32; v < nv; v += kTmaThreads - 32)
                dst[vb + v] = *reinterpret_cast<const uint4*>(stage + s * kChunk + v * 16);
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
        }
    }
}

// Bulk-async push: one thread per CTA stages chunks of the local `src` in shared memory (bulk copy
// global -> shared) and sends every arrived chunk on to `dst` (any GPU) with a bulk copy shared ->
// global; a stage is reused once the copy out of it has read the shared memory.
__global__ void __launch_bounds__(64, 4) bulk_push_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t nvec) {
    extern __shared__ __align__(128) unsigned char stage[];
    __shared__ __align__(8) uint64_t full[kStages];
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full[s])), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const size_t chunk_vec = kChunk / 16, n_chunks = (nvec + chunk_vec - 1) / chunk_vec;
        const size_t mine = blockIdx.x < n_chunks ? (n_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        auto chunk_bytes = [&](size_t it) {
            const size_t vb = (blockIdx.x + it * gridDim.x) * chunk_vec;
            return static_cast<uint32_t>((nvec - vb < chunk_vec ? nvec - vb : chunk_vec) * 16);
        };
        auto load = [&](size_t it) {
            const int s = it % kStages;
            const size_t vb = (blockIdx.x + it * gridDim.x) * chunk_vec;
            const uint32_t bytes = chunk_bytes(it);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&full[s])), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             smem_u32(stage + s * kChunk)), "l"(src + vb), "r"(bytes), "r"(smem_u32(&full[s])) : "memory");
        };
        for (size_t it = 0; it < mine && it < static_cast<size_t>(kStages) - 1; ++it) load(it);
        for (size_t it = 0; it < mine; ++it) {
            const int s = it % kStages;
            if (!mbar_wait(&full[s], (it / kStages) & 1u)) break;
            const size_t vb = (blockIdx.x + it * gridDim.x) * chunk_vec;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + vb),
                         "r"(smem_u32(stage + s * kChunk)), "r"(chunk_bytes(it)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            // The stage loaded next is the one sent in the previous step: wait until that copy has read it.
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            if (it + kStages - 1 < mine) load(it + kStages - 1);
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}

int main(int argc, char** argv) {
    const size_t bytes = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : (1ull << 30);
    const int iters = argc > 2 ? std::atoi(argv[2]) : 10;
    const int ga = argc > 3 ? std::atoi(argv[3]) : 0, gb = argc > 4 ? std::atoi(argv[4]) : 1;
    int n = 0;
    CK(cudaGetDeviceCount(&n));
    if (n <= ga || n <= gb || ga == gb) {
        std::printf("{\"unavailable\":\"needs two distinct GPUs\"}\n");
        return 0;
    }
    int can = 0;
    CK(cudaDeviceCanAccessPeer(&can, ga, gb));
    if (!can) {
        std::printf("{\"unavailable\":\"no peer access between GPU %d and %d\"}\n", ga, gb);
        return 0;
    }
    void *a_src, *a_dst, *b_src, *b_dst;
    cudaStream_t sa, sb;
    cudaEvent_t a0, a1, b0, b1;
    CK(cudaSetDevice(ga));
    cudaDeviceEnablePeerAccess(gb, 0);
    (void)cudaGetLastError();
    CK(cudaMalloc(&a_src, bytes));
    CK(cudaMalloc(&a_dst, bytes));
    CK(cudaStreamCreate(&sa));
    CK(cudaEventCreate(&a0));
    CK(cudaEventCreate(&a1));
    CK(cudaSetDevice(gb));
    cudaDeviceEnablePeerAccess(ga, 0);
    (void)cudaGetLastError();
    CK(cudaMalloc(&b_src, bytes));
    CK(cudaMalloc(&b_dst, bytes));
    CK(cudaStreamCreate(&sb));
    CK(cudaEventCreate(&b0));
    CK(cudaEventCreate(&b1));

    cudaStream_t sa2, sb2;
    cudaEvent_t a2, b2;
    CK(cudaSetDevice(ga));
    CK(cudaStreamCreate(&sa2));
    CK(cudaEventCreate(&a2));
    CK(cudaSetDevice(gb));
    CK(cudaStreamCreate(&sb2));
    CK(cudaEventCreate(&b2));
    auto sync_both = [&]() {
        CK(cudaSetDevice(ga));
        CK(cudaDeviceSynchronize());
        CK(cudaSetDevice(gb));
        CK(cudaDeviceSynchronize());
    };
    // one direction, copy engine: A -> B
    CK(cudaSetDevice(ga));
    CK(cudaMemcpyPeerAsync(b_dst, gb, a_src, ga, bytes, sa));
    sync_both();
    CK(cudaSetDevice(ga));
    CK(cudaEventRecord(a0, sa));
    for (int i = 0; i < iters; ++i) CK(cudaMemcpyPeerAsync(b_dst, gb, a_src, ga, bytes, sa));
    CK(cudaEventRecord(a1, sa));
    sync_both();
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, a0, a1));
    const double uni = bytes * static_cast<double>(iters) / (ms * 1e-3) / 1e9;
    // both directions at once
    CK(cudaSetDevice(ga));
    CK(cudaEventRecord(a0, sa));
    CK(cudaSetDevice(gb));
    CK(cudaEventRecord(b0, sb));
    for (int i = 0; i < iters; ++i) {
        CK(cudaSetDevice(ga));
        CK(cudaMemcpyPeerAsync(b_dst, gb, a_src, ga, bytes, sa));
        CK(cudaSetDevice(gb));
        CK(cudaMemcpyPeerAsync(a_dst, ga, b_src, gb, bytes, sb));
    }
    CK(cudaSetDevice(ga));
    CK(cudaEventRecord(a1, sa));
    CK(cudaSetDevice(gb));
    CK(cudaEventRecord(b1, sb));
    sync_both();
    float msa = 0, msb = 0;
    CK(cudaEventElapsedTime(&msa, a0, a1));
    CK(cudaEventElapsedTime(&msb, b0, b1));
    const double bidir_each = bytes * static_cast<double>(iters) / ((msa > msb ? msa : msb) * 1e-3) / 1e9;
    // Kernel-driven transfers.  run(kernel on A, kernel on B): both GPUs at once when both are given;
    // the rate is bytes per GPU over the slower of the two.
    const size_t nvec = bytes / 16;
    CK(cudaFuncSetAttribute(bulk_pull_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStages * kChunk));
    CK(cudaFuncSetAttribute(bulk_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStages * kChunk));
    CK(cudaSetDevice(ga));
    CK(cudaFuncSetAttribute(bulk_pull_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStages * kChunk));
    CK(cudaFuncSetAttribute(bulk_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStages * kChunk));
    struct Job {
        int kind;  // 0 none, 1 ld/st kernel, 2 bulk pull kernel
        void* dst;
        const void* src;
        size_t nvec;
    };
    auto launch = [&](const Job& j, cudaStream_t st) {
        if (j.kind == 1)
            remote_store_kernel<<<148 * 4, 512, 0, st>>>(static_cast<uint4*>(j.dst), static_cast<const uint4*>(j.src), j.nvec);
        else if (j.kind == 2)
            bulk_pull_kernel<<<148 * 2, kTmaThreads, kStages * kChunk, st>>>(static_cast<uint4*>(j.dst),
                                                                              static_cast<const uint4*>(j.src), j.nvec);
        else if (j.kind == 3)
            bulk_push_kernel<<<148 * 4, 64, kStages * kChunk, st>>>(static_cast<uint4*>(j.dst),
                                                                     static_cast<const uint4*>(j.src), j.nvec);
    };
    auto run = [&](const Job& on_a, const Job& on_b, const Job& on_a2, const Job& on_b2, size_t bytes_per_gpu) {
        for (int rep = 0; rep < 2; ++rep) {  // first round warms up
            const int n_it = rep == 0 ? 1 : iters;
            sync_both();
            CK(cudaSetDevice(ga));
            CK(cudaEventRecord(a0, sa));
            CK(cudaSetDevice(gb));
            CK(cudaEventRecord(b0, sb));
            CK(cudaSetDevice(ga));
            CK(cudaStreamWaitEvent(sa2, a0, 0));
            CK(cudaSetDevice(gb));
            CK(cudaStreamWaitEvent(sb2, b0, 0));
            for (int i = 0; i < n_it; ++i) {  // the second job of a GPU runs beside the first, on a stream of its own
                CK(cudaSetDevice(ga));
                launch(on_a, sa);
                launch(on_a2, sa2);
                CK(cudaSetDevice(gb));
                launch(on_b, sb);
                launch(on_b2, sb2);
            }
            CK(cudaSetDevice(ga));
            CK(cudaEventRecord(a2, sa2));
            CK(cudaStreamWaitEvent(sa, a2, 0));
            CK(cudaEventRecord(a1, sa));
            CK(cudaSetDevice(gb));
            CK(cudaEventRecord(b2, sb2));
            CK(cudaStreamWaitEvent(sb, b2, 0));
            CK(cudaEventRecord(b1, sb));
            sync_both();
        }
        float ta = 0, tb = 0;
        CK(cudaEventElapsedTime(&ta, a0, a1));
        CK(cudaEventElapsedTime(&tb, b0, b1));
        const float t = ta > tb ? ta : tb;
        return bytes_per_gpu * static_cast<double>(iters) / (t * 1e-3) / 1e9;
    };
    const Job none{0, nullptr, nullptr, 0};
    const double sm_store = run(Job{1, b_dst, a_src, nvec}, none, none, none, bytes);
    const double sm_store_bi = run(Job{1, b_dst, a_src, nvec}, Job{1, a_dst, b_src, nvec}, none, none, bytes);
    const double sm_load = run(Job{1, a_dst, b_src, nvec}, none, none, none, bytes);
    const double sm_load_bi = run(Job{1, a_dst, b_src, nvec}, Job{1, b_dst, a_src, nvec}, none, none, bytes);
    const double bulk_load = run(Job{2, a_dst, b_src, nvec}, none, none, none, bytes);
    const double bulk_load_bi = run(Job{2, a_dst, b_src, nvec}, Job{2, b_dst, a_src, nvec}, none, none, bytes);
    const double bulk_push = run(Job{3, b_dst, a_src, nvec}, none, none, none, bytes);
    const double bulk_push_bi = run(Job{3, b_dst, a_src, nvec}, Job{3, a_dst, b_src, nvec}, none, none, bytes);
    // Two-shot mix: each GPU pulls the first half from its peer and pushes the second half to it, so
    // every link direction carries read responses and write data at once.
    const size_t half = nvec / 2;
    const char* a_src_c = static_cast<const char*>(a_src);
    const char* b_src_c = static_cast<const char*>(b_src);
    const double mix = run(Job{2, a_dst, b_src, half}, Job{2, b_dst, a_src, half},
                           Job{1, static_cast<char*>(b_dst) + half * 16, a_src_c + half * 16, nvec - half},
                           Job{1, static_cast<char*>(a_dst) + half * 16, b_src_c + half * 16, nvec - half}, bytes);
    std::printf("{\"bytes\":%zu,\"gpu_a\":%d,\"gpu_b\":%d,\"copy_engine_unidirectional_gbs\":%.1f,"
                "\"copy_engine_bidirectional_per_direction_gbs\":%.1f,\"sm_remote_store_gbs\":%.1f,"
                "\"sm_remote_store_bidirectional_gbs\":%.1f,\"sm_remote_load_gbs\":%.1f,"
                "\"sm_remote_load_bidirectional_gbs\":%.1f,\"bulk_pull_gbs\":%.1f,\"bulk_pull_bidirectional_gbs\":%.1f,"
                "\"bulk_push_gbs\":%.1f,\"bulk_push_bidirectional_gbs\":%.1f,"
                "\"pull_half_push_half_bidirectional_gbs\":%.1f}\n",
                bytes, ga, gb, uni, bidir_each, sm_store, sm_store_bi, sm_load, sm_load_bi, bulk_load, bulk_load_bi, bulk_push,
                bulk_push_bi, mix);
    return 0;
}
