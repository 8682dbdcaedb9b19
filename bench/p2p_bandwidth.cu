// p2p_bandwidth: device-to-device copy bandwidth between GPU pairs with the copy engines
// (cudaMemcpyPeerAsync), one direction and both directions at once, plus SM-driven remote stores
// (a kernel on the source writing into the destination).  These are the speed-of-light denominators
// the all-reduce results are compared against on the same box.
//
//   p2p_bandwidth [bytes=1073741824] [iters=10] [gpu_a=0] [gpu_b=1]
//
// Reference counterpart: the nvbandwidth runs of `make hw-baseline` (device_to_device_memcpy_read_ce,
// device_to_device_bidirectional_memcpy_*), which need the nvbandwidth submodule.
#include <cuda_runtime.h>

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
    // SM-driven remote stores A -> B
    CK(cudaSetDevice(ga));
    remote_store_kernel<<<148 * 4, 512, 0, sa>>>(static_cast<uint4*>(b_dst), static_cast<const uint4*>(a_src), bytes / 16);
    CK(cudaStreamSynchronize(sa));
    CK(cudaEventRecord(a0, sa));
    for (int i = 0; i < iters; ++i)
        remote_store_kernel<<<148 * 4, 512, 0, sa>>>(static_cast<uint4*>(b_dst), static_cast<const uint4*>(a_src), bytes / 16);
    CK(cudaEventRecord(a1, sa));
    CK(cudaStreamSynchronize(sa));
    CK(cudaEventElapsedTime(&ms, a0, a1));
    const double sm_store = bytes * static_cast<double>(iters) / (ms * 1e-3) / 1e9;
    std::printf("{\"bytes\":%zu,\"gpu_a\":%d,\"gpu_b\":%d,\"copy_engine_unidirectional_gbs\":%.1f,"
                "\"copy_engine_bidirectional_per_direction_gbs\":%.1f,\"sm_remote_store_gbs\":%.1f}\n",
                bytes, ga, gb, uni, bidir_each, sm_store);
    return 0;
}
