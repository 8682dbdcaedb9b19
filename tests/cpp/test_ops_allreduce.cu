// Integration tests of the C++ API in one process: peer-access helpers, yali::Comm +
// yali::allreduce on two GPUs (constant fills as in the reference, then seeded random
// data), the N-GPU array form, fused forms, the large-message (two-shot) path, a
// bandwidth floor.  With one GPU the multi-GPU cases run on emulated ranks.
// Reference counterparts: tests/test_ops_allreduce.cu, tests/test_bw_ops.cu,
// tests/unit/test_peer_access.cu, tests/unit/test_all_reduce_correctness.cu:106-159.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <chrono>
#include <algorithm>
#include <cmath>
#include <vector>

#include "comm/topology.h"
#include "ops/buffer_ops.h"
#include "ops/yali.h"
#include "test_framework.h"

using namespace yali;

TEST(peer_access_helpers) {
    if (!ytest::HasNGPUs(2)) SKIP_TEST("needs 2 GPUs");
    P2PCapability cap = CheckP2PAccess(0, 1);
    EXPECT_EQ(cap.bidirectional, cap.can_access_0_to_1 && cap.can_access_1_to_0);
    if (!cap.bidirectional) SKIP_TEST("no peer access between GPU 0 and 1");
    EXPECT_TRUE(EnableBidirectionalP2P(0, 1));
    EXPECT_TRUE(EnableBidirectionalP2P(0, 1));  // idempotent
    TopologyInfo t = QueryTopology();
    EXPECT_GE(t.device_count, 2);
    EXPECT_LE(t.ConnectedPairs(), t.device_count * (t.device_count - 1) / 2);
    // peer memcpy works once access is on
    float *a, *b;
    cudaSetDevice(0);
    CUDA_CHECK(cudaMalloc(&a, 1024));
    cudaSetDevice(1);
    CUDA_CHECK(cudaMalloc(&b, 1024));
    CUDA_CHECK(cudaMemcpyPeer(b, 1, a, 0, 1024));
    cudaFree(b);
    cudaSetDevice(0);
    cudaFree(a);
}

TEST(nvlink_and_sol) {
    NVLinkInfo nv = NVLinkConfigForComputeCapability(10, 0);
    EXPECT_TRUE(nv.valid);
    EXPECT_EQ(nv.linkCount, 18);
    EXPECT_NEAR(nv.unidirectionalGBs, 900.0, 1e-9);
    SoLMetrics m = CalculateSoL(1ull << 30, 1e-3, 8, nv);
    EXPECT_NEAR(m.algBwGBs, 1073.741824, 1e-6);
    EXPECT_NEAR(m.busBwGBs, m.algBwGBs * 1.75, 1e-6);
    EXPECT_NEAR(m.solPercent, 100.0 * m.busBwGBs / 900.0, 1e-9);
    EXPECT_NEAR(BusBwFactor(2), 1.0, 1e-12);
}

template <typename T>
static void TwoGpuConstant(Comm& comm, size_t n, Dtype dt, float tol) {
    T *s0, *r0, *s1, *r1;
    const int d0 = comm.gpu(0), d1 = comm.gpu(1);
    cudaSetDevice(d0);
    AllocAndSeed(reinterpret_cast<void**>(&s0), n, dt, 1.0f);
    AllocAndSeed(reinterpret_cast<void**>(&r0), n, dt, 0.0f);
    cudaSetDevice(d1);
    AllocAndSeed(reinterpret_cast<void**>(&s1), n, dt, 2.0f);
    AllocAndSeed(reinterpret_cast<void**>(&r1), n, dt, 0.0f);
    EXPECT_TRUE(allreduce(comm, s0, r0, s1, r1, n) == cudaSuccess);
    std::vector<float> h(n);
    cudaSetDevice(d0);
    EXPECT_TRUE(ConvertBufferToFloat(r0, h.data(), n, dt) == cudaSuccess);
    EXPECT_TRUE(VerifyAllReduceSum(h.data(), n, 3.0f, tol, nullptr, nullptr));
    cudaSetDevice(d1);
    EXPECT_TRUE(ValidateRankResult(r1, n, dt, 1, 2));
    cudaFree(s1);
    cudaFree(r1);
    cudaSetDevice(d0);
    cudaFree(s0);
    cudaFree(r0);
}

static Comm MakeComm(int world) {
    if (ytest::HasNGPUs(world)) {
        std::vector<int> g(world);
        for (int i = 0; i < world; ++i) g[i] = i;
        return Comm(g);
    }
    return Comm::Emulated(world, 0);
}

TEST(two_gpu_api_constant_fills) {
    if (!ytest::HasNGPUs(1)) SKIP_TEST("needs a GPU");
    Comm comm = MakeComm(2);
    EXPECT_TRUE(comm.ok());
    if (!comm.ok()) return;
    TwoGpuConstant<float>(comm, 1024, Dtype::FP32, 1e-5f);
    TwoGpuConstant<float>(comm, 1 << 20, Dtype::FP32, 1e-5f);
    TwoGpuConstant<__half>(comm, 1 << 20, Dtype::FP16, 0.01f);
    TwoGpuConstant<__nv_bfloat16>(comm, 1 << 20, Dtype::BF16, 0.01f);
}

template <typename T>
static void RandomN(Comm& comm, size_t n, Dtype dt, bool scale_cast) {
    const int W = comm.world_size();
    std::vector<T*> send(W), recv(W);
    for (int i = 0; i < W; ++i) {
        cudaSetDevice(comm.gpu(i));
        cudaMalloc(&send[i], n * sizeof(T));
        cudaMalloc(&recv[i], n * sizeof(T));
        FillRandom(send[i], n, dt, kDistNormal, 1234 + i, nullptr);
        cudaDeviceSynchronize();
    }
    const float scale = scale_cast ? 1.0f / W : 1.0f;
    cudaError_t e = scale_cast ? allreduce_scale_cast<T, T>(comm, send.data(), recv.data(), n, scale)
                               : allreduce<T>(comm, send.data(), recv.data(), n);
    EXPECT_TRUE(e == cudaSuccess);
    for (int i = 0; i < W; ++i) {
        cudaSetDevice(comm.gpu(i));
        EXPECT_TRUE(ValidateRandomResult(recv[i], n, dt, dt, kDistNormal, 1234, W, scale, nullptr));
        cudaFree(send[i]);
        cudaFree(recv[i]);
    }
}

TEST(n_gpu_api_random_data) {
    if (!ytest::HasNGPUs(1)) SKIP_TEST("needs a GPU");
    for (int world : {2, 4, 8}) {
        Comm comm = MakeComm(world);
        EXPECT_TRUE(comm.ok());
        if (!comm.ok()) continue;
        RandomN<float>(comm, 4099, Dtype::FP32, false);
        RandomN<__nv_bfloat16>(comm, 1 << 20, Dtype::BF16, false);
        RandomN<__half>(comm, 300001, Dtype::FP16, true);
        RandomN<float>(comm, (32u << 20) + 12, Dtype::FP32, false);  // 128 MiB: the two-shot path
    }
}

// Page-locked host buffers in and out: the chunked three-stream pipeline must give the plain sum.
TEST(host_to_host_allreduce) {
    if (!ytest::HasNGPUs(1)) SKIP_TEST("needs a GPU");
    for (int world : {2, 4}) {
        Comm comm = MakeComm(world);
        EXPECT_TRUE(comm.ok());
        if (!comm.ok()) continue;
        const size_t n = 5 * 65536 + 123;  // six chunks of 256 KiB: more chunks than staging slots
        std::vector<float*> src(world), dst(world);
        for (int i = 0; i < world; ++i) {
            EXPECT_TRUE(cudaMallocHost(&src[i], n * sizeof(float)) == cudaSuccess);
            EXPECT_TRUE(cudaMallocHost(&dst[i], n * sizeof(float)) == cudaSuccess);
            for (size_t k = 0; k < n; ++k) src[i][k] = static_cast<float>((k * 7 + i * 13) % 101) * 0.25f - 3.0f;
        }
        for (int rep = 0; rep < 2; ++rep) {
            for (int i = 0; i < world; ++i) std::fill(dst[i], dst[i] + n, -1.0f);
            cudaError_t e = allreduce_host<float>(comm, src.data(), dst.data(), n, nullptr, true, 256u << 10);
            EXPECT_TRUE(e == cudaSuccess);
            size_t bad = 0;
            for (size_t k = 0; k < n; ++k) {
                float want = 0.f;
                for (int i = 0; i < world; ++i) want += src[i][k];
                for (int i = 0; i < world; ++i) bad += std::fabs(dst[i][k] - want) > 1e-4f;
            }
            EXPECT_EQ(bad, static_cast<size_t>(0));
        }
        for (int i = 0; i < world; ++i) {
            cudaFreeHost(src[i]);
            cudaFreeHost(dst[i]);
        }
    }
}

TEST(bandwidth_floor_64MiB) {
    if (!ytest::HasNGPUs(2)) SKIP_TEST("needs 2 GPUs");
    Comm comm(0, 1);
    EXPECT_TRUE(comm.ok());
    if (!comm.ok()) return;
    const size_t n = 16u << 20;
    float *s0, *r0, *s1, *r1;
    cudaSetDevice(0);
    cudaMalloc(&s0, n * 4);
    cudaMalloc(&r0, n * 4);
    cudaSetDevice(1);
    cudaMalloc(&s1, n * 4);
    cudaMalloc(&r1, n * 4);
    for (int i = 0; i < 3; ++i) allreduce(comm, s0, r0, s1, r1, n);
    auto t0 = std::chrono::steady_clock::now();
    const int iters = 10;
    for (int i = 0; i < iters; ++i) allreduce(comm, s0, r0, s1, r1, n, nullptr, false);
    comm.sync();
    double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() / iters;
    double gbps = n * 4.0 / sec / 1e9;
    std::printf("    64 MiB through the ops API: %.1f GB/s\n", gbps);
    EXPECT_GE(gbps, 100.0);  // the reference's floor is 30 GB/s on 2x A100 NV2
    cudaFree(s1);
    cudaFree(r1);
    cudaSetDevice(0);
    cudaFree(s0);
    cudaFree(r0);
}

int main() { return RUN_ALL_TESTS(); }
