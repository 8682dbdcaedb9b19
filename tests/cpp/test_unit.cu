// Host-only and one-GPU unit tests: types and names, interface defaults, tuning ranges,
// value conversions, buffer utilities, conversion + host verification.
// Reference counterparts: tests/unit/test_all_reduce_interface.cu, test_dtypes.cu,
// test_buffer_ops.cu, test_validation.cu, test_all_reduce_correctness.cu:165-208.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <vector>

#include "core/status.h"
#include "ops/buffer_ops.h"
#include "ops/tuning.h"
#include "test_framework.h"

using namespace yali;

TEST(result_and_dtype_names) {
    EXPECT_TRUE(std::string(GetErrorString(Result::Success)) == "Success");
    EXPECT_TRUE(std::string(GetErrorString(Result::Timeout)).find("timed out") != std::string::npos);
    EXPECT_EQ(DtypeSize(Dtype::FP32), 4u);
    EXPECT_EQ(DtypeSize(Dtype::FP16), 2u);
    EXPECT_EQ(DtypeSize(Dtype::BF16), 2u);
    EXPECT_TRUE(std::string(DtypeName(Dtype::BF16)) == "bf16");
    EXPECT_EQ(ElementSize(DataType::Float16), 2u);
    EXPECT_TRUE(std::string(DataTypeName(DataType::Float32)) == "fp32");
    EXPECT_TRUE(std::string(KernelModeName(KernelMode::Auto)) == "auto");
    EXPECT_TRUE(std::string(KernelModeName(KernelMode::Flash)) == "flash");
    EXPECT_TRUE(std::string(KernelModeName(KernelMode::Stream)) == "stream");
    EXPECT_TRUE(std::string(KernelModeName(KernelMode::NVLS)) == "nvls");
    Dtype d;
    EXPECT_TRUE(ParseDtype("bfloat16", &d) && d == Dtype::BF16);
    EXPECT_FALSE(ParseDtype("int8", &d));
    KernelMode m;
    EXPECT_TRUE(ParseKernelMode("STREAM", &m) && m == KernelMode::Stream);
}

TEST(interface_defaults) {
    AllReduceConfig c;
    EXPECT_EQ(c.num_ranks, 2);
    EXPECT_EQ(c.lanes, -1);
    EXPECT_EQ(c.ctas_per_lane, -1);
    EXPECT_TRUE(c.kernel_mode == KernelMode::Auto);
    EXPECT_EQ(c.warmup_iters, 1);
    EXPECT_EQ(c.measure_iters, 5);
    EXPECT_EQ(static_cast<int>(ReduceOp::Sum), 0);
    EXPECT_EQ(static_cast<int>(DataType::BFloat16), 2);
}

TEST(tuning_ranges) {
    for (int w : {2, 4, 8}) {
        EXPECT_GE(FlashCrossoverBytes(Dtype::FP32, w), 64ull << 10);
        for (uint64_t b = 1024; b <= (2ull << 30); b <<= 1) {
            int fl = FlashLanePreset(b, Dtype::FP32, w), sl = StreamLanePreset(b, Dtype::BF16, w);
            EXPECT_TRUE(fl >= 1 && fl <= kMaxFlashCtas);
            EXPECT_TRUE(sl >= 1 && sl <= kMaxLanes);
            uint64_t slot = AutoSlotBytes(b, w);
            EXPECT_TRUE(slot >= 8192 && slot <= (256u << 10));
        }
    }
    EXPECT_EQ(ClampSlotBytes(1, 1 << 20), 256u);
    EXPECT_EQ(AutoCtasPerLane(false, 16, 1 << 20, 1024), 1);
    PlanCaps caps;
    caps.flash_cap = 64 << 20;
    caps.ring_bytes = 256 << 20;
    Plan p;
    std::string why;
    EXPECT_TRUE(MakePlan(2, 262144, Dtype::FP32, Dtype::FP32, 0, KernelMode::Auto, caps, nullptr, &p, &why) == Result::Success);
    EXPECT_TRUE(p.variant == Variant::Flash);
    EXPECT_TRUE(MakePlan(2, 1ull << 28, Dtype::FP32, Dtype::FP32, 0, KernelMode::Auto, caps, nullptr, &p, &why) == Result::Success);
    EXPECT_TRUE(p.variant == Variant::Stream);
}

TEST(verify_allreduce_sum_host) {
    std::vector<float> v(64, 3.0f);
    size_t first = 0, count = 0;
    EXPECT_TRUE(VerifyAllReduceSum(v.data(), v.size(), 3.0f, 1e-3f, &first, &count));
    EXPECT_EQ(count, 0u);
    v[9] = 2.5f;
    v[40] = 9.0f;
    EXPECT_FALSE(VerifyAllReduceSum(v.data(), v.size(), 3.0f, 1e-3f, &first, &count));
    EXPECT_EQ(first, 9u);
    EXPECT_EQ(count, 2u);
    EXPECT_TRUE(VerifyAllReduceSum(v.data(), 0, 3.0f, 1e-3f, &first, &count));
}

template <typename T>
static void RoundTrip(Dtype dt, float value, float tol) {
    void* d = nullptr;
    if (AllocAndSeed(&d, 1000, dt, value) != cudaSuccess) {
        YT_FAIL_("AllocAndSeed failed");
        return;
    }
    std::vector<float> h(1000);
    EXPECT_TRUE(ConvertBufferToFloat(d, h.data(), 1000, dt) == cudaSuccess);
    for (float x : h) EXPECT_NEAR(x, value, tol);
    EXPECT_TRUE(ZeroBuffer(d, 1000 * DtypeSize(dt)) == cudaSuccess);
    EXPECT_TRUE(ConvertBufferToFloat(d, h.data(), 1000, dt) == cudaSuccess);
    for (float x : h) EXPECT_EQ(x, 0.0f);
    cudaFree(d);
}

TEST(seed_convert_zero_per_dtype) {
    if (!ytest::HasNGPUs(1)) SKIP_TEST("needs a GPU");
    RoundTrip<float>(Dtype::FP32, 42.5f, 1e-6f);
    RoundTrip<__half>(Dtype::FP16, 42.5f, 0.1f);
    RoundTrip<__nv_bfloat16>(Dtype::BF16, 42.5f, 0.5f);
    void* d = nullptr;
    EXPECT_TRUE(AllocAndSeed(&d, 0, Dtype::FP32, 1.0f) == cudaSuccess);  // count 0 is fine
    cudaFree(d);
}

TEST(random_fill_matches_host_generator) {
    if (!ytest::HasNGPUs(1)) SKIP_TEST("needs a GPU");
    const size_t n = 4096;
    float* d = nullptr;
    CUDA_CHECK(cudaMalloc(&d, n * sizeof(float)));
    CUDA_CHECK(FillRandom(d, n, Dtype::FP32, kDistUniformPm1, 77, nullptr));
    std::vector<float> h(n);
    CUDA_CHECK(cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < n; ++i) EXPECT_EQ(h[i], RandomValue(kDistUniformPm1, 77, i));  // same bits on host and device
    // a "result" equal to one rank's data validates for world = 1 and fails for world = 2
    EXPECT_TRUE(ValidateRandomResult(d, n, Dtype::FP32, Dtype::FP32, kDistUniformPm1, 77, 1, 1.0f, nullptr));
    ValidateReport rep;
    EXPECT_FALSE(ValidateRandomResult(d, n, Dtype::FP32, Dtype::FP32, kDistUniformPm1, 77, 2, 1.0f, &rep));
    EXPECT_GE(rep.mismatches, n / 2);
    cudaFree(d);
}

int main() { return RUN_ALL_TESTS(); }
