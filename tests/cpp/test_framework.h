// Minimal unit-test scaffolding for the C++ / CUDA tests: TEST registration, EXPECT_*
// checks that record failures and continue, skips for machines with too few GPUs.
// Reference counterpart: tests/unit/test_framework.h.
#pragma once

#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <functional>
#include <string>
#include <vector>

namespace ytest {

struct Case {
    const char* name;
    std::function<void()> fn;
};
inline std::vector<Case>& Cases() {
    static std::vector<Case> c;
    return c;
}
inline int& Failures() {
    static int f = 0;
    return f;
}
inline bool& Skipped() {
    static bool s = false;
    return s;
}
struct Registrar {
    Registrar(const char* n, std::function<void()> f) { Cases().push_back({n, std::move(f)}); }
};
inline int GpuCount() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    return n;
}
inline bool HasNGPUs(int n) { return GpuCount() >= n; }
inline bool HasP2PAccess(int a, int b) {
    int x = 0, y = 0;
    if (cudaDeviceCanAccessPeer(&x, a, b) != cudaSuccess || cudaDeviceCanAccessPeer(&y, b, a) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return x && y;
}
inline int RunAll() {
    int passed = 0, failed = 0, skipped = 0;
    for (const Case& c : Cases()) {
        const int before = Failures();
        Skipped() = false;
        c.fn();
        if (Skipped()) {
            ++skipped;
            std::printf("[ SKIP ] %s\n", c.name);
        } else if (Failures() == before) {
            ++passed;
            std::printf("[  OK  ] %s\n", c.name);
        } else {
            ++failed;
            std::printf("[ FAIL ] %s\n", c.name);
        }
    }
    std::printf("%d passed, %d failed, %d skipped\n", passed, failed, skipped);
    return failed ? 1 : 0;
}

}  // namespace ytest

#define TEST(name)                                             \
    static void ytest_fn_##name();                             \
    static ytest::Registrar ytest_reg_##name(#name, ytest_fn_##name); \
    static void ytest_fn_##name()
#define YT_FAIL_(msg)                                                          \
    do {                                                                       \
        ++ytest::Failures();                                                   \
        std::printf("    %s:%d: %s\n", __FILE__, __LINE__, std::string(msg).c_str()); \
    } while (0)
#define EXPECT_TRUE(c) do { if (!(c)) YT_FAIL_("expected true: " #c); } while (0)
#define EXPECT_FALSE(c) do { if (c) YT_FAIL_("expected false: " #c); } while (0)
#define EXPECT_EQ(a, b) do { if (!((a) == (b))) YT_FAIL_("expected equal: " #a " == " #b); } while (0)
#define EXPECT_NE(a, b) do { if (!((a) != (b))) YT_FAIL_("expected different: " #a " != " #b); } while (0)
#define EXPECT_GE(a, b) do { if (!((a) >= (b))) YT_FAIL_("expected " #a " >= " #b); } while (0)
#define EXPECT_LE(a, b) do { if (!((a) <= (b))) YT_FAIL_("expected " #a " <= " #b); } while (0)
#define EXPECT_NEAR(a, b, tol) do { if (!(std::fabs(double(a) - double(b)) <= (tol))) YT_FAIL_("expected " #a " near " #b); } while (0)
#define CUDA_CHECK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { YT_FAIL_(std::string("CUDA: ") + cudaGetErrorString(e_)); return; } } while (0)
#define SKIP_TEST(why) do { ytest::Skipped() = true; std::printf("    skipped: %s\n", why); return; } while (0)
#define RUN_ALL_TESTS() ytest::RunAll()
