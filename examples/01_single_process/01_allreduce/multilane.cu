// Single-process example that drives the lower-level interface: explicit kernel
// variant and CTA / lane count per call, pre-allocated symmetric buffers, the fused
// scale+cast epilogue, and validation of every element.  Works on 2, 4 or 8 GPUs
// (YALI_GPUS), element count from YALI_ELEMS, lanes from YALI_LANES, dtype from YALI_DTYPE.
//
// Reference counterpart: examples/01_single_process/01_allreduce/multilane.cu, which
// fills YaliLaunchArgs by hand and launches FlashKernel<float,3> on two GPUs.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <memory>

#include "comm/communicator.h"
#include "ops/buffer_ops.h"

using namespace yali;

int main() {
    const int W = std::getenv("YALI_GPUS") ? std::atoi(std::getenv("YALI_GPUS")) : 2;
    const size_t n = std::getenv("YALI_ELEMS") ? std::strtoull(std::getenv("YALI_ELEMS"), nullptr, 10) : (1u << 22);
    const int lanes = std::getenv("YALI_LANES") ? std::atoi(std::getenv("YALI_LANES")) : 16;
    Dtype dt = Dtype::FP32;
    if (const char* e = std::getenv("YALI_DTYPE")) ParseDtype(e, &dt);

    std::vector<int> devs(W);
    for (int i = 0; i < W; ++i) devs[i] = i;
    std::unique_ptr<Communicator> comm;
    std::string err;
    if (Communicator::CreateSingleProcess(devs, CommOptions(), &comm, &err) != Result::Success) {
        std::printf("communicator setup failed: %s\n", err.c_str());
        return 1;
    }
    std::vector<void*> send, recv;
    if (comm->SymmAlloc(n * DtypeSize(dt), &send) != Result::Success ||
        comm->SymmAlloc(n * DtypeSize(dt), &recv) != Result::Success) {
        std::printf("%s\n", comm->last_error().c_str());
        return 1;
    }
    for (int i = 0; i < W; ++i) {
        cudaSetDevice(i);
        FillRandom(send[i], n, dt, kDistUniformPm1, 1234 + i, comm->default_stream(i));
    }
    std::vector<const void*> csend(send.begin(), send.end());
    bool all_ok = true;
    const KernelMode modes[] = {KernelMode::Flash, KernelMode::Stream};
    for (KernelMode m : modes) {
        OpOptions opt;
        opt.mode = m;
        opt.ctas = lanes;
        opt.epilogue = kEpiScaleCast;  // gradient averaging fused into the all-reduce
        opt.scale = 1.0f / W;
        Result r = comm->AllReduce(csend.data(), recv.data(), n, dt, dt, opt, nullptr);
        if (r == Result::Success) r = comm->Sync();
        if (r != Result::Success) {
            std::printf("%s: %s (%s)\n", KernelModeName(m), GetErrorString(r), comm->last_error().c_str());
            return 1;
        }
        for (int i = 0; i < W; ++i) {
            cudaSetDevice(i);
            ValidateReport rep;
            bool ok = ValidateRandomResult(recv[i], n, dt, dt, kDistUniformPm1, 1234, W, 1.0f / W, &rep);
            std::printf("%-6s lanes=%u rank %d: %s (max abs err %.3g)\n", KernelModeName(m), comm->last_call().ctas, i,
                        ok ? "OK" : "MISMATCH", rep.max_abs_err);
            all_ok &= ok;
        }
    }
    std::printf("=== Example %s ===\n", all_ok ? "PASSED" : "FAILED");
    return all_ok ? 0 : 1;
}
