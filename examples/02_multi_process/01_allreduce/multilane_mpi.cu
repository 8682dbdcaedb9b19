// Multi-process example with pre-allocated symmetric buffers (exported once at start-up,
// zero-copy on every call), explicit variant and lanes, back-to-back calls without host
// synchronisation, and validation of every element on every rank.
// YALI_DTYPE / YALI_ELEMS / YALI_LANES select dtype, element count and lanes.
//
// Reference counterpart: examples/02_multi_process/01_allreduce/multilane_mpi.cu (manual
// IPC exchange and MPI barriers around every launch).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "ops/buffer_ops.h"
#include "ops/yali.h"

using namespace yali;

int main(int argc, char** argv) {
    MPIComm comm(&argc, &argv);
    if (!comm.ok()) return 1;
    const int rank = comm.rank(), W = comm.world_size();
    const size_t n = std::getenv("YALI_ELEMS") ? std::strtoull(std::getenv("YALI_ELEMS"), nullptr, 10) : (1u << 22);
    const int lanes = std::getenv("YALI_LANES") ? std::atoi(std::getenv("YALI_LANES")) : 0;
    Dtype dt = Dtype::BF16;
    if (const char* e = std::getenv("YALI_DTYPE")) ParseDtype(e, &dt);
    void* send = comm.alloc(n * DtypeSize(dt));
    void* recv = comm.alloc(n * DtypeSize(dt));
    if (!send || !recv) {
        std::printf("rank %d: %s\n", rank, comm.error().c_str());
        return 1;
    }
    FillRandom(send, n, dt, kDistUniformPm1, 1234 + rank, comm.stream());
    bool all_ok = true;
    const KernelMode modes[] = {KernelMode::Flash, KernelMode::Stream, KernelMode::NVLS};
    for (KernelMode m : modes) {
        if (m == KernelMode::NVLS && !comm.impl()->has_multicast()) continue;
        if (m == KernelMode::Flash && n * DtypeSize(dt) > comm.impl()->layout().flash_cap) continue;
        OpOptions opt;
        opt.mode = m;
        opt.ctas = lanes;
        for (int it = 0; it < 8; ++it) {  // no host barrier between calls: the kernels synchronise themselves
            if (allreduce_raw(comm, send, recv, n, dt, nullptr, true, opt) != cudaSuccess) {
                std::printf("rank %d: %s failed: %s\n", rank, KernelModeName(m), comm.impl()->last_error().c_str());
                return 1;
            }
        }
        if (comm.sync() != cudaSuccess) {
            std::printf("rank %d: %s\n", rank, comm.impl()->last_error().c_str());
            return 1;
        }
        ValidateReport rep;
        bool ok = ValidateRandomResult(recv, n, dt, dt, kDistUniformPm1, 1234, W, 1.0f, &rep);
        std::printf("rank %d %-6s: %s (max abs err %.3g)\n", rank, KernelModeName(m), ok ? "OK" : "MISMATCH",
                    rep.max_abs_err);
        all_ok &= ok;
    }
    comm.barrier();
    if (rank == 0) std::printf("=== Example %s ===\n", all_ok ? "PASSED" : "FAILED");
    return all_ok ? 0 : 1;
}
