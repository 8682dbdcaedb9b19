// Host side of the fused tensor-parallel layer:
//     out = RMSNorm(residual + sum over ranks of x @ W^T) * norm_weight
// x: [T, K] bf16 per rank, W: [N, K] bf16 per rank (torch.nn.Linear layout), out / residual:
// [T, N] bf16, norm_weight: [N] bf16.  N a multiple of 128 and at most 4096, K a multiple of 64.
// Two-shot (rows sharded over the ranks, results written to every rank's output) needs every
// rank's `out` to be peer-addressable: buffers of one process, or symmetric buffers.
#pragma once

#include <cuda_runtime.h>

#include "../comm/communicator.h"

namespace yali {

struct FusedLinearDesc {
    const void* x = nullptr;
    const void* w = nullptr;
    const void* residual = nullptr;  // optional
    void* residual_out = nullptr;    // optional
    const void* norm_weight = nullptr;
    void* out = nullptr;
};

struct FusedLinearOptions {
    int force_oneshot = -1;  // -1: by size; 0: two-shot; 1: one-shot
    // Few-token form (128 x 256 tiles split along K over the CTAs, partial rows as flag-in-data lines, every rank
    // normalises all rows): -1 by size (T <= FusedLinearDecodeMaxRows), 0 never, 1 required.
    int decode = -1;
    int ctas = 0;            // 0: as many as are resident
    float eps = 1e-5f;
    // Use of the NVSwitch multicast object by the two-shot form: -1 by measurement, 0 none (peer
    // pushes, peer stores), 1 in-switch reduce + multicast store, 2 peer pushes + multicast store.
    // 1 and 2 fail with Unsupported when the multicast mapping or symmetric outputs are missing.
    int nvls = -1;
    unsigned long long* const* trace = nullptr;  // per local rank: device buffer of 8 timestamps, or nullptr
};

// descs: one per local rank.  Launches one kernel per rank (one cooperative launch for emulated ranks).
Result FusedLinearAllReduceRmsNorm(Communicator& comm, const FusedLinearDesc* descs, uint32_t T, uint32_t N,
                                   uint32_t K, const FusedLinearOptions& opt, const cudaStream_t* streams);

// Largest T the few-token form takes for rows of N elements (limited by its landing zone and by
// the two TMEM lane quarters its epilogue reads); 0 when it cannot run.
uint32_t FusedLinearDecodeMaxRows(const HeapLayout& lay, uint32_t N, int world);
// K splits per 256-column tile of the few-token form (1, 2, 4 or 8); `want` = 0: by the measured rule.
// K splits per tile of a one-shot call of the tile form (1, 2 or 4); `want` = 0: by the k-block rule.
uint32_t FusedLinearTileSplit(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t gemm_cap,
                              uint32_t want);
// Tile width of the few-token form for that split: 128 if the work items fit the resident CTAs, else 256.
uint32_t FusedLinearDecodeTile(uint32_t N, uint32_t ksplit, uint32_t resident_ctas);
uint32_t FusedLinearDecodeSplit(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t ll_cap,
                                uint32_t want);
// Rows from which the two-shot form is used when `force_oneshot` is -1.
uint32_t FusedLinearOneShotMaxRows(int world);
int FusedLinearAutoMulticastMode(int world, uint32_t T);
// Per owner q: tile announcements it receives from EACH source, and rows it delivers (arrays of W).
void FusedLinearCounts(uint32_t T, uint32_t N, int W, bool oneshot, uint32_t* arrivals, uint32_t* rows_of);

}  // namespace yali
