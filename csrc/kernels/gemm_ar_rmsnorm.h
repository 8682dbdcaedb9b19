// Argument block and host entry points of the fused row-parallel GEMM +
// all-reduce + residual + RMSNorm kernel (gemm_ar_rmsnorm.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../comm/layout.h"

namespace yali {

constexpr int kGemmTileM = 128;
constexpr int kGemmTileN = 256;
constexpr int kGemmThreads = 352;  // TMA warp, MMA warp, eight epilogue warps, announcer warp
constexpr int kGemmMaxVecPerThread = 2;  // N <= 2 * 352 threads * 8 bf16 = 5632 (the host caps N at 4096)

struct alignas(64) GemmArArgs {
    CUtensorMap tmap_a;  // x  [T, K] bf16, box 64 x 128, 128-byte swizzle
    CUtensorMap tmap_b;  // W  [N, K] bf16, box 64 x 256 (rows beyond N read as zeros), 128-byte swizzle
    CommView cv;
    const void* residual;     // [T, N] bf16 or nullptr
    void* residual_out;       // [T, N] bf16 or nullptr (sum + residual), this rank's copy
    void* residual_out_all[kMaxRanks];  // two-shot: every rank's residual_out (the row owner writes all copies)
    const void* norm_weight;  // [N] bf16
    void* out[kMaxRanks];     // every rank's output [T, N] (two-shot writes all, one-shot only its own)
    uint32_t T, N, K;
    uint32_t rows_per_owner;  // two-shot: rows normalised by each rank
    uint32_t oneshot;         // 1: every rank receives all partial rows and normalises all of them
    uint32_t ksplit;          // one-shot, few tiles: CTAs that share the K extent of a tile (1, 2 or 4; world x ksplit <= 8)
    uint32_t kper;            // k-blocks (of 64) per split
    uint32_t cnt_inc;         // arrivals per source that complete this rank's partial rows in this call
    uint32_t done_inc[kMaxRanks];  // per owner: rows it delivers to every rank's output in this call
    float eps;
    // NVLS form of the two-shot (nvls != 0): every rank keeps its partial rows in its OWN landing
    // zone, the owner of a row sums all ranks' copies in the switch (multimem.ld_reduce) and
    // writes the normalised row to every rank with one multimem.st through these addresses.
    // out_mc alone (nvls == 0) keeps the peer pushes of phase 1 and only delivers through the switch.
    uint32_t nvls;
    char* out_mc;           // multicast address of out, or nullptr: write every rank's copy with peer stores
    char* residual_out_mc;  // multicast address of residual_out, or nullptr
    unsigned long long* trace;  // optional: 8 x %globaltimer of CTA 0 at the phase boundaries (debugging aid)
};

struct GemmArEmuArgs {
    GemmArArgs r[kMaxRanks];
};

const void* GemmArKernel(bool emu);
uint32_t GemmArSmemBytes();

// ---- few-token form (gemm_ar_decode.cu): 128 x 256 tiles with the K extent split over CTAs, partial rows
// travel as flag-in-data lines in landing tiles of 32 columns
constexpr int kGemmDecodeTileN = 32;
constexpr int kGemmDecodeMmaN = 256;
constexpr uint32_t kGemmDecodeMaxSplit = 8;   // K splits per tile (sources per rank of the reduction)
constexpr int kGemmDecodeThreads = 512;       // TMA warp, MMA warp, eight epilogue warps; all 16 warps reduce rows
constexpr int kGemmDecodeVecPerThread = 1;    // N <= 512 threads * 8 bf16 = 4096
constexpr uint32_t kGemmDecodeMaxRows = 64;   // two TMEM lane quarters

struct alignas(64) GemmDecodeArgs {
    CUtensorMap tmap_a;  // x  [T, K] bf16, box 64 x a_box_rows (rows beyond T read as zeros), 128-byte swizzle
    CUtensorMap tmap_b;  // W  [N, K] bf16, box 64 x tile_n (rows beyond N read as zeros), 128-byte swizzle
    CommView cv;
    const void* residual;     // [T, N] bf16 or nullptr
    void* residual_out;       // [T, N] bf16 or nullptr
    const void* norm_weight;  // [N] bf16
    void* out;                // [T, N] bf16, this rank's
    uint32_t T, N, K;
    uint32_t a_box_rows;  // rows of x one TMA copy brings in: 8, 16, 32 or 64 (the smallest that holds T)
    uint32_t tile_n;      // columns of a tile = N of the MMA and rows of the box of W: 128 or 256
    uint32_t ksplit;      // CTAs that share the K extent of one tile (1, 2, 4 or 8)
    uint32_t kper;        // k-blocks (of 64) per split: split ks takes [ks * kper, min(K / 64, (ks + 1) * kper))
    float eps;
    unsigned long long* trace;  // optional: %globaltimer of CTA 0 at the phase boundaries
};
struct GemmDecodeEmuArgs {
    GemmDecodeArgs r[kMaxRanks];
};
const void* GemmDecodeKernel(bool emu);
uint32_t GemmDecodeSmemBytes();

}  // namespace yali
