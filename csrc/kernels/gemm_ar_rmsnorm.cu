// Tensor-parallel output projection fused with its all-reduce, residual add and
// RMSNorm in ONE kernel per rank:
//
//     out = RMSNorm(residual + sum_r x_r @ W_r^T) * norm_weight
//
// x_r is [T, K] (this rank's slice of the attention / MLP activations), W_r is
// [N, K] (this rank's slice of the row-parallel weight, K contiguous, the layout of
// torch.nn.Linear.weight), both bf16; the sum runs over the ranks.
//
// Phase 1 (GEMM): a persistent grid walks 128x128 output tiles.  One elected thread
// feeds a 3-stage shared-memory pipeline with TMA (cp.async.bulk.tensor, 128-byte
// swizzle, no multicast) and issues tcgen05.mma (bf16 x bf16 -> fp32) into a
// 128-column TMEM accumulator; completion arrives on mbarriers through
// tcgen05.commit.  The four warps read the accumulator back with tcgen05.ld, round
// to bf16, transpose through shared memory and PUSH every row straight into the
// landing zone of the rank that owns that row (peer stores over NVLink), then bump
// that rank's arrival counter with red.release.sys.
// Phase 2 (reduce): the same CTAs wait (bounded) until all ranks' partial rows for
// the rows this rank owns have landed, add them in fp32 in rank order, add the
// residual, normalise the row and write the bf16 result into EVERY rank's output
// (two-shot: rows are sharded over the ranks), or, for few rows, every rank owns
// all rows and writes only its own output (one-shot).  A final counter tells each
// rank when all rows of its output have arrived.
//
// Parity: none in the reference (it has no GEMM, no fused op and no tensor-core
// code; see its src/kernels and src/all_reduce).  The unfused composition (library
// GEMM, all-reduce, separate norm kernel) is kept in Python as the baseline.
#include <cuda.h>

#include "coll_common.cuh"
#include "gemm_ar_rmsnorm.h"

namespace yali {

namespace {

constexpr int BM = kGemmTileM, BN = kGemmTileN, BK = 64;  // BK bf16 = one 128-byte swizzle row
constexpr int kStages = 3;
constexpr uint32_t kStageABytes = BM * BK * 2, kStageBBytes = BN * BK * 2;
constexpr uint32_t kStageBytes = kStageABytes + kStageBBytes;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;  // + slack to align the base to 1024 bytes
constexpr uint32_t kTmemCols = 128;

// tcgen05 instruction descriptor: D = fp32, A = B = bf16, both K-major, N at bit 17 (>>3), M at bit 24 (>>4).
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                            (static_cast<uint32_t>(BM >> 4) << 24);

// Shared-memory matrix descriptor of a K-major operand tile stored by TMA with 128-byte
// swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);  // start address
    d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset: next 8-row group
    d |= static_cast<uint64_t>(1) << 46;                      // descriptor version of sm_100
    d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ bool mbar_wait_deadline(uint64_t* bar, uint32_t parity, uint64_t deadline_ns) {
    uint32_t tries = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if ((++tries & 15u) == 0 && ptx::globaltimer() > deadline_ns) return false;
    }
    return true;
}

__device__ __forceinline__ char* landing(const GemmArArgs& a, int on_rank, int src, uint32_t parity) {
    return a.cv.heap[on_rank] + a.cv.lay.gemm_off +
           (static_cast<uint64_t>(parity) * a.cv.world + src) * a.cv.lay.gemm_cap;
}

__device__ __forceinline__ void gemm_ar_body(const GemmArArgs& a, const CUtensorMap* tmap_a, const CUtensorMap* tmap_b,
                                             uint32_t cta, uint32_t nctas) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], accum_bar;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ float s_red[32];

    const CommView& cv = a.cv;
    const int W = cv.world, r = cv.rank;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
    // Call number and counter targets come from this rank's call words (advanced by the last
    // CTA of the previous launch), so the launch itself carries no per-call state.
    __shared__ uint32_t s_call[2 + kMaxRanks];
    if (tid < 2 + W) {
        const uint32_t word = tid == 0 ? kCallGemmEpoch : (tid == 1 ? kCallGemmCnt : kCallGemmDone + (tid - 2));
        s_call[tid] = *reinterpret_cast<volatile uint32_t*>(flag_word(cv, r, word));
    }
    __syncthreads();
    const uint32_t parity = (s_call[0] + 1u) & 1u;
    const uint32_t cnt_wanted = s_call[1] + a.cnt_inc;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        ptx::mbar_init(&accum_bar, 1);
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(tmap_a);
        ptx::tma_prefetch_desc(tmap_b);
    }
    if (warp == 0) {
        ptx::tmem_alloc(&s_tmem, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = s_tmem;

    const uint32_t ntm = (a.T + BM - 1) / BM, ntn = a.N / BN, kblocks = a.K / BK;
    const uint32_t ntiles = ntm * ntn;
    const uint32_t Rs = a.rows_per_owner;
    uint32_t g_load = 0, g_mma = 0, tile_iter = 0;
    bool ok = true;

    // ------------------------------------------------------------------ phase 1: GEMM tiles
    for (uint32_t tile = cta; ok && tile < ntiles; tile += nctas, ++tile_iter) {
        const uint32_t mt = tile / ntn, nt = tile % ntn;
        if (tid == 0) {
            uint32_t issued = 0, consumed = 0;
            while (consumed < kblocks) {
                while (issued < kblocks && issued - consumed < kStages) {
                    const uint32_t s = g_load % kStages;
                    if (g_load >= kStages && !mbar_wait_deadline(&empty_bar[s], ((g_load / kStages) - 1) & 1, deadline)) {
                        report_timeout(cv, kSiteMbar, r, cta, 1, g_load);
                        s_abort = 1;
                        break;
                    }
                    ptx::mbar_expect_tx(&full_bar[s], kStageBytes);
                    ptx::tma_load_2d(smem + s * kStageBytes, tmap_a, issued * BK, mt * BM, &full_bar[s]);
                    ptx::tma_load_2d(smem + s * kStageBytes + kStageABytes, tmap_b, issued * BK, nt * BN, &full_bar[s]);
                    ++g_load;
                    ++issued;
                }
                if (s_abort) break;
                const uint32_t s = g_mma % kStages;
                if (!mbar_wait_deadline(&full_bar[s], (g_mma / kStages) & 1, deadline)) {
                    report_timeout(cv, kSiteMbar, r, cta, 2, g_mma);
                    s_abort = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t a_addr = ptx::smem_u32(smem + s * kStageBytes);
                const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + kStageABytes);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    // 16 bf16 = 32 bytes further along K inside the swizzle row: +2 in the address field
                    ptx::tc_mma_f16(tmem, da + 2 * k, db + 2 * k, kIdesc, (consumed | k) != 0 ? 1u : 0u);
                }
                ptx::tc_commit(&empty_bar[s]);  // frees the stage when these MMAs have read it
                ++g_mma;
                ++consumed;
            }
            if (!s_abort) ptx::tc_commit(&accum_bar);
        }
        // Everybody waits for the accumulator of this tile.
        if (!mbar_wait_deadline(&accum_bar, tile_iter & 1, deadline)) {
            if (tid == 0 && !s_abort) report_timeout(cv, kSiteMbar, r, cta, 3, tile_iter);
            s_abort = 1;
        }
        __syncthreads();
        if (s_abort) {
            ok = false;
            break;
        }
        ptx::tc_fence_after_sync();

        // ---- epilogue: TMEM -> bf16 -> swizzled shared memory (stage 0 is idle now) -> owner's landing zone
        uint8_t* stage = smem + warp * (32 * BN * 2);  // 32 rows x 256 bytes per warp
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
            uint32_t v[32];
            ptx::tmem_ld_32x32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c * 32, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 4 chunks of 8 columns = 16 bytes of bf16
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[j * 8 + i]);
                const uint4 packed = pack16<__nv_bfloat16>(f);
                const int chunk = c * 4 + j;  // logical 16-byte chunk of the 256-byte row
                *reinterpret_cast<uint4*>(stage + lane * (BN * 2) + ((chunk ^ (lane & 15)) << 4)) = packed;
            }
        }
        __syncwarp();
        const int half = lane >> 4, c16 = lane & 15;
#pragma unroll 4
        for (int rr = 0; rr < 32; rr += 2) {
            const int row_in_warp = rr + half;
            const uint32_t grow = mt * BM + warp * 32 + row_in_warp;  // global row
            if (grow < a.T) {
                const uint4 x =
                    *reinterpret_cast<const uint4*>(stage + row_in_warp * (BN * 2) + ((c16 ^ (row_in_warp & 15)) << 4));
                const uint64_t col_off = (static_cast<uint64_t>(nt) * BN) * 2 + c16 * 16;
                if (a.oneshot) {
                    for (int k = 0; k < W; ++k) {
                        const int d = (r + k) % W;
                        ptx::st_v4(landing(a, d, r, parity) + static_cast<uint64_t>(grow) * a.N * 2 + col_off, x);
                    }
                } else {
                    const int d = grow / Rs;
                    ptx::st_v4(landing(a, d, r, parity) + static_cast<uint64_t>(grow - d * Rs) * a.N * 2 + col_off, x);
                }
            }
        }
        ptx::tc_fence_before_sync();
        __syncthreads();  // all pushes of this tile are issued; TMEM and stage 0 are free again
        // One arrival per (tile, destination that received rows of it).
        if (tid < W) {
            const uint32_t row_lo = mt * BM, row_hi = min(a.T, row_lo + BM);
            bool touched = a.oneshot != 0;
            if (!touched) touched = static_cast<uint32_t>(tid) * Rs < row_hi && (static_cast<uint32_t>(tid) + 1) * Rs > row_lo;
            if (touched) ptx::red_release_sys_add(flag_word(cv, tid, kGemmCntOff + r), 1u);
        }
        ptx::tc_fence_after_sync();
    }

    // TMEM is not needed any more (also on the abort path).
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, kTmemCols);
    if (!ok) return;

    // ------------------------------------------------------------------ phase 2: reduce + residual + RMSNorm
    // Rows this rank normalises: its shard (two-shot) or all rows (one-shot).
    const uint32_t row_lo = a.oneshot ? 0u : min(a.T, static_cast<uint32_t>(r) * Rs);
    const uint32_t row_hi = a.oneshot ? a.T : min(a.T, row_lo + Rs);
    const uint32_t my_rows = row_hi - row_lo;
    // Wait for the partial rows of every rank (own rows arrive through the same counters).
    if (my_rows > 0) {
        if (tid < W) {
            uint32_t seen;
            if (!ptx::wait_flag_reached(flag_word(cv, r, kGemmCntOff + tid), cnt_wanted, deadline, &seen)) {
                report_timeout(cv, kSiteGemmPartials, tid, cta, cnt_wanted, seen);
                s_abort = 1;
            }
        }
        __syncthreads();
        if (s_abort) return;

        constexpr int VEC = 8;  // bf16 per 16 bytes
        const uint32_t vec_per_row = a.N / VEC;
        const char* res = static_cast<const char*>(a.residual);
        char* res_out = static_cast<char*>(a.residual_out);
        const char* wgt = static_cast<const char*>(a.norm_weight);
        const float inv_n = 1.f / static_cast<float>(a.N);
        uint32_t rows_done = 0;
        for (uint32_t lr = cta; lr < my_rows; lr += nctas) {
            const uint32_t grow = row_lo + lr;
            float f[kGemmMaxVecPerThread][VEC];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < kGemmMaxVecPerThread; ++j) {
                const uint32_t c = tid + j * blockDim.x;
                if (c < vec_per_row) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) f[j][i] = 0.f;
                    const uint64_t off = (static_cast<uint64_t>(lr) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                    for (int q = 0; q < W; ++q) accumulate<__nv_bfloat16>(f[j], ptx::ld_cg_v4(landing(a, r, q, parity) + off));
                    const uint64_t goff = (static_cast<uint64_t>(grow) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                    if (res) accumulate<__nv_bfloat16>(f[j], ptx::ld_cg_v4(res + goff));
                    if (res_out) {
                        const uint4 pre = pack16<__nv_bfloat16>(f[j]);
                        if (a.oneshot) {
                            ptx::st_v4(res_out + goff, pre);
                        } else {  // the owner of the row fills every rank's copy
                            for (int k = 0; k < W; ++k) {
                                char* dst = static_cast<char*>(a.residual_out_all[(r + k) % W]);
                                if (dst) ptx::st_v4(dst + goff, pre);
                            }
                        }
                    }
#pragma unroll
                    for (int i = 0; i < VEC; ++i) ss += f[j][i] * f[j][i];
                }
            }
            const float inv_rms = rsqrtf(block_sum(ss, s_red) * inv_n + a.eps);
#pragma unroll
            for (int j = 0; j < kGemmMaxVecPerThread; ++j) {
                const uint32_t c = tid + j * blockDim.x;
                if (c < vec_per_row) {
                    float w[VEC];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) w[i] = 0.f;
                    accumulate<__nv_bfloat16>(w, *reinterpret_cast<const uint4*>(wgt + static_cast<uint64_t>(c) * 16));
#pragma unroll
                    for (int i = 0; i < VEC; ++i) f[j][i] = f[j][i] * inv_rms * w[i];
                    const uint4 y = pack16<__nv_bfloat16>(f[j]);
                    const uint64_t goff = (static_cast<uint64_t>(grow) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                    if (a.oneshot) {
                        ptx::st_v4(static_cast<char*>(a.out[r]) + goff, y);
                    } else {
                        for (int k = 0; k < W; ++k) {
                            const int d = (r + k) % W;
                            ptx::st_v4(static_cast<char*>(a.out[d]) + goff, y);
                        }
                    }
                }
            }
            ++rows_done;
        }
        // Two-shot: tell every rank how many of its output rows this CTA delivered.
        if (!a.oneshot) {
            __syncthreads();
            if (tid < W && rows_done > 0) ptx::red_release_sys_add(flag_word(cv, tid, kGemmDoneOff + r), rows_done);
        }
    }
    // Two-shot: this rank's output is complete when every owner's rows have landed.  One CTA
    // waits; the kernel cannot finish before it does.
    if (!a.oneshot && cta == 0) {
        if (tid < W) {
            uint32_t seen;
            const uint32_t want = s_call[2 + tid] + a.done_inc[tid];
            if (!ptx::wait_flag_reached(flag_word(cv, r, kGemmDoneOff + tid), want, deadline, &seen)) {
                report_timeout(cv, kSiteGemmDone, tid, cta, want, seen);
                s_abort = 1;
            }
        }
        __syncthreads();
        if (s_abort) return;
    }
    if (tid == 0 && check_out_last(cv, 3, nctas)) {
        advance_call_word(cv, kCallGemmEpoch, 1);
        advance_call_word(cv, kCallGemmCnt, a.cnt_inc);
        for (int q = 0; q < W; ++q) advance_call_word(cv, kCallGemmDone + q, a.done_inc[q]);
    }
}

}  // namespace

__global__ void __launch_bounds__(kGemmThreads, 2) gemm_ar_rmsnorm_kernel(const __grid_constant__ GemmArArgs a) {
    gemm_ar_body(a, &a.tmap_a, &a.tmap_b, blockIdx.x, gridDim.x);
}

// All ranks of an emulated communicator in one cooperative launch (ranks = blockIdx.y).
__global__ void __launch_bounds__(kGemmThreads, 2) gemm_ar_rmsnorm_kernel_emu(const __grid_constant__ GemmArEmuArgs e) {
    const GemmArArgs& a = e.r[blockIdx.y];
    gemm_ar_body(a, &a.tmap_a, &a.tmap_b, blockIdx.x, gridDim.x);
}

const void* GemmArKernel(bool emu) {
    return emu ? reinterpret_cast<const void*>(gemm_ar_rmsnorm_kernel_emu)
               : reinterpret_cast<const void*>(gemm_ar_rmsnorm_kernel);
}
uint32_t GemmArSmemBytes() { return kSmemBytes; }

}  // namespace yali
