// Tensor-parallel output projection fused with its all-reduce, residual add and
// RMSNorm in ONE kernel per rank:
//
//     out = RMSNorm(residual + sum_r x_r @ W_r^T) * norm_weight
//
// x_r is [T, K] (this rank's slice of the attention / MLP activations), W_r is
// [N, K] (this rank's slice of the row-parallel weight, K contiguous, the layout of
// torch.nn.Linear.weight), both bf16; the sum runs over the ranks.
//
// Phase 1 (GEMM): a persistent grid (one 11-warp CTA per SM) walks 128x256 output
// tiles, warp-specialised.  Warp 0 feeds a 4-stage shared-memory pipeline with TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast); warp 1 issues tcgen05.mma
// (bf16 x bf16 -> fp32, M = 128, N = 256: an MMA of K = 16 was measured at about 90 ns
// whether it computes 32 or 128 columns, so the widest instruction halves the GEMM
// phase of 128-column tiles) into one of two 256-column TMEM accumulators (all of
// TMEM) and signals stage release and accumulator completion through tcgen05.commit
// on mbarriers; warps 2..9 (two per TMEM lane quarter, each taking half of the columns
// in two passes of 64) read a
// finished accumulator back with tcgen05.ld while the next tile's MMAs run into the
// other one, round to bf16, transpose through swizzled shared memory and PUSH every
// row straight into the landing zone of the rank that owns that row (peer stores
// over NVLink): while one warp of a pair reads TMEM and converts, the other one's
// stores are in flight.  Warp 10 announces each pushed tile to the
// owners with red.release.sys on their arrival counters: the fence in front of that
// reduction waits for the peer stores to land, so it sits in a warp of its own and
// the epilogue warps go straight on to the next tile.
// Phase 2 (reduce): the same CTAs wait (bounded) until all ranks' partial rows for
// the rows this rank owns have landed, add them in fp32 in rank order, add the
// residual, normalise the row and write the bf16 result into EVERY rank's output
// (two-shot: rows are sharded over the ranks), or, for few rows, every rank owns
// all rows and writes only its own output (one-shot).  A final counter tells each
// rank when all rows of its output have arrived.
// NVLS form of the two-shot (ranks joined by an NVSwitch multicast object): the
// epilogue keeps the partial rows in this rank's OWN landing zone, so phase 1 has no
// peer stores at all; the owner of a row reads the sum over all ranks with one
// multimem.ld_reduce per 16 bytes (fp32 accumulation in the switch) and delivers the
// normalised row to every rank with one multimem.st.  An SM then issues 1/W of the
// loads and stores; on the links the switch still pulls (W-1)/W * T*N*2 bytes out of
// every rank for the sums, while delivery sends only T*N*2/W per rank.  A third form
// keeps the peer pushes of phase 1 and uses the switch for delivery alone.
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
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 8;  // two per TMEM lane quarter, each takes half of the tile's columns
constexpr uint32_t kStageABytes = BM * BK * 2, kStageBBytes = BN * BK * 2;
constexpr uint32_t kStageBytes = kStageABytes + kStageBBytes;
constexpr int kEpiPassCols = 64;  // columns an epilogue warp moves per pass: 128 bytes of bf16 per row
constexpr uint32_t kEpiStageBytes = kEpilogueWarps * 32 * kEpiPassCols * 2;  // transposition buffers of the epilogue warps
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpiStageBytes + 1024;  // + slack to align the base
constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators of BN fp32 columns
static_assert(kTmemCols == 512 && kSmemBytes <= 227 * 1024, "one CTA per SM: all of TMEM, at most 227 KiB of shared memory");

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

// Landing zone of the partial rows of source `src` on a rank, relative to that rank's heap base.
__device__ __forceinline__ uint64_t landing_off(const GemmArArgs& a, int src, uint32_t parity) {
    return a.cv.lay.gemm_off + (static_cast<uint64_t>(parity) * a.cv.world + src) * a.cv.lay.gemm_cap;
}

// NVLS form: one [T, N] bf16 image per call parity at the same offset of every rank's heap.
__device__ __forceinline__ uint64_t landing_nvls_off(const GemmArArgs& a, uint32_t parity) {
    return a.cv.lay.gemm_off + static_cast<uint64_t>(parity) * a.cv.world * a.cv.lay.gemm_cap;
}

__device__ __forceinline__ void gemm_ar_body(const GemmArArgs& a, const CUtensorMap* tmap_a, const CUtensorMap* tmap_b,
                                             uint32_t cta, uint32_t nctas) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ __align__(8) uint64_t pushed_bar[2], announced_bar[2];  // epilogue warps -> announcer warp and back
    __shared__ uint32_t s_tmem;
    __shared__ char* s_heap[kMaxRanks];  // the heap bases: read with a run-time rank by the epilogue warps
    __shared__ volatile int s_abort;
    __shared__ float s_red[32];

    const CommView& cv = a.cv;
    const int W = cv.world, r = cv.rank;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
    // Optional timeline of CTA 0 (a.trace != nullptr): %globaltimer at the phase boundaries.
#define YALI_STAMP(slot, who)                                                              \
    do {                                                                                   \
        if (a.trace && cta == 0 && tid == (who)) a.trace[slot] = ptx::globaltimer();       \
    } while (0)
    YALI_STAMP(0, 0);  // entry
    // Call number and counter targets come from this rank's call words (advanced by the last
    // CTA of the previous launch), so the launch itself carries no per-call state.
    __shared__ uint32_t s_call[2 + kMaxRanks];
    if (tid >= 32 && tid < 32 + kMaxRanks) s_heap[tid - 32] = cv.heap[tid - 32];
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
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&tmem_full_bar[b], 1);
            ptx::mbar_init(&tmem_empty_bar[b], kEpilogueWarps);
            ptx::mbar_init(&pushed_bar[b], kEpilogueWarps);
            ptx::mbar_init(&announced_bar[b], 1);
        }
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(tmap_a);
        ptx::tma_prefetch_desc(tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(&s_tmem, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    YALI_STAMP(1, 0);  // barriers initialised, TMEM allocated

    const uint32_t ntm = (a.T + BM - 1) / BM, ntn = (a.N + BN - 1) / BN, kblocks = a.K / BK;
    const uint32_t ntiles = ntm * ntn;
    // One-shot calls of few tiles split the K extent of a tile over `ksplit` CTAs (an MMA costs the same
    // 90 ns for every tile, so the k-blocks one CTA walks set the length of the GEMM phase): a work item is
    // (tile, split), its partial rows land in a zone of their own (source rank r, split), and the reduction
    // adds world x ksplit partial rows.  ksplit = 1 everywhere else.
    const uint32_t ksplit = a.ksplit, ks_shift = 31 - __clz(ksplit), kper = a.kper;
    const uint32_t nitems = ntiles << ks_shift;
    const uint64_t split_cap = cv.lay.gemm_cap >> ks_shift;  // landing bytes per (source rank, split)
    const uint32_t Rs = a.rows_per_owner;
    // Two-shot: every rank starts with the row blocks owned by its right-hand neighbour and walks
    // on from there, so that at any moment the ranks push to different owners instead of all
    // converging on the owner of the first rows (which would serialise on that rank's links).
    const uint32_t mt_shift = a.oneshot ? 0u : (((static_cast<uint32_t>(r) + 1u) % W) * Rs / BM) % ntm;

    // ------------------------------------------------------------------ phase 1: GEMM tiles, warp-specialised
    // warp 0: TMA producer; warp 1: MMA issuer; warps 2..9: epilogue (TMEM -> bf16 -> peers);
    // warp 10: announcer (arrival counters of the owners).
    // Two TMEM accumulators of 128 columns alternate, so the MMAs of tile i+1 run while tile i
    // is read back and pushed.
    if (warp == 0) {
        if (lane == 0) {
            uint32_t g = 0;  // k-blocks loaded so far
            for (uint32_t item = cta; item < nitems && !s_abort; item += nctas) {
                const uint32_t tile = item >> ks_shift, split = item & (ksplit - 1);
                const uint32_t mt = (tile / ntn + mt_shift) % ntm, nt = tile % ntn;
                const uint32_t kb_end = min(kblocks, (split + 1) * kper);
                for (uint32_t kb = split * kper; kb < kb_end; ++kb, ++g) {
                    const uint32_t s = g % kStages;
                    if (!mbar_wait_deadline(&empty_bar[s], ((g / kStages) & 1u) ^ 1u, deadline)) {
                        report_timeout(cv, kSiteMbar, r, cta, 1, g);
                        s_abort = 1;
                        break;
                    }
                    ptx::mbar_expect_tx(&full_bar[s], kStageBytes);
                    ptx::tma_load_2d(smem + s * kStageBytes, tmap_a, kb * BK, mt * BM, &full_bar[s]);
                    ptx::tma_load_2d(smem + s * kStageBytes + kStageABytes, tmap_b, kb * BK, nt * BN, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t g = 0, it = 0;
            for (uint32_t item = cta; item < nitems && !s_abort; item += nctas, ++it) {
                const uint32_t split = item & (ksplit - 1);
                const uint32_t kb_begin = split * kper, kb_end = min(kblocks, (split + 1) * kper);
                const uint32_t b = it & 1u;
                if (!mbar_wait_deadline(&tmem_empty_bar[b], ((it >> 1) & 1u) ^ 1u, deadline)) {
                    report_timeout(cv, kSiteMbar, r, cta, 4, it);
                    s_abort = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem + b * BN;
                for (uint32_t kb = kb_begin; kb < kb_end; ++kb, ++g) {
                    const uint32_t s = g % kStages;
                    if (!mbar_wait_deadline(&full_bar[s], (g / kStages) & 1u, deadline)) {
                        report_timeout(cv, kSiteMbar, r, cta, 2, g);
                        s_abort = 1;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = ptx::smem_u32(smem + s * kStageBytes);
                    const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + kStageABytes);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 bf16 = 32 bytes further along K inside the swizzle row: +2 in the address field
                        ptx::tc_mma_f16(d_tmem, da + 2 * k, db + 2 * k, kIdesc, (kb != kb_begin || k != 0) ? 1u : 0u);
                    }
                    ptx::tc_commit(&empty_bar[s]);  // frees the stage when these MMAs have read it
                }
                if (s_abort) break;
                ptx::tc_commit(&tmem_full_bar[b]);  // accumulator complete
            }
        }
    } else if (warp == 2 + kEpilogueWarps) {
        // Announcer: when the eight epilogue warps have issued the pushes of a tile, tell every owner
        // that received rows of it.  red.release.sys orders the pushes (made visible to this warp by
        // the mbarrier) before the counter; waiting for them costs an NVLink round trip, which this
        // warp absorbs instead of the epilogue warps.
        uint32_t it = 0;
        for (uint32_t item = cta; item < nitems; item += nctas, ++it) {
            const uint32_t tile = item >> ks_shift;
            const uint32_t mt = (tile / ntn + mt_shift) % ntm, b = it & 1u;
            if (!mbar_wait_deadline(&pushed_bar[b], (it >> 1) & 1u, deadline)) {
                if (lane == 0 && !s_abort) report_timeout(cv, kSiteMbar, r, cta, 5, it);
                s_abort = 1;
                break;
            }
            if (lane < W) {
                const uint32_t row_lo = mt * BM, row_hi = min(a.T, row_lo + BM);
                bool touched = a.oneshot != 0;
                if (!touched)
                    touched = static_cast<uint32_t>(lane) * Rs < row_hi && (static_cast<uint32_t>(lane) + 1) * Rs > row_lo;
                if (touched) ptx::red_release_sys_add(flag_word(cv, lane, kGemmCntOff + r), 1u);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&announced_bar[b]);
            if (it == 0) YALI_STAMP(3, (2 + kEpilogueWarps) * 32);  // first tile pushed and announced
        }
    } else {
        const int q = warp & 3;         // TMEM lane quarter this warp may read
        const int h = (warp - 2) >> 2;  // column half of the tile this warp handles: [128h, 128h + 128)
        constexpr int HN = kEpiPassCols;  // 64 columns = 128 bytes of bf16 per row and pass
        constexpr int kPasses = BN / 2 / HN;
        uint8_t* stage = smem + kStages * kStageBytes + (warp - 2) * (32 * HN * 2);  // 32 rows x 128 bytes per warp
        const int rsub = lane >> 3, c16 = lane & 7;  // four rows per step, eight 16-byte chunks per row
        const uint64_t rowbytes = static_cast<uint64_t>(a.N) * 2;
        const uint64_t land_off = landing_off(a, r, parity);  // where this rank's partial rows go on every owner
        uint32_t it = 0;
        for (uint32_t item = cta; item < nitems; item += nctas, ++it) {
            const uint32_t tile = item >> ks_shift, split = item & (ksplit - 1);
            const uint32_t mt = (tile / ntn + mt_shift) % ntm, nt = tile % ntn, b = it & 1u;
            // Address arithmetic of the pushes, done while the MMAs of the tile still run.
            const uint32_t grow0 = mt * BM + q * 32 + rsub;  // this lane's first row
            uint32_t d0 = 0, local0 = grow0;
            if (!a.nvls && !a.oneshot) {
                d0 = grow0 / Rs;
                local0 = grow0 - d0 * Rs;
            }
            if (!mbar_wait_deadline(&tmem_full_bar[b], (it >> 1) & 1u, deadline)) {
                if (lane == 0 && !s_abort) report_timeout(cv, kSiteMbar, r, cta, 3, it);
                s_abort = 1;
                break;
            }
            ptx::tc_fence_after_sync();
            if (it == 0) YALI_STAMP(2, 64);  // first accumulator complete
            // Warps whose 32 rows lie entirely beyond T (small batches) or whose columns lie beyond N (the
            // last tile of an N that is not a multiple of 256) have nothing to read back.
            const bool warp_has_rows = mt * BM + q * 32 < a.T && nt * BN + h * (BN / 2) < a.N;
#pragma unroll
            for (int p = 0; p < kPasses; ++p) {
                const int cb = h * (BN / 2) + p * HN;  // first column of this pass inside the tile
#pragma unroll
                for (int c = 0; c < HN / 32; ++c) {
                    if (!warp_has_rows) break;
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(tmem + b * BN + (static_cast<uint32_t>(q * 32) << 16) + cb + c * 32, v);
                    ptx::tmem_ld_wait();
                    if (mt * BM + q * 32 + lane >= a.T) continue;  // this lane's row is padding
#pragma unroll
                    for (int j = 0; j < 4; ++j) {  // 4 chunks of 8 columns = 16 bytes of bf16
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[j * 8 + i]);
                        const int chunk = c * 4 + j;  // logical 16-byte chunk of the 128-byte row
                        *reinterpret_cast<uint4*>(stage + lane * (HN * 2) + ((chunk ^ (lane & 7)) << 4)) =
                            pack16<__nv_bfloat16>(f);
                    }
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                // After the last pass the accumulator half is out of TMEM: hand it back to the MMA warp.
                if (p == kPasses - 1 && lane == 0) ptx::mbar_arrive(&tmem_empty_bar[b]);
                if (!warp_has_rows) continue;
                // Lane = (row % 4, 16-byte chunk): eight steps of four rows.  A warp executes this part alone
                // and every instruction waits for the one before it, so the loop carries pointers that grow
                // by additions; the one division (owner of the first row) was made before the accumulator
                // was awaited.
                uint4 x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row_in_warp = i * 4 + rsub;
                    x[i] = *reinterpret_cast<const uint4*>(stage + row_in_warp * (HN * 2) + ((c16 ^ (row_in_warp & 7)) << 4));
                }
                const uint64_t col_off = (static_cast<uint64_t>(nt) * BN + cb) * 2 + c16 * 16;
                if (a.nvls) {
                    char* p = s_heap[r] + landing_nvls_off(a, parity) + static_cast<uint64_t>(grow0) * rowbytes + col_off;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (grow0 + 4 * i < a.T) ptx::st_v4(p + static_cast<uint64_t>(4 * i) * rowbytes, x[i]);
                } else if (a.oneshot) {
                    int d = r;
                    for (int k = 0; k < W; ++k) {
                        char* p = s_heap[d] + land_off + split * split_cap + static_cast<uint64_t>(grow0) * rowbytes + col_off;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (grow0 + 4 * i < a.T) ptx::st_v4(p + static_cast<uint64_t>(4 * i) * rowbytes, x[i]);
                        if (++d == W) d = 0;
                    }
                } else {
                    uint32_t d = d0, local = local0;
                    char* p = s_heap[d < static_cast<uint32_t>(W) ? d : 0] + land_off + static_cast<uint64_t>(local) * rowbytes + col_off;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (grow0 + 4 * i < a.T) ptx::st_v4(p, x[i]);
                        local += 4;
                        p += 4 * rowbytes;
                        while (local >= Rs && d + 1 < static_cast<uint32_t>(W)) {  // the next rows belong to the next owner
                            local -= Rs;
                            ++d;
                            p = s_heap[d] + land_off + static_cast<uint64_t>(local) * rowbytes + col_off;
                        }
                    }
                }
                __syncwarp();  // the next pass overwrites the transposition buffer
            }
            // This warp's pushes of the tile are issued: hand the tile to the announcer warp.  Its
            // barrier for this parity must have been consumed for the tile before last (it has, unless
            // the announcer lags two tiles behind).
            if (it >= 2 && !mbar_wait_deadline(&announced_bar[b], ((it >> 1) - 1u) & 1u, deadline)) {
                if (lane == 0 && !s_abort) report_timeout(cv, kSiteMbar, r, cta, 6, it);
                s_abort = 1;
                break;
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&pushed_bar[b]);
        }
    }

    // TMEM is not needed any more (also on the abort path).
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem, kTmemCols);
    if (s_abort) return;
    YALI_STAMP(4, 0);  // all tiles of this CTA done

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
        YALI_STAMP(5, 0);  // partial rows of every rank have landed

        constexpr int VEC = 8;  // bf16 per 16 bytes
        const uint32_t vec_per_row = a.N / VEC;
        const char* res = static_cast<const char*>(a.residual);
        char* res_out = static_cast<char*>(a.residual_out);
        const char* wgt = static_cast<const char*>(a.norm_weight);
        const float inv_n = 1.f / static_cast<float>(a.N);
        uint32_t rows_done = 0;
        if (a.nvls) {
            // The switch adds the W copies of a row (fp32 accumulation, bf16 result); two rows are in
            // flight per CTA so that their round trips through the switch overlap.
            constexpr int R = 2;
            const uint32_t rows_at_once = my_rows > nctas ? R : 1;  // few rows: one per CTA, on more CTAs
            const char* mc_in = cv.mc_heap + landing_nvls_off(a, parity);
            for (uint32_t lr0 = cta * rows_at_once; lr0 < my_rows; lr0 += nctas * rows_at_once) {
                uint4 sum[R][kGemmMaxVecPerThread], rv[R][kGemmMaxVecPerThread], wv[kGemmMaxVecPerThread];
#pragma unroll
                for (int j = 0; j < kGemmMaxVecPerThread; ++j) {
                    const uint32_t c = tid + j * blockDim.x;
                    if (c < vec_per_row) {
#pragma unroll
                        for (int u = 0; u < R; ++u) {
                            if (u < rows_at_once && lr0 + u < my_rows) {
                                const uint64_t goff =
                                    (static_cast<uint64_t>(row_lo + lr0 + u) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                                sum[u][j] = ptx::multimem_ld_reduce_bf16x8(mc_in + goff);
                                rv[u][j] = res ? ptx::ld_cg_v4(res + goff) : make_uint4(0, 0, 0, 0);
                            }
                        }
                        wv[j] = *reinterpret_cast<const uint4*>(wgt + static_cast<uint64_t>(c) * 16);
                    }
                }
#pragma unroll
                for (int u = 0; u < R; ++u) {
                    if (u >= rows_at_once || lr0 + u >= my_rows) break;  // same for the whole CTA
                    const uint32_t grow = row_lo + lr0 + u;
                    float f[kGemmMaxVecPerThread][VEC];
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < kGemmMaxVecPerThread; ++j) {
                        const uint32_t c = tid + j * blockDim.x;
                        if (c < vec_per_row) {
#pragma unroll
                            for (int i = 0; i < VEC; ++i) f[j][i] = 0.f;
                            accumulate<__nv_bfloat16>(f[j], sum[u][j]);
                            if (res) accumulate<__nv_bfloat16>(f[j], rv[u][j]);
                            if (a.residual_out_mc) {
                                const uint64_t goff = (static_cast<uint64_t>(grow) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                                ptx::multimem_st_v4(a.residual_out_mc + goff, pack16<__nv_bfloat16>(f[j]));
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
                            accumulate<__nv_bfloat16>(w, wv[j]);
#pragma unroll
                            for (int i = 0; i < VEC; ++i) f[j][i] = f[j][i] * inv_rms * w[i];
                            const uint64_t goff = (static_cast<uint64_t>(grow) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                            ptx::multimem_st_v4(a.out_mc + goff, pack16<__nv_bfloat16>(f[j]));
                        }
                    }
                    ++rows_done;
                }
            }
        } else {
        const char* const own_landing = s_heap[r] + landing_off(a, 0, parity);
        const int nsrc = W << ks_shift;  // at most kMaxRanks (the host keeps world x ksplit <= 8)
        for (uint32_t lr = cta; lr < my_rows; lr += nctas) {
            const uint32_t grow = row_lo + lr;
            // Every load of the row (W partial vectors, residual, weight, for each of this thread's
            // vectors) is issued before the first one is consumed: one memory round trip per row.
            uint4 part[kGemmMaxVecPerThread][kMaxRanks], rv[kGemmMaxVecPerThread], wv[kGemmMaxVecPerThread];
#pragma unroll
            for (int j = 0; j < kGemmMaxVecPerThread; ++j) {
                const uint32_t c = tid + j * blockDim.x;
                if (c < vec_per_row) {
                    const uint64_t off = (static_cast<uint64_t>(lr) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                    const uint64_t goff = (static_cast<uint64_t>(grow) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
#pragma unroll
                    for (int q = 0; q < kMaxRanks; ++q)  // source q = (rank q / ksplit, split q % ksplit)
                        if (q < nsrc)
                            part[j][q] = ptx::ld_cg_v4(own_landing + static_cast<uint64_t>(q >> ks_shift) * cv.lay.gemm_cap +
                                                       (q & (ksplit - 1)) * split_cap + off);
                    rv[j] = res ? ptx::ld_cg_v4(res + goff) : make_uint4(0, 0, 0, 0);
                    wv[j] = *reinterpret_cast<const uint4*>(wgt + static_cast<uint64_t>(c) * 16);
                }
            }
            float f[kGemmMaxVecPerThread][VEC];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < kGemmMaxVecPerThread; ++j) {
                const uint32_t c = tid + j * blockDim.x;
                if (c < vec_per_row) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) f[j][i] = 0.f;
#pragma unroll
                    for (int q = 0; q < kMaxRanks; ++q)
                        if (q < nsrc) accumulate<__nv_bfloat16>(f[j], part[j][q]);
                    if (res) accumulate<__nv_bfloat16>(f[j], rv[j]);
                    if (res_out) {
                        const uint64_t goff = (static_cast<uint64_t>(grow) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                        const uint4 pre = pack16<__nv_bfloat16>(f[j]);
                        if (a.oneshot) {
                            ptx::st_v4(res_out + goff, pre);
                        } else if (a.residual_out_mc) {  // one store through the switch fills every rank's copy
                            ptx::multimem_st_v4(a.residual_out_mc + goff, pre);
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
                    accumulate<__nv_bfloat16>(w, wv[j]);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) f[j][i] = f[j][i] * inv_rms * w[i];
                    const uint4 y = pack16<__nv_bfloat16>(f[j]);
                    const uint64_t goff = (static_cast<uint64_t>(grow) * a.N + static_cast<uint64_t>(c) * VEC) * 2;
                    if (a.oneshot) {
                        ptx::st_v4(static_cast<char*>(a.out[r]) + goff, y);
                    } else if (a.out_mc) {
                        ptx::multimem_st_v4(a.out_mc + goff, y);
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
        }
        YALI_STAMP(6, 0);  // own rows reduced and written
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
    YALI_STAMP(7, 0);  // output complete
#undef YALI_STAMP
    if (tid == 0 && check_out_last(cv, 3, nctas)) {
        advance_call_word(cv, kCallGemmEpoch, 1);
        advance_call_word(cv, kCallGemmCnt, a.cnt_inc);
        for (int q = 0; q < W; ++q) advance_call_word(cv, kCallGemmDone + q, a.done_inc[q]);
    }
}

}  // namespace

__global__ void __launch_bounds__(kGemmThreads, 1) gemm_ar_rmsnorm_kernel(const __grid_constant__ GemmArArgs a) {
    gemm_ar_body(a, &a.tmap_a, &a.tmap_b, blockIdx.x, gridDim.x);
}

// All ranks of an emulated communicator in one cooperative launch (ranks = blockIdx.y).
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_ar_rmsnorm_kernel_emu(const __grid_constant__ GemmArEmuArgs e) {
    const GemmArArgs& a = e.r[blockIdx.y];
    gemm_ar_body(a, &a.tmap_a, &a.tmap_b, blockIdx.x, gridDim.x);
}

const void* GemmArKernel(bool emu) {
    return emu ? reinterpret_cast<const void*>(gemm_ar_rmsnorm_kernel_emu)
               : reinterpret_cast<const void*>(gemm_ar_rmsnorm_kernel);
}
uint32_t GemmArSmemBytes() { return kSmemBytes; }

}  // namespace yali
