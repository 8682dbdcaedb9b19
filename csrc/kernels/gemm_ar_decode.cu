// Few-token form of the fused tensor-parallel layer (decode: T <= 64 rows):
//
//     out = RMSNorm(residual + sum_r x_r @ W_r^T) * norm_weight
//
// The full-size kernel (gemm_ar_rmsnorm.cu) cuts the output into 128x128 tiles, which for a
// handful of tokens leaves N/128 = 32 CTAs streaming the weight slice and pays a release
// fence plus a counter round trip before the reduction.  This form is built for latency.
//
// What sets the pace of a GEMM with so few rows is the number of tcgen05.mma instructions one
// CTA issues: measured on B200, an MMA of K = 16 costs about 90 ns whether it computes 32 or
// 128 columns, 64 or 128 rows, and whether consecutive MMAs add into one accumulator or
// into four (0.36 us per 64-deep k-block; a slice of K = 2048 in 128x32 tiles took 11.6 us).
// So the MMAs here are wide (N = 128, or 256 where a GPU holds few CTAs), and the K extent of a
// tile is split over several CTAs instead:
//
//   * a work item is (tile of 128 padded rows x 128 or 256 columns, K split ks of `ksplit`);
//     with N = 4096 and K = 2048 per rank that is 32 x 4 = 128 items of eight k-blocks each,
//     one per CTA.  Warp 2 feeds a shared-memory ring with TMA (cp.async.bulk.tensor, 128-byte
//     swizzle, no multicast; the box of x has 8, 16, 32 or 64 rows, rows beyond T are out of
//     bounds and arrive as zeros; the box of W has as many rows as the tile has columns), warp 3
//     issues the MMAs (M = 128, bf16 x bf16 -> fp32) into one of two TMEM accumulators.
//     A stage holds only the rows the box of x brings in: the 128-row operand the MMA reads
//     runs on into the following stages, and what it finds there only reaches accumulator
//     rows that nobody reads (rows are independent);
//   * the eight warps of TMEM lane quarters 0 and 1 read the accumulator back (tcgen05.ld,
//     32 or 64 columns each) and send every row's partial sums to EVERY rank, this one included, as
//     16-byte lines that carry 8 bytes of payload and the 64-bit call number {data, call_lo,
//     data, call_hi}: the flag travels in the data, so there is no release fence, no counter
//     and no barrier between the GEMM and the reduction.  The landing zone of a source
//     (rank, ks) is cut into 32-column tiles ([tile][row][8 lines]) and the lines pass
//     through shared memory on their way out, so one store instruction of a warp covers 512
//     contiguous bytes of the peer's memory;
//   * CTA t (t < T) then owns row t on this rank: its 512 threads poll the lines of all
//     world x ksplit sources for one 16-byte output vector each (eight sources in flight
//     together), add them in fp32 in source order, add the residual, normalise and store.
// Every rank normalises all T rows for itself (one-shot), so nothing is sent back.
//
// Parity: none in the reference (no GEMM, no fused op, no tensor-core code there).
#include <cuda.h>

#include "coll_common.cuh"
#include "gemm_ar_rmsnorm.h"

namespace yali {

namespace {

constexpr int DBM = 128, DBNMax = kGemmDecodeMmaN, DBK = 64;  // the tile is 128 or 256 columns wide (a.tile_n)
constexpr int kLineTile = kGemmDecodeTileN;  // 32 columns = eight lines per row and landing tile
constexpr int kDMaxStages = 8;
// All A tiles first (a_box_rows * 128 bytes each), then all B tiles.  The MMA reads 128 rows (16 KiB)
// from the start of an A tile; past the last A tile that runs into the B tiles, never past the allocation.
constexpr uint32_t kDRingBytes = 160 * 1024;
constexpr uint32_t kDSmemBytes = kDRingBytes + 1024;  // + slack to align the base
constexpr uint32_t kDTmemCols = 2 * DBNMax;           // two accumulators of up to 256 fp32 columns: all of TMEM
constexpr int kDEpilogueWarps = 8;                    // lane quarters 0 and 1, four column groups of 32 or 64 each

// D = fp32, A = B = bf16, both K-major, N at bit 17 (>>3), M at bit 24 (>>4).
__device__ __forceinline__ uint32_t decode_idesc(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (static_cast<uint32_t>(DBM >> 4) << 24);
}

__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
                 : "memory");
    return v;
}

// Flag-in-data landing zone of source (rank `src`, K split `ks`) on every rank: at offset gemm_ll_off +
// (parity * world + src) * gemm_ll_cap + ks * (gemm_ll_cap / ksplit) of the heap, cut into 32-column tiles:
// line ((tile * T + row) * 8 + j) (16 bytes) holds columns 32 * tile + 4j .. 4j+3 of row `row`.

__device__ __forceinline__ void decode_body(const GemmDecodeArgs& a, const CUtensorMap* tmap_a,
                                            const CUtensorMap* tmap_b, uint32_t cta, uint32_t nctas) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kDMaxStages], empty_bar[kDMaxStages], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ __align__(16) uint4 s_lines[kDEpilogueWarps][32 * 8];  // per epilogue warp: 32 rows x 8 lines, swizzled
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ float s_red[32];
    __shared__ uint32_t s_call[2];
    __shared__ char* s_heap[kMaxRanks];  // the heap bases, read with a run-time rank in the epilogue and the reduction

    const CommView& cv = a.cv;
    const int W = cv.world, r = cv.rank;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = &s_abort;
    const uint64_t deadline = ptx::globaltimer() + cv.timeout_ns;
#define YALI_DSTAMP(slot, who)                                                       \
    do {                                                                             \
        if (a.trace && cta == 0 && tid == (who)) a.trace[slot] = ptx::globaltimer(); \
    } while (0)
    YALI_DSTAMP(0, 0);
    if (tid < 2)
        s_call[tid] = *reinterpret_cast<volatile uint32_t*>(flag_word(cv, r, tid == 0 ? kCallGemmLLEpoch : kCallGemmLLEpochHi));
    if (tid >= 32 && tid < 32 + kMaxRanks) s_heap[tid - 32] = cv.heap[tid - 32];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < kDMaxStages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&tmem_full_bar[b], 1);
            ptx::mbar_init(&tmem_empty_bar[b], kDEpilogueWarps);
        }
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(tmap_a);
        ptx::tma_prefetch_desc(tmap_b);
    }
    if (warp == 3) {
        ptx::tmem_alloc(&s_tmem, kDTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t lo = s_call[0] + 1u;                                    // this call's number
    const uint32_t hi = (s_call[1] + (lo == 0u ? 1u : 0u)) | 0x80000000u;  // never zero: fresh memory never matches
    const uint32_t parity = lo & 1u;
    YALI_DSTAMP(1, 0);

    const uint32_t DBN = a.tile_n;             // 128 or 256
    const uint32_t kDStageB = DBN * DBK * 2;  // 16 or 32 KiB
    const uint32_t wcols = DBN / 4;           // columns of an epilogue warp: one or two halves of 32
    const uint32_t ntn = (a.N + DBN - 1) / DBN, kblocks = a.K / DBK;
    const uint32_t ksplit = a.ksplit, kper = a.kper;  // k-blocks [ks * kper, min(kblocks, (ks + 1) * kper)) per split
    const uint32_t nitems = ntn * ksplit;
    const uint64_t split_bytes = cv.lay.gemm_ll_cap >> (31 - __clz(ksplit));  // ksplit is a power of two
    // The TMA box of x holds a.a_box_rows (8, 16, 32 or 64) rows, not 128: the copy engine spends its time per
    // 128-byte row, real or out of bounds.
    const uint32_t a_bytes = a.a_box_rows * DBK * 2;
    const uint32_t stages = min(kDRingBytes / (a_bytes + kDStageB), static_cast<uint32_t>(kDMaxStages));  // 4 to 8
    uint8_t* const smem_b = smem + stages * a_bytes;

    // ------------------------------------------------------------------ phase 1: GEMM items [128 x 256 x K / ksplit]
    if (warp == 2) {
        if (lane == 0) {
            uint32_t s = 0, round = 0;
            for (uint32_t item = cta; item < nitems && !*abort_flag; item += nctas) {
                const uint32_t tile = item / ksplit, ks = item % ksplit;
                const uint32_t kb_end = min(kblocks, (ks + 1) * kper);
                for (uint32_t kb = ks * kper; kb < kb_end; ++kb) {
                    if (!mbar_wait_deadline(&empty_bar[s], (round & 1u) ^ 1u, deadline, abort_flag)) {
                        if (!*abort_flag) report_timeout(cv, kSiteMbar, r, cta, 11, round * stages + s);
                        *abort_flag = 1;
                        break;
                    }
                    ptx::mbar_expect_tx(&full_bar[s], a_bytes + kDStageB);
                    ptx::tma_load_2d(smem_b + s * kDStageB, tmap_b, kb * DBK, tile * DBN, &full_bar[s]);
                    ptx::tma_load_2d(smem + s * a_bytes, tmap_a, kb * DBK, 0, &full_bar[s]);
                    if (++s == stages) s = 0, ++round;
                }
            }
        }
    } else if (warp == 3) {
        if (lane == 0) {
            uint32_t s = 0, round = 0, it = 0;
            for (uint32_t item = cta; item < nitems && !*abort_flag; item += nctas, ++it) {
                const uint32_t ks = item % ksplit;
                const uint32_t kb_begin = ks * kper, kb_end = min(kblocks, (ks + 1) * kper);
                const uint32_t b = it & 1u;
                if (!mbar_wait_deadline(&tmem_empty_bar[b], ((it >> 1) & 1u) ^ 1u, deadline, abort_flag)) {
                    if (!*abort_flag) report_timeout(cv, kSiteMbar, r, cta, 14, it);
                    *abort_flag = 1;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem + b * DBNMax;
                const uint32_t idesc = decode_idesc(DBN);
                for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait_deadline(&full_bar[s], round & 1u, deadline, abort_flag)) {
                        if (!*abort_flag) report_timeout(cv, kSiteMbar, r, cta, 12, round * stages + s);
                        *abort_flag = 1;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint64_t da = desc_sw128(ptx::smem_u32(smem + s * a_bytes));
                    const uint64_t db = desc_sw128(ptx::smem_u32(smem_b + s * kDStageB));
#pragma unroll
                    for (int k = 0; k < DBK / 16; ++k)
                        ptx::tc_mma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb != kb_begin || k != 0) ? 1u : 0u);
                    ptx::tc_commit(&empty_bar[s]);
                    if (++s == stages) s = 0, ++round;
                }
                if (*abort_flag) break;
                ptx::tc_commit(&tmem_full_bar[b]);
            }
        }
    } else if ((warp & 3) < 2) {
        const int q = warp & 3;   // TMEM lane quarter this warp may read
        const int g = warp >> 2;  // its 64 columns of the 256
        const int ew = q * 4 + g;
        uint32_t it = 0;
        for (uint32_t item = cta; item < nitems; item += nctas, ++it) {
            const uint32_t tile = item / ksplit, ks = item % ksplit;
            const uint32_t b = it & 1u;
            // Address arithmetic of the pushes, done while the MMAs still run: a warp executes its epilogue
            // alone, every instruction waiting for the one before it, so what is left after the wait is
            // one shared-memory load and one addition per destination.
            const uint32_t col0 = tile * DBN + g * wcols;  // first of this warp's columns
            const uint64_t push_off = cv.lay.gemm_ll_off + (static_cast<uint64_t>(parity) * W + r) * cv.lay.gemm_ll_cap +
                                      static_cast<uint64_t>(ks) * split_bytes + lane * 16 +
                                      (static_cast<uint64_t>(col0 / kLineTile) * a.T + static_cast<uint64_t>(q) * 32) * 128;
            const uint64_t half_step = static_cast<uint64_t>(a.T) * 128;  // the next 32-column landing tile
            if (!mbar_wait_deadline(&tmem_full_bar[b], (it >> 1) & 1u, deadline, abort_flag)) {
                if (lane == 0 && !*abort_flag) report_timeout(cv, kSiteMbar, r, cta, 13, it);
                *abort_flag = 1;
                break;
            }
            ptx::tc_fence_after_sync();
            if (it == 0) YALI_DSTAMP(2, 0);  // first accumulator complete
            const bool rows_here = static_cast<uint32_t>(q) * 32 < a.T && col0 < a.N;
            uint32_t v[2][32];
            if (rows_here) {
                const uint32_t base = tmem + b * DBNMax + g * wcols + (static_cast<uint32_t>(q * 32) << 16);
                ptx::tmem_ld_32x32(base, v[0]);
                if (wcols > 32) ptx::tmem_ld_32x32(base + 32, v[1]);
                ptx::tmem_ld_wait();
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tmem_empty_bar[b]);
            if (!rows_here) continue;
            uint4* stage = s_lines[ew];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (h * 32 >= static_cast<int>(wcols) || col0 + h * 32 >= a.N) break;
                // 32 fp32 -> 32 bf16 -> eight lines {2 bf16, call_lo, 2 bf16, call_hi}, lane = row; through
                // shared memory (line j of row at j ^ (row & 7)) they come back as lane = (row % 4, line).
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[h][4 * j]), __uint_as_float(v[h][4 * j + 1]));
                    const __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[h][4 * j + 2]), __uint_as_float(v[h][4 * j + 3]));
                    stage[lane * 8 + (j ^ (lane & 7))] = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), lo,
                                                                   *reinterpret_cast<const uint32_t*>(&h1), hi);
                }
                __syncwarp();
                uint4 mine[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rl = i * 4 + (lane >> 3);
                    mine[i] = stage[rl * 8 + ((lane & 7) ^ (rl & 7))];
                }
                __syncwarp();  // the next half may overwrite the staging lines
                if (it == 0 && h == 0) YALI_DSTAMP(7, 0);  // first half packed and transposed
                // This warp's rows of this 32-column tile are one contiguous block of the landing zone.
                if (a.T <= 2) {
                    // One or two rows fill 8 or 16 lanes of a store: the other lanes take the same lines to
                    // further destinations, so one instruction serves four (two) ranks instead of one.
                    const uint32_t lanes_per_dst = 8 * a.T, dst_per_store = 32 / lanes_per_dst;
                    const uint32_t src_lane = lane % lanes_per_dst, slot = lane / lanes_per_dst;
                    uint4 y;
                    y.x = __shfl_sync(0xffffffffu, mine[0].x, src_lane);
                    y.y = __shfl_sync(0xffffffffu, mine[0].y, src_lane);
                    y.z = __shfl_sync(0xffffffffu, mine[0].z, src_lane);
                    y.w = __shfl_sync(0xffffffffu, mine[0].w, src_lane);
                    const uint64_t off = push_off - lane * 16 + src_lane * 16 + h * half_step;
                    for (uint32_t k0 = 0; k0 < static_cast<uint32_t>(W); k0 += dst_per_store) {
                        const uint32_t k = k0 + slot;
                        if (k < static_cast<uint32_t>(W)) {
                            uint32_t d = static_cast<uint32_t>(r) + k;
                            if (d >= static_cast<uint32_t>(W)) d -= W;
                            ptx::st_v4(s_heap[d] + off, y);
                        }
                    }
                    continue;
                }
                int d = r + 1 == W ? 0 : r + 1;  // the peers first (their lines have the longer way), the own copy last
                for (int k = 0; k < W; ++k) {
                    char* dst = s_heap[d] + push_off + h * half_step;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (static_cast<uint32_t>(q * 32 + i * 4 + (lane >> 3)) < a.T) ptx::st_v4(dst + i * 512, mine[i]);
                    if (it == 0 && h == 0 && k == 0) YALI_DSTAMP(5, 0);  // first half stored into the first peer's zone
                    if (++d == W) d = 0;
                }
            }
        }
    }

    // TMEM is not needed any more (also on the abort path).
    YALI_DSTAMP(6, 0);  // this warp's pushes issued
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 3) ptx::tmem_dealloc(tmem, kDTmemCols);
    if (s_abort) return;
    YALI_DSTAMP(3, 0);  // all items of this CTA pushed

    // ------------------------------------------------------------------ phase 2: rows, all threads
    constexpr int VEC = 8;  // bf16 per 16 bytes
    const uint32_t vec_per_row = a.N / VEC;
    const char* res = static_cast<const char*>(a.residual);
    char* res_out = static_cast<char*>(a.residual_out);
    const char* wgt = static_cast<const char*>(a.norm_weight);
    const float inv_n = 1.f / static_cast<float>(a.N);
    const uint32_t nsrc = static_cast<uint32_t>(W) * ksplit;  // source s = rank s / ksplit, K split s % ksplit
    const char* const landing0 = s_heap[r] + cv.lay.gemm_ll_off + static_cast<uint64_t>(parity) * W * cv.lay.gemm_ll_cap;
    for (uint32_t row = cta; row < a.T; row += nctas) {
        float f[VEC];
        float ss = 0.f;
        bool timed_out = false;
        const uint32_t c = tid;
        uint4 wv = make_uint4(0, 0, 0, 0);  // the norm weights of this thread's columns, fetched before the wait
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = 0.f;
        if (c < vec_per_row) {
            wv = *reinterpret_cast<const uint4*>(wgt + static_cast<uint64_t>(c) * 16);
            // Output vector c = columns 8c..8c+7 = lines 2 (c % 4) and the next of 32-column tile c / 4, from every source.
            const uint64_t off = ((static_cast<uint64_t>(c >> 2) * a.T + row) * 8 + (c & 3u) * 2) * 16;
            const uint4 rv = res ? ptx::ld_cg_v4(res + (static_cast<uint64_t>(row) * a.N + static_cast<uint64_t>(c) * VEC) * 2)
                                 : make_uint4(0, 0, 0, 0);
            for (uint32_t s0 = 0; s0 < nsrc && !timed_out; s0 += 8) {
                const uint32_t n = min(8u, nsrc - s0);
                uint4 l0[8], l1[8];
                uint32_t pending = (1u << n) - 1u, polls = 0;
                while (pending) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (static_cast<uint32_t>(q) < n && (pending >> q & 1u)) {
                            const char* p = landing0 + static_cast<uint64_t>(s0 + q) * split_bytes + off;
                            l0[q] = ld_volatile16(p);
                            l1[q] = ld_volatile16(p + 16);
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (static_cast<uint32_t>(q) < n && (pending >> q & 1u) && l0[q].y == lo && l0[q].w == hi &&
                            l1[q].y == lo && l1[q].w == hi)
                            pending &= ~(1u << q);
                    }
                    if (pending && (++polls & 63u) == 0u && (*abort_flag || ptx::globaltimer() > deadline)) {
                        if (!*abort_flag) report_timeout(cv, kSiteGemmPartials, (s0 + __ffs(pending) - 1) / ksplit, cta, lo, 0u);
                        timed_out = true;
                        break;
                    }
                }
                if (!timed_out) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        if (static_cast<uint32_t>(q) < n) accumulate<__nv_bfloat16>(f, make_uint4(l0[q].x, l0[q].z, l1[q].x, l1[q].z));
                }
            }
            if (!timed_out) {
                if (res) accumulate<__nv_bfloat16>(f, rv);
                if (res_out)
                    ptx::st_v4(res_out + (static_cast<uint64_t>(row) * a.N + static_cast<uint64_t>(c) * VEC) * 2,
                               pack16<__nv_bfloat16>(f));
#pragma unroll
                for (int i = 0; i < VEC; ++i) ss += f[i] * f[i];
            }
        }
        if (__syncthreads_or(timed_out ? 1 : 0)) {
            if (tid == 0) s_abort = 1;
            break;
        }
        const float inv_rms = rsqrtf(block_sum(ss, s_red) * inv_n + a.eps);
        if (c < vec_per_row) {
            float w[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) w[i] = 0.f;
            accumulate<__nv_bfloat16>(w, wv);
#pragma unroll
            for (int i = 0; i < VEC; ++i) f[i] = f[i] * inv_rms * w[i];
            ptx::st_v4(static_cast<char*>(a.out) + (static_cast<uint64_t>(row) * a.N + static_cast<uint64_t>(c) * VEC) * 2,
                       pack16<__nv_bfloat16>(f));
        }
    }
    __syncthreads();
    if (s_abort) return;
    YALI_DSTAMP(4, 0);  // rows written
#undef YALI_DSTAMP
    if (tid == 0 && check_out_last(cv, 3, nctas)) {
        advance_call_word(cv, kCallGemmLLEpoch, 1);
        if (lo == 0u) advance_call_word(cv, kCallGemmLLEpochHi, 1);
    }
}

}  // namespace

__global__ void __launch_bounds__(kGemmDecodeThreads, 1) gemm_ar_decode_kernel(const __grid_constant__ GemmDecodeArgs a) {
    decode_body(a, &a.tmap_a, &a.tmap_b, blockIdx.x, gridDim.x);
}

// All ranks of an emulated communicator in one cooperative launch (ranks = blockIdx.y).
__global__ void __launch_bounds__(kGemmDecodeThreads, 1)
    gemm_ar_decode_kernel_emu(const __grid_constant__ GemmDecodeEmuArgs e) {
    const GemmDecodeArgs& a = e.r[blockIdx.y];
    decode_body(a, &a.tmap_a, &a.tmap_b, blockIdx.x, gridDim.x);
}

const void* GemmDecodeKernel(bool emu) {
    return emu ? reinterpret_cast<const void*>(gemm_ar_decode_kernel_emu)
               : reinterpret_cast<const void*>(gemm_ar_decode_kernel);
}
uint32_t GemmDecodeSmemBytes() { return kDSmemBytes; }

}  // namespace yali
