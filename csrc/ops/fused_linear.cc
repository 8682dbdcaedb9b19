#include "fused_linear.h"

#include "../core/env.h"
#include "../core/nvtx.h"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <set>

#include "../comm/cuda_driver.h"
#include "../kernels/gemm_ar_rmsnorm.h"

namespace yali {

namespace {

bool EncodeTileMap(const DriverApi* d, CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols_k,
                   uint32_t box_rows, std::string* err);

// Few-token form: one launch of gemm_ar_decode.cu per rank.
Result LaunchDecode(Communicator& comm, const DriverApi* drv, const FusedLinearDesc* descs, uint32_t T, uint32_t N,
                    uint32_t K, const FusedLinearOptions& opt, const cudaStream_t* streams) {
    const int W = comm.world(), nlocal = comm.nlocal();
    auto fail = [&](Result r, const std::string& what) {
        comm.set_error(what);
        return r;
    };
    const void* fn = GemmDecodeKernel(comm.emulated());
    const uint32_t smem = GemmDecodeSmemBytes();
    static std::mutex attr_mu;
    static std::set<std::pair<int, int>> attr_done;
    {
        std::lock_guard<std::mutex> lock(attr_mu);
        for (int i = 0; i < nlocal; ++i) {
            const std::pair<int, int> key(comm.emulated() ? 1 : 0, comm.device_of(i));
            if (attr_done.count(key)) continue;
            if (nlocal > 1) cudaSetDevice(comm.device_of(i));
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (e != cudaSuccess) return fail(Result::CudaError, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
            attr_done.insert(key);
        }
    }
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, comm.device_of(0));
    // One CTA per SM (160 KiB of stages each); emulated ranks share the GPU.
    uint32_t resident = static_cast<uint32_t>(std::max(1, sms));
    if (comm.emulated()) resident = std::max<uint32_t>(1, resident / W);
    const uint32_t kblocks = K / 64;
    static const long long forced = env::GetInt("YALI_GEMM_DECODE_KSPLIT", 0);  // measurements only
    static const long long forced_tile = env::GetInt("YALI_GEMM_DECODE_TILE", 0);
    const uint32_t ksplit = FusedLinearDecodeSplit(T, N, K, W, resident, comm.layout().gemm_ll_cap,
                                                   forced > 0 ? static_cast<uint32_t>(forced) : 0u);
    uint32_t tile_n = FusedLinearDecodeTile(N, ksplit, resident);
    if (forced_tile == 128 || forced_tile == 256) tile_n = static_cast<uint32_t>(forced_tile);
    const uint32_t ntn = (N + tile_n - 1) / tile_n;
    const uint32_t kper = (kblocks + ksplit - 1) / ksplit;
    uint32_t ctas = std::min<uint32_t>(resident, ntn * ksplit);
    ctas = std::max<uint32_t>(ctas, std::min<uint32_t>(resident, T));  // CTA t normalises row t
    if (opt.ctas > 0) ctas = std::min<uint32_t>(ctas, opt.ctas);
    std::string derr;
    std::vector<GemmDecodeArgs> args(nlocal);
    for (int i = 0; i < nlocal; ++i) {
        GemmDecodeArgs& a = args[i];
        std::memset(&a, 0, sizeof(a));
        const FusedLinearDesc& d = descs[i];
        if (nlocal > 1) cudaSetDevice(comm.device_of(i));
        const uint32_t a_box_rows = T <= 8 ? 8u : T <= 16 ? 16u : T <= 32 ? 32u : 64u;
        if (!EncodeTileMap(drv, &a.tmap_a, d.x, T, K, a_box_rows, &derr) ||
            !EncodeTileMap(drv, &a.tmap_b, d.w, N, K, tile_n, &derr))
            return fail(Result::CudaError, derr);
        a.a_box_rows = a_box_rows;
        a.tile_n = tile_n;
        a.ksplit = ksplit;
        a.kper = kper;
        a.cv = comm.View(i);
        a.residual = d.residual;
        a.residual_out = d.residual_out;
        a.norm_weight = d.norm_weight;
        a.out = d.out;
        a.T = T;
        a.N = N;
        a.K = K;
        a.eps = opt.eps;
        a.trace = opt.trace ? opt.trace[i] : nullptr;
    }
    if (comm.emulated()) {
        GemmDecodeEmuArgs* e = new GemmDecodeEmuArgs();
        std::memset(e, 0, sizeof(*e));
        for (int i = 0; i < nlocal; ++i) e->r[comm.rank_of(i)] = args[i];
        cudaStream_t s = streams && streams[0] ? streams[0] : comm.default_stream(0);
        void* params[] = {e};
        cudaError_t ce = cudaLaunchCooperativeKernel(fn, dim3(ctas, W), dim3(kGemmDecodeThreads), params, smem, s);
        delete e;
        if (ce != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(Result::CudaError, std::string("cooperative launch failed: ") + cudaGetErrorString(ce));
        }
        comm.CountLaunch(1);
        return Result::Success;
    }
    for (int i = 0; i < nlocal; ++i) {
        if (nlocal > 1) cudaSetDevice(comm.device_of(i));
        cudaStream_t s = streams && streams[i] ? streams[i] : comm.default_stream(i);
        void* params[] = {&args[i]};
        cudaError_t ce = cudaLaunchKernel(fn, dim3(ctas), dim3(kGemmDecodeThreads), params, smem, s);
        if (ce != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(Result::CudaError, std::string("kernel launch failed: ") + cudaGetErrorString(ce));
        }
        comm.CountLaunch(1);
    }
    return Result::Success;
}

bool EncodeTileMap(const DriverApi* d, CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols_k,
                   uint32_t box_rows, std::string* err) {
    const cuuint64_t dims[2] = {cols_k, rows};             // innermost first
    const cuuint64_t strides[1] = {cols_k * 2};            // bytes between rows
    const cuuint32_t box[2] = {64, box_rows};              // 64 bf16 = 128 bytes = one swizzle row
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = d->TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (err) *err = "cuTensorMapEncodeTiled: " + d->ErrorText(r);
        return false;
    }
    return true;
}

}  // namespace

// Up to how many rows every rank receives all partial rows and normalises all of them itself (one NVLink
// phase instead of two, (W - 1) times the bytes).  Measured with 128 x 256 tiles, us one-shot / two-shot:
// 2 ranks T = 128: 25.3 / 30.8, T = 512: 35.0 / 36.5; 4 ranks T = 128: 25.0 / 27.5, T = 512: 42.3 / 33.6.
uint32_t FusedLinearOneShotMaxRows(int world) { return world <= 2 ? 256u : world <= 4 ? 128u : 32u; }

// K splits per 256-column tile of the few-token form.  An MMA of K = 16 costs about 90 ns whatever its
// width, so the k-blocks a CTA walks set the length of the GEMM phase (0.36 us each); every split is one more
// source for the reduction, which takes its sources eight at a time (about 1.8 us per eight, measured).  So:
// world x ksplit = 8 sources where K allows (2 x B200, K = 2048, T = 1: 12.7 us with 4 splits, 13.2 with 8,
// 15.5 with 2, 20.6 with 1), as long as the landing zone holds T rows per split, the work items fit the
// resident CTAs and no split is empty.  `want` > 0 replaces the first rule (measurements).
// Width of a tile of the few-token form: an MMA costs the same for 128 and for 256 columns, so the narrower
// tile is free for the GEMM and halves what an epilogue warp has to convert and push (32 columns instead of
// 64, to every rank); the wide one is for GPUs that hold fewer CTAs than there are narrow work items
// (several emulated ranks on one GPU).
uint32_t FusedLinearDecodeTile(uint32_t N, uint32_t ksplit, uint32_t resident_ctas) {
    return ((N + 127) / 128) * ksplit <= resident_ctas ? 128u : 256u;
}

uint32_t FusedLinearDecodeSplit(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t ll_cap,
                                uint32_t want) {
    const uint32_t ntn = (N + kGemmDecodeMmaN - 1) / kGemmDecodeMmaN, kblocks = K / 64;
    if (want == 0) want = std::max<uint32_t>(1, std::min<uint32_t>(kblocks / 4, 8u / static_cast<uint32_t>(std::max(world, 1))));
    uint32_t ksplit = 1;
    while (ksplit * 2 <= std::min<uint32_t>(want, kGemmDecodeMaxSplit)) ksplit *= 2;
    auto fits = [&](uint32_t ks) {
        const uint32_t kper = (kblocks + ks - 1) / ks;
        return static_cast<uint64_t>(T) * N * 4 * ks <= ll_cap && ntn * ks <= resident_ctas &&
               static_cast<uint64_t>(ks - 1) * kper < kblocks;
    };
    while (ksplit > 1 && !fits(ksplit)) ksplit /= 2;
    return ksplit;
}

uint32_t FusedLinearDecodeMaxRows(const HeapLayout& lay, uint32_t N, int world) {
    if (world < 2 || N == 0 || N % kGemmDecodeTileN != 0 ||
        N > static_cast<uint32_t>(kGemmDecodeThreads) * kGemmDecodeVecPerThread * 8 || lay.gemm_ll_cap == 0)
        return 0;
    // Payload bytes double as flag-in-data lines.
    const uint64_t rows = lay.gemm_ll_cap / (static_cast<uint64_t>(N) * 4);
    return static_cast<uint32_t>(std::min<uint64_t>(rows, kGemmDecodeMaxRows));
}

// Counter targets of one call: every source announces each 128x128 tile once to every owner
// that has rows in the tile's row block (one-shot: to everybody), and every owner reports the
// rows it delivered.  The kernel's announcer warp applies the same rule tile by tile.
void FusedLinearCounts(uint32_t T, uint32_t N, int W, bool oneshot, uint32_t* arrivals, uint32_t* rows_of) {
    const uint32_t ntm = (T + kGemmTileM - 1) / kGemmTileM, ntn = (N + kGemmTileN - 1) / kGemmTileN;
    const uint32_t Rs = oneshot ? T : (T + W - 1) / W;
    for (int q = 0; q < W; ++q) {
        arrivals[q] = rows_of[q] = 0;
        if (oneshot) {
            arrivals[q] = ntm * ntn;
        } else {
            const uint32_t lo = std::min<uint32_t>(T, q * Rs), hi = std::min<uint32_t>(T, lo + Rs);
            if (hi > lo) {
                const uint32_t first = lo / kGemmTileM, last = (hi - 1) / kGemmTileM;
                arrivals[q] = (last - first + 1) * ntn;
            }
            rows_of[q] = hi - lo;
        }
    }
}

// K splits per tile of a one-shot call of the tile form: powers of two while world x ksplit <= 8 (the reduction
// holds eight partial rows in registers), every split keeps at least four k-blocks, the work items fit the
// resident CTAs, a split's partial rows fit its share of the landing zone, and the partial rows a rank sends
// to its peers (every split sends its own) stay within 2 MiB (4 MiB for two splits): measured on 2 x B200,
// K = 2048, us with 1 / 2 / 4 splits: T = 128: 25.0 / 21.1 / 23.4; T = 256: - / 27.2 / 32.3 (two-shot: 30.8).
// `want` > 0 replaces the k-block and traffic rules (measurements).
uint32_t FusedLinearTileSplit(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t gemm_cap,
                              uint32_t want) {
    const uint32_t ntiles = ((T + kGemmTileM - 1) / kGemmTileM) * ((N + kGemmTileN - 1) / kGemmTileN), kblocks = K / 64;
    uint32_t ks = 1;
    auto fits = [&](uint32_t s) {
        const uint32_t kper = (kblocks + s - 1) / s;
        const uint64_t sent = static_cast<uint64_t>(T) * N * 2 * s * static_cast<uint64_t>(std::max(world - 1, 1));
        const bool by_rule = kblocks / s >= 4 && sent <= (s == 2 ? (4ull << 20) : (2ull << 20));
        return static_cast<uint32_t>(world) * s <= static_cast<uint32_t>(kMaxRanks) && (want > 0 ? s <= want : by_rule) &&
               ntiles * s <= resident_ctas && static_cast<uint64_t>(T) * N * 2 * s <= gemm_cap &&
               static_cast<uint64_t>(s - 1) * kper < kblocks;
    };
    while (ks < 4 && fits(ks * 2)) ks *= 2;
    return ks;
}

// Which multicast form the two-shot takes by default (0 none, 1 in-switch reduce + multicast store,
// 2 peer pushes + multicast store), from measurements on 2, 4 and 8 B200.
// 8 x B200, K = 512 per rank, N = 4096, CUDA-graph timing (us, modes 0 / 1 / 2): T = 128: 31.4 / 28.9 /
// 29.5; T = 512: 37.4 / 36.0 / 35.6; T = 2048: 80.1 / 78.7 / 78.1.  2 x B200 (K = 2048): mode 1 loses
// (109 against 90 us at T = 2048, the switch adds a hop and saves no bytes), mode 2 ties with mode 0.
// 4 x B200 (K = 1024, 128 x 256 tiles): T = 512: 33.6 / 35.4 / 33.9; T = 2048: 65.9 / 73.0 / 68.6: the peer
// pushes win or tie, so the switch is used from 8 ranks on.  8 x B200 with 128 x 256 tiles: T = 128: 28.2 /
// 28.4 / 27.2; T = 512: 36.5 / 35.5 / 35.9; T = 2048: 73.6 / 77.1 / 72.7: pushes + multicast delivery throughout.
int FusedLinearAutoMulticastMode(int world, uint32_t /*T*/) {
    return world < 8 ? 0 : 2;
}

Result FusedLinearAllReduceRmsNorm(Communicator& comm, const FusedLinearDesc* descs, uint32_t T, uint32_t N,
                                   uint32_t K, const FusedLinearOptions& opt, const cudaStream_t* streams) {
    YALI_NVTX_RANGE("yali::FusedLinear");
    auto fail = [&](Result r, const std::string& what) {
        comm.set_error(what);
        return r;
    };
    if (comm.poisoned()) return fail(Result::Timeout, "communicator is poisoned by an earlier timeout; call Reset()");
    if (T == 0) return Result::Success;
    if (N % 128 != 0 || N > 4096 || K % 64 != 0 || K == 0)
        return fail(Result::Unsupported, "fused linear needs N a multiple of 128 (at most 4096) and K a multiple of 64");
    const int W = comm.world(), nlocal = comm.nlocal();
    for (int i = 0; i < nlocal; ++i) {
        const FusedLinearDesc& d = descs[i];
        if (!d.x || !d.w || !d.norm_weight || !d.out) return fail(Result::InvalidArg, "null tensor");
        if ((reinterpret_cast<uintptr_t>(d.x) | reinterpret_cast<uintptr_t>(d.w) | reinterpret_cast<uintptr_t>(d.out) |
             reinterpret_cast<uintptr_t>(d.norm_weight) | reinterpret_cast<uintptr_t>(d.residual) |
             reinterpret_cast<uintptr_t>(d.residual_out)) & 15u)
            return fail(Result::InvalidArg, "tensors must be 16-byte aligned");
    }
    std::string derr;
    const DriverApi* drv = DriverApi::Get(&derr);
    if (!drv) return fail(Result::CudaError, derr);

    const HeapLayout& lay = comm.layout();
    const uint64_t row_bytes = static_cast<uint64_t>(N) * 2;
    {
        // Few tokens: the latency form (every rank normalises all rows; nothing else to decide).
        const uint32_t decode_max = FusedLinearDecodeMaxRows(lay, N, W);
        static const long long decode_env = env::GetInt("YALI_GEMM_DECODE", -1);
        const int want = opt.decode >= 0 ? opt.decode : static_cast<int>(decode_env);
        if (want == 1 && T > decode_max)
            return fail(Result::Unsupported, "the few-token form of the fused linear takes at most " +
                                                 std::to_string(decode_max) + " rows of this width");
        if (want != 0 && T <= decode_max && (want == 1 || (opt.force_oneshot != 0 && opt.nvls <= 0)))
            return LaunchDecode(comm, drv, descs, T, N, K, opt, streams);
    }
    bool oneshot = opt.force_oneshot >= 0 ? opt.force_oneshot != 0 : T <= FusedLinearOneShotMaxRows(W);
    if (W == 1) oneshot = true;
    // Two-shot writes into every rank's output: those must be addressable from here.
    bool outs_addressable = nlocal == W;
    uint64_t out_off = 0;
    if (!outs_addressable) {
        outs_addressable = comm.IsSymmetric(0, descs[0].out, static_cast<uint64_t>(T) * row_bytes);
        if (outs_addressable) out_off = static_cast<const char*>(descs[0].out) - comm.View(0).heap[comm.rank_of(0)];
    }
    uint64_t res_out_off = 0;
    if (nlocal != W && descs[0].residual_out) {
        // One GPU per process, two-shot: the owner of a row also writes every rank's residual_out.
        if (comm.IsSymmetric(0, descs[0].residual_out, static_cast<uint64_t>(T) * row_bytes))
            res_out_off = static_cast<const char*>(descs[0].residual_out) - comm.View(0).heap[comm.rank_of(0)];
        else
            outs_addressable = false;
    }
    if (!oneshot && !outs_addressable) {
        if (opt.force_oneshot == 0)
            return fail(Result::Unsupported, "two-shot fused linear needs out (and residual_out) in symmetric memory");
        oneshot = true;
    }
    uint32_t Rs = oneshot ? T : (T + W - 1) / W;
    if (static_cast<uint64_t>(Rs) * row_bytes > lay.gemm_cap) {
        if (oneshot && outs_addressable && static_cast<uint64_t>((T + W - 1) / W) * row_bytes <= lay.gemm_cap &&
            opt.force_oneshot != 1) {
            oneshot = false;
            Rs = (T + W - 1) / W;
        } else {
            return fail(Result::Unsupported, "rows do not fit the landing zone of the fused linear (" +
                                                 std::to_string(lay.gemm_cap) + " bytes per source)");
        }
    }

    // Forms of the two-shot that go through the NVSwitch multicast object: they need the multicast
    // mapping and out / residual_out at one common heap offset on every rank (tensors from SymmAlloc
    // are); the in-switch reduce also needs the [T, N] image to fit the landing region of one call
    // parity.  Mode 1: in-switch reduce + multicast store; mode 2: peer pushes + multicast store.
    int mc_mode = 0;
    uint64_t mc_out_off = 0, mc_res_out_off = 0;
    {
        const long long nvls_env = env::GetInt("YALI_GEMM_NVLS", -1);
        const int want = opt.nvls >= 0 ? opt.nvls : (nvls_env >= 0 ? static_cast<int>(nvls_env) : -1);
        bool possible = !oneshot && !comm.emulated() && W > 1 && want != 0 && comm.View(0).mc_heap != nullptr;
        for (int i = 0; i < nlocal && possible; ++i) {
            const char* base = comm.View(i).heap[comm.rank_of(i)];
            if (!comm.IsSymmetric(i, descs[i].out, static_cast<uint64_t>(T) * row_bytes)) possible = false;
            const uint64_t off = static_cast<const char*>(descs[i].out) - base;
            if (i == 0) mc_out_off = off;
            else if (off != mc_out_off) possible = false;
            if (descs[i].residual_out) {
                if (!comm.IsSymmetric(i, descs[i].residual_out, static_cast<uint64_t>(T) * row_bytes)) possible = false;
                const uint64_t roff = static_cast<const char*>(descs[i].residual_out) - base;
                if (i == 0) mc_res_out_off = roff;
                else if (roff != mc_res_out_off) possible = false;
            }
        }
        const bool image_fits = static_cast<uint64_t>(T) * row_bytes <= lay.gemm_cap * W;
        if (want > 0) {
            if (!possible || (want == 1 && !image_fits))
                return fail(Result::Unsupported,
                            "the multicast forms of the fused linear need two-shot, the multicast mapping and symmetric out tensors");
            mc_mode = want == 1 ? 1 : 2;
        } else if (possible) {
            mc_mode = FusedLinearAutoMulticastMode(W, T);
            if (mc_mode == 1 && !image_fits) mc_mode = 2;
        }
    }
    const bool nvls = mc_mode == 1;

    const uint32_t ntm = (T + kGemmTileM - 1) / kGemmTileM, ntn = (N + kGemmTileN - 1) / kGemmTileN;
    // Arrivals owner q expects from every source in this call, and rows owner q delivers.
    uint32_t arrivals[kMaxRanks] = {}, rows_of[kMaxRanks] = {};
    FusedLinearCounts(T, N, W, oneshot, arrivals, rows_of);
    const void* fn = GemmArKernel(comm.emulated());
    const uint32_t smem = GemmArSmemBytes();
    // The dynamic shared-memory limit is a per-device property of the kernel: raise it once for every
    // (kernel flavour, device) this process launches on.
    static std::mutex attr_mu;
    static std::set<std::pair<int, int>> attr_done;
    {
        std::lock_guard<std::mutex> lock(attr_mu);
        for (int i = 0; i < nlocal; ++i) {
            const std::pair<int, int> key(comm.emulated() ? 1 : 0, comm.device_of(i));
            if (attr_done.count(key)) continue;
            if (nlocal > 1) cudaSetDevice(comm.device_of(i));
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (e != cudaSuccess) return fail(Result::CudaError, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
            attr_done.insert(key);
        }
    }
    // Resident CTAs per GPU (queried once per kernel flavour; all GPUs of a group are alike).
    static int cached_per_sm[2] = {0, 0}, cached_sms[2] = {0, 0};
    const int flavour = comm.emulated() ? 1 : 0;
    if (cached_sms[flavour] == 0) {
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[flavour], fn, kGemmThreads, smem);
        cudaDeviceGetAttribute(&cached_sms[flavour], cudaDevAttrMultiProcessorCount, comm.device_of(0));
    }
    const int per_sm = cached_per_sm[flavour], sms = cached_sms[flavour];
    uint32_t resident = static_cast<uint32_t>(std::max(1, per_sm) * std::max(1, sms));
    if (comm.emulated()) resident = std::max<uint32_t>(1, resident / W);
    // One-shot calls split the K extent of their tiles while that shortens the GEMM phase (see FusedLinearTileSplit).
    static const long long forced_split = env::GetInt("YALI_GEMM_KSPLIT", 0);  // measurements only
    uint32_t ksplit = oneshot && mc_mode == 0 && W > 1
                          ? FusedLinearTileSplit(T, N, K, W, resident, lay.gemm_cap, forced_split > 0 ? static_cast<uint32_t>(forced_split) : 0u)
                          : 1u;
    const uint32_t kper = (K / 64 + ksplit - 1) / ksplit;
    const uint32_t work = std::max<uint32_t>(ntm * ntn * ksplit, oneshot ? T : Rs);
    uint32_t ctas = std::min<uint32_t>(resident, work);
    if (opt.ctas > 0) ctas = std::min<uint32_t>(ctas, opt.ctas);

    std::vector<GemmArArgs> args(nlocal);
    for (int i = 0; i < nlocal; ++i) {
        GemmArArgs& a = args[i];
        std::memset(&a, 0, sizeof(a));
        const FusedLinearDesc& d = descs[i];
        const int rank = comm.rank_of(i);
        if (nlocal > 1) cudaSetDevice(comm.device_of(i));
        if (!EncodeTileMap(drv, &a.tmap_a, d.x, T, K, kGemmTileM, &derr) ||
            !EncodeTileMap(drv, &a.tmap_b, d.w, N, K, kGemmTileN, &derr))
            return fail(Result::CudaError, derr);
        a.cv = comm.View(i);
        a.residual = d.residual;
        a.residual_out = d.residual_out;
        a.norm_weight = d.norm_weight;
        for (int q = 0; q < W; ++q) a.out[q] = a.residual_out_all[q] = nullptr;
        a.out[rank] = d.out;
        a.residual_out_all[rank] = d.residual_out;
        if (!oneshot) {
            if (nlocal == W) {
                for (int j = 0; j < nlocal; ++j) {
                    a.out[comm.rank_of(j)] = descs[j].out;
                    a.residual_out_all[comm.rank_of(j)] = descs[j].residual_out;
                }
            } else {
                for (int q = 0; q < W; ++q) {
                    a.out[q] = a.cv.heap[q] + out_off;
                    if (d.residual_out) a.residual_out_all[q] = a.cv.heap[q] + res_out_off;
                }
            }
        }
        a.T = T;
        a.N = N;
        a.K = K;
        a.rows_per_owner = Rs;
        a.oneshot = oneshot ? 1u : 0u;
        a.ksplit = ksplit;
        a.kper = kper;
        a.cnt_inc = arrivals[rank] * ksplit;  // every (tile, split) is announced
        for (int q = 0; q < W; ++q) a.done_inc[q] = rows_of[q];
        a.eps = opt.eps;
        a.nvls = nvls ? 1u : 0u;
        if (mc_mode != 0) {
            a.out_mc = a.cv.mc_heap + mc_out_off;
            a.residual_out_mc = d.residual_out ? a.cv.mc_heap + mc_res_out_off : nullptr;
        }
        a.trace = opt.trace ? opt.trace[i] : nullptr;
    }
    if (comm.emulated()) {
        GemmArEmuArgs* e = new GemmArEmuArgs();
        std::memset(e, 0, sizeof(*e));
        for (int i = 0; i < nlocal; ++i) e->r[comm.rank_of(i)] = args[i];
        cudaStream_t s = streams && streams[0] ? streams[0] : comm.default_stream(0);
        void* params[] = {e};
        cudaError_t ce = cudaLaunchCooperativeKernel(fn, dim3(ctas, W), dim3(kGemmThreads), params, smem, s);
        delete e;
        if (ce != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(Result::CudaError, std::string("cooperative launch failed: ") + cudaGetErrorString(ce));
        }
        comm.CountLaunch(1);
        return Result::Success;
    }
    for (int i = 0; i < nlocal; ++i) {
        if (nlocal > 1) cudaSetDevice(comm.device_of(i));
        cudaStream_t s = streams && streams[i] ? streams[i] : comm.default_stream(i);
        void* params[] = {&args[i]};
        cudaError_t ce = cudaLaunchKernel(fn, dim3(ctas), dim3(kGemmThreads), params, smem, s);
        if (ce != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(Result::CudaError, std::string("kernel launch failed: ") + cudaGetErrorString(ce));
        }
        comm.CountLaunch(1);
    }
    return Result::Success;
}

}  // namespace yali
