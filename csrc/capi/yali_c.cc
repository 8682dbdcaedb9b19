#include "yali_c.h"

#include "../ops/fused_linear.h"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../comm/bootstrap.h"
#include "../comm/layout.h"
#include "../ops/buffer_ops.h"
#include "../ops/host_oracle.h"
#include "../ops/tuning.h"

using namespace yali;

namespace {
void CopyErr(const std::string& e, char* err, size_t n) {
    if (err && n) std::snprintf(err, n, "%s", e.c_str());
}
Bootstrap* BS(void* p) { return static_cast<Bootstrap*>(p); }
}  // namespace

extern "C" {

const char* yali_c_version(void) { return "yali-b200 0.1"; }
const char* yali_c_error_string(int r) { return GetErrorString(static_cast<Result>(r)); }

void* yali_c_bootstrap_create(int rank, int world, int local_rank, const char* job_id, int timeout_ms, char* err,
                              size_t err_len) {
    Result r;
    std::string e;
    auto b = MakeSocketBootstrap(rank, world, local_rank, job_id ? job_id : "default", timeout_ms, &r, &e);
    if (!b) CopyErr(e, err, err_len);
    return b.release();
}
void* yali_c_bootstrap_from_env(char* err, size_t err_len) {
    Result r;
    std::string e;
    auto b = MakeEnvBootstrap(&r, &e);
    if (!b) CopyErr(e, err, err_len);
    return b.release();
}
void yali_c_bootstrap_destroy(void* bs) { delete BS(bs); }
int yali_c_bootstrap_rank(void* bs) { return BS(bs)->rank(); }
int yali_c_bootstrap_world(void* bs) { return BS(bs)->world(); }
int yali_c_bootstrap_allgather(void* bs, const void* in, void* out, size_t n) {
    return static_cast<int>(BS(bs)->allgather(in, out, n));
}
int yali_c_bootstrap_broadcast(void* bs, void* buf, size_t n, int root) {
    return static_cast<int>(BS(bs)->broadcast(buf, n, root));
}
int yali_c_bootstrap_barrier(void* bs) { return static_cast<int>(BS(bs)->barrier()); }
int yali_c_bootstrap_allgather_fd(void* bs, int my_fd, int* fds_out) {
    std::vector<int> fds;
    Result r = BS(bs)->allgather_fd(my_fd, &fds);
    if (r == Result::Success)
        for (size_t i = 0; i < fds.size(); ++i) fds_out[i] = fds[i];
    return static_cast<int>(r);
}
int yali_c_bootstrap_broadcast_fd(void* bs, int* fd) { return static_cast<int>(BS(bs)->broadcast_fd(fd, 0)); }
const char* yali_c_bootstrap_last_error(void* bs) { return BS(bs)->last_error().c_str(); }

uint64_t yali_c_flash_crossover_bytes(int dt, int world) { return FlashCrossoverBytes(static_cast<Dtype>(dt), world); }
int yali_c_flash_lane_preset(uint64_t b, int dt, int w) { return FlashLanePreset(b, static_cast<Dtype>(dt), w); }
int yali_c_stream_lane_preset(uint64_t b, int dt, int w) { return StreamLanePreset(b, static_cast<Dtype>(dt), w); }
uint64_t yali_c_auto_slot_bytes(uint64_t b, int w) { return AutoSlotBytes(b, w); }
uint64_t yali_c_clamp_slot_bytes(uint64_t s, uint64_t m) { return ClampSlotBytes(s, m); }
int yali_c_auto_ctas_per_lane(int f, int lanes, uint64_t e, uint64_t t) { return AutoCtasPerLane(f != 0, lanes, e, t); }
uint64_t yali_c_shard_elems(uint64_t count, int world) { return ShardElems(count, world); }

int yali_c_make_plan(int world, uint64_t count, int in_dt, int out_dt, int epilogue, int mode, const YaliPlanCaps* c,
                     const char* tuning_json, YaliPlan* out, char* err, size_t err_len) {
    PlanCaps caps;
    caps.flash_cap = c->flash_cap;
    caps.ring_bytes = c->ring_bytes;
    caps.nvls_cap = c->nvls_cap;
    caps.has_multicast = c->has_multicast != 0;
    caps.symmetric = c->symmetric != 0;
    caps.peer_recv = c->peer_recv != 0;
    caps.vec_ok = c->vec_ok != 0;
    caps.max_ctas = c->max_ctas;
    caps.ll_cap = c->ll_cap;
    caps.peer_send = c->peer_send != 0;
    caps.in_place = c->in_place != 0;
    caps.one_gpu_per_rank = c->one_gpu_per_rank != 0;
    TuningTable table;
    const TuningTable* tp = nullptr;
    std::string e;
    if (tuning_json && *tuning_json) {
        if (!TuningTable::Parse(tuning_json, &table, &e)) {
            CopyErr(e, err, err_len);
            return static_cast<int>(Result::InvalidArg);
        }
        tp = &table;
    }
    Plan p;
    Result r = MakePlan(world, count, static_cast<Dtype>(in_dt), static_cast<Dtype>(out_dt), epilogue,
                        static_cast<KernelMode>(mode), caps, tp, &p, &e);
    if (r != Result::Success) {
        CopyErr(e, err, err_len);
        return static_cast<int>(r);
    }
    out->variant = static_cast<int>(p.variant);
    out->ctas = p.ctas;
    out->slot_bytes = p.slot_bytes;
    out->max_iters = p.max_iters;
    out->flags = p.flags;
    out->shard_elems = p.shard_elems;
    out->stages = p.stages;
    out->smem_bytes = p.smem_bytes;
    return 0;
}

int yali_c_heap_layout(int world, uint64_t requested_total, uint64_t* f) {
    HeapLayout l;
    if (!MakeHeapLayout(world, requested_total, 0, &l)) return 1;
    const uint64_t v[16] = {l.total_bytes, l.flags_off, l.flash_off, l.flash_cap, l.ring_off,    l.ring_bytes,
                            l.nvls_off,    l.nvls_cap,  l.gemm_off,  l.gemm_cap,  l.user_off,    l.user_bytes,
                            l.ll_off,      l.ll_cap,    l.gemm_ll_off, l.gemm_ll_cap};
    std::memcpy(f, v, sizeof(v));
    return 0;
}

void yali_c_flash_slice(uint64_t count, int vec, uint32_t ctas, uint32_t cta, int vec_ok, uint64_t* o) {
    oracle::FlashSlice(count, vec, ctas, cta, vec_ok != 0, &o[0], &o[1], &o[2], &o[3]);
}
void yali_c_stream_piece(uint64_t count, uint64_t shard, uint64_t piece, uint32_t lanes, uint32_t lane, uint32_t it,
                         int q, uint64_t* o) {
    oracle::StreamPiece(count, shard, piece, lanes, lane, it, q, &o[0], &o[1]);
}
uint32_t yali_c_stream_iters(uint64_t shard, uint64_t piece, uint32_t lanes, uint32_t lane) {
    return oracle::StreamIters(shard, piece, lanes, lane);
}

void yali_c_philox(uint64_t seed, uint64_t index, uint32_t* out4) { Philox4x32(seed, index, out4); }
float yali_c_random_value(int dist, uint64_t seed, uint64_t index) { return RandomValue(dist, seed, index); }
void yali_c_fill_random(float* dst, uint64_t n, int dist, uint64_t seed, int round_dtype) {
    for (uint64_t i = 0; i < n; ++i) {
        float v = RandomValue(dist, seed, i);
        if (round_dtype == 1) v = oracle::RoundFp16(v);
        else if (round_dtype == 2) v = oracle::RoundBf16(v);
        dst[i] = v;
    }
}
float yali_c_round_bf16(float x) { return oracle::RoundBf16(x); }
float yali_c_round_fp16(float x) { return oracle::RoundFp16(x); }
void yali_c_oracle_allreduce(const float* const* in, int world, size_t n, double scale, double* out) {
    oracle::AllReduceSum(in, world, n, scale, out);
}
void yali_c_oracle_residual_rmsnorm(const double* sum, const float* residual, const float* weight, size_t rows,
                                    size_t hidden, double eps, double* y, double* pre_norm) {
    oracle::ResidualRmsNorm(sum, residual, weight, rows, hidden, eps, y, pre_norm);
}
void yali_c_fused_linear_counts(uint32_t T, uint32_t N, int world, int oneshot, uint32_t* arrivals, uint32_t* rows_of) {
    FusedLinearCounts(T, N, world, oneshot != 0, arrivals, rows_of);
}
uint32_t yali_c_fused_linear_oneshot_max_rows(int world) { return FusedLinearOneShotMaxRows(world); }
uint32_t yali_c_fused_tile_split(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t gemm_cap,
                                 uint32_t want) {
    return FusedLinearTileSplit(T, N, K, world, resident_ctas, gemm_cap, want);
}
uint32_t yali_c_fused_decode_tile(uint32_t N, uint32_t ksplit, uint32_t resident_ctas) {
    return FusedLinearDecodeTile(N, ksplit, resident_ctas);
}
uint32_t yali_c_fused_decode_split(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t ll_cap,
                                   uint32_t want) {
    return FusedLinearDecodeSplit(T, N, K, world, resident_ctas, ll_cap, want);
}
int yali_c_fused_linear_multicast_mode(int world, uint32_t T) { return FusedLinearAutoMulticastMode(world, T); }
void yali_c_oracle_gemm(const float* a, const float* b, size_t m, size_t n, size_t k, double* c) {
    oracle::Gemm(a, b, m, n, k, c);
}
int yali_c_verify_allreduce_sum(const float* host, size_t n, float expected, float tol, size_t* first,
                                size_t* count) {
    return VerifyAllReduceSum(host, n, expected, tol, first, count) ? 1 : 0;
}

}  // extern "C"
