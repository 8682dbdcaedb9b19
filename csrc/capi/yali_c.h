/* Flat C interface to the host-side parts of the library (no GPU needed):
 * bootstrap, tuning / planning, partition arithmetic, the counter-based
 * generator, CPU oracles and the host-thread simulation of the ring protocol.
 * Python reaches these through ctypes for the CPU test tier; C and C++ users can
 * call them directly.
 *
 * Parity: the reference exposes its tuning functions only as C++ inlines
 * (src/include/yali_tuning.h) and has no host-side protocol model.
 */
#ifndef YALI_B200_C_H_
#define YALI_B200_C_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* yali_c_version(void);
const char* yali_c_error_string(int result);

/* ---- bootstrap ---- */
void* yali_c_bootstrap_create(int rank, int world, int local_rank, const char* job_id, int timeout_ms, char* err,
                              size_t err_len);
void* yali_c_bootstrap_from_env(char* err, size_t err_len);
void yali_c_bootstrap_destroy(void* bs);
int yali_c_bootstrap_rank(void* bs);
int yali_c_bootstrap_world(void* bs);
int yali_c_bootstrap_allgather(void* bs, const void* in, void* out, size_t bytes_each);
int yali_c_bootstrap_broadcast(void* bs, void* buf, size_t bytes, int root);
int yali_c_bootstrap_barrier(void* bs);
/* Every rank passes one descriptor; fds_out receives world descriptors. */
int yali_c_bootstrap_allgather_fd(void* bs, int my_fd, int* fds_out);
int yali_c_bootstrap_broadcast_fd(void* bs, int* fd_inout);
const char* yali_c_bootstrap_last_error(void* bs);

/* ---- tuning ---- */
uint64_t yali_c_flash_crossover_bytes(int dtype, int world);
int yali_c_flash_lane_preset(uint64_t bytes, int dtype, int world);
int yali_c_stream_lane_preset(uint64_t bytes, int dtype, int world);
uint64_t yali_c_auto_slot_bytes(uint64_t bytes, int world);
uint64_t yali_c_clamp_slot_bytes(uint64_t slot_bytes, uint64_t max_bytes);
int yali_c_auto_ctas_per_lane(int use_flash, int lanes, uint64_t max_lane_elems, uint64_t tile_elems);
uint64_t yali_c_shard_elems(uint64_t count, int world);

typedef struct YaliPlanCaps {
    uint64_t flash_cap, ring_bytes, nvls_cap;
    int has_multicast, symmetric, peer_recv, vec_ok;
    uint32_t max_ctas;
    uint64_t ll_cap;
    int peer_send, in_place; /* every input peer-addressable; some rank reduces in place */
    int one_gpu_per_rank;    /* every rank is a process with a GPU of its own (needed by the copy-engine path) */
} YaliPlanCaps;
typedef struct YaliPlan {
    int variant; /* 0 flash, 1 stream, 2 nvls one-shot, 3 nvls two-shot, 4 pipelined one-shot pull, 5 pipelined two-shot, 6 copy engines */
    uint32_t ctas, slot_bytes, max_iters, flags;
    uint64_t shard_elems;
    uint32_t stages, smem_bytes;
} YaliPlan;
/* mode: 0 auto, 1 flash, 2 stream, 3 nvls, 4 flash_pull, 5 stream_direct, 6 copy_engine.  tuning_json may be NULL.  Returns a Result code. */
int yali_c_make_plan(int world, uint64_t count, int in_dtype, int out_dtype, int epilogue, int mode,
                     const YaliPlanCaps* caps, const char* tuning_json, YaliPlan* plan, char* err, size_t err_len);
int yali_c_heap_layout(int world, uint64_t requested_total, uint64_t* fields /* 16 values: the 12 region fields, then ll_off, ll_cap, gemm_ll_off, gemm_ll_cap */);

/* ---- partition arithmetic (mirrors the device code) ---- */
void yali_c_flash_slice(uint64_t count, int vec, uint32_t ctas, uint32_t cta, int vec_ok, uint64_t* out4);
void yali_c_stream_piece(uint64_t count, uint64_t shard_elems, uint64_t piece_elems, uint32_t lanes, uint32_t lane,
                         uint32_t it, int q, uint64_t* out2);
uint32_t yali_c_stream_iters(uint64_t shard_elems, uint64_t piece_elems, uint32_t lanes, uint32_t lane);

/* ---- generator and oracles ---- */
void yali_c_philox(uint64_t seed, uint64_t index, uint32_t* out4);
float yali_c_random_value(int dist, uint64_t seed, uint64_t index);
void yali_c_fill_random(float* dst, uint64_t n, int dist, uint64_t seed, int round_dtype);
float yali_c_round_bf16(float x);
float yali_c_round_fp16(float x);
void yali_c_oracle_allreduce(const float* const* in, int world, size_t n, double scale, double* out);
void yali_c_oracle_residual_rmsnorm(const double* sum, const float* residual, const float* weight, size_t rows,
                                    size_t hidden, double eps, double* y, double* pre_norm);
// Fused linear layer: counter targets per owner (arrays of `world`), default one-shot limit and multicast form.
/* K splits per 256-column tile of the few-token fused layer (want = 0: the measured rule). */
uint32_t yali_c_fused_tile_split(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t gemm_cap,
                                 uint32_t want);
uint32_t yali_c_fused_decode_tile(uint32_t N, uint32_t ksplit, uint32_t resident_ctas);
uint32_t yali_c_fused_decode_split(uint32_t T, uint32_t N, uint32_t K, int world, uint32_t resident_ctas, uint64_t ll_cap,
                                   uint32_t want);
void yali_c_fused_linear_counts(uint32_t T, uint32_t N, int world, int oneshot, uint32_t* arrivals, uint32_t* rows_of);
uint32_t yali_c_fused_linear_oneshot_max_rows(int world);
int yali_c_fused_linear_multicast_mode(int world, uint32_t T);
void yali_c_oracle_gemm(const float* a, const float* b, size_t m, size_t n, size_t k, double* c);
int yali_c_verify_allreduce_sum(const float* host, size_t n, float expected, float tol, size_t* first_mismatch,
                                size_t* mismatch_count);

/* ---- host-thread simulation of the kernels' flag protocols ----
 * Runs `world` x `lanes` host threads that execute the same stage structure as
 * the two-shot ring kernel (mode 1), the one-shot kernel (mode 0), its flag-in-data form (mode 2) or
 * the staged two-shot through the switch (mode 3: per-CTA barriers, sums written back to every rank), the
 * pipelined two-shot in place (mode 4) or the pipelined one-shot pull (mode 5; both: two per-CTA barriers
 * per call, chunks of slot_elems elements, every rank rewrites its input between calls), or the copy-engine path
 * in place (mode 6 one-shot, mode 7 two-shot; lanes = 2: the caller's stream and the stream of the incoming
 * copies; direct_ag = 1 in mode 6 is the negative control without the wait before overwriting) on host memory, `calls` back-to-back calls without any barrier between them, fp32 data
 * from the generator.  fault: 0 none, 1 rank `fault_rank` never runs call
 * `fault_call` (its peers must time out, not hang), 2 one flag publication of
 * that rank is dropped.  Returns 0 when every output matches the fp64 oracle,
 * 1 on a data mismatch, 2 when a wait timed out (expected with a fault),
 * 3 on a protocol-invariant violation (credit > capacity, sequence going back).
 */
typedef struct YaliSimConfig {
    int mode, world, lanes, calls;
    uint64_t count;
    uint32_t slot_elems;
    int direct_ag;
    int fault, fault_rank, fault_call;
    int timeout_ms;
    uint64_t seed;
} YaliSimConfig;
typedef struct YaliSimReport {
    int status;
    uint64_t mismatches, timeouts, max_outstanding_slots, flag_writes;
    int timeout_rank, timeout_peer, timeout_site;
} YaliSimReport;
int yali_c_simulate(const YaliSimConfig* cfg, YaliSimReport* rep);

/* Host-thread model of the fused GEMM layer's cross-rank protocol (sim/gemm_protocol_sim.cc):
 * `world` x `ctas` threads, `calls` back-to-back calls of a [rows, col_tiles x 128] layer, two-shot or
 * one-shot.  fault: 0 none, 1 rank `fault_rank` stops launching from call `fault_call`, 2 one tile
 * announcement of that rank is lost.  slow_rank (-1: none) sleeps before its reduce phase, so that the
 * other ranks run ahead.  single_parity = 1 removes the double buffering of the landing zones (a
 * negative control: the stamps must then catch the reuse in one-shot mode).  in_switch = 1 models the
 * two-shot form whose owners read every rank's own image.  Same return codes and
 * report as yali_c_simulate; flag_writes counts counter updates. */
typedef struct YaliFusedSimConfig {
    int world, ctas, calls, oneshot;
    uint32_t rows, col_tiles;
    int fault, fault_rank, fault_call;
    int slow_rank, single_parity;
    int timeout_ms;
    int in_switch; /* 1: partial rows stay in the producer's own image and the owner reads all ranks' images */
    int ksplit;    /* > 0: the few-token form instead (flag-in-data lines from world x ksplit sources to every rank,
                      CTA t sums row t; rows <= 64; flag_writes counts lines; fault 2 loses the lines of one item) */
} YaliFusedSimConfig;
int yali_c_simulate_fused(const YaliFusedSimConfig* cfg, YaliSimReport* rep);

#ifdef __cplusplus
}
#endif
#endif
