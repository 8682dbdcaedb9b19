// Variant selection and launch geometry: which kernel (one-shot Flash, two-shot
// Stream, NVLS one-/two-shot), how many CTAs or lanes, which slot size.
//
// Parity: FlashCrossoverBytes / StreamLanePreset / FlashLanePreset /
// AutoSlotBytes / ClampSlotBytes / AutoCtasPerLane (src/include/yali_tuning.h:26-132)
// are compile-time constants tuned on 2x A100.  The same function names exist
// here, take the world size as well, and can be overridden at run time by a
// measured table (YALI_TUNING_FILE, written by the sweep tool) or by the
// YALI_KERNEL_MODE / YALI_DEV_* knobs.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "../comm/layout.h"
#include "../core/status.h"

namespace yali {

enum class Variant : int { Flash = 0, Stream = 1, NvlsOneShot = 2, NvlsTwoShot = 3, FlashPull = 4, StreamDirect = 5, CopyEngine = 6 };
const char* VariantName(Variant v);

// What the communicator can offer for this call.
struct PlanCaps {
    uint64_t flash_cap = 0;        // bytes of one-shot staging per source
    uint64_t ring_bytes = 0;       // bytes of the ring region
    uint64_t nvls_cap = 0;         // bytes of one NVLS staging half
    uint64_t ll_cap = 0;           // largest payload of the flag-in-data one-shot protocol
    bool has_multicast = false;
    bool symmetric = false;        // send and recv of every rank live in the heap at equal offsets
    bool peer_recv = false;        // every rank's recv is peer-addressable (direct all-gather possible)
    bool peer_send = false;        // every rank's send is peer-addressable (the pipelined kernels can pull it)
    bool in_place = false;         // some rank's send and recv ranges overlap
    bool one_gpu_per_rank = false; // every rank is a process with a GPU of its own (the copy-engine path needs it)
    bool half_collective = false;  // reduce-scatter-only / all-gather-only call (ring kernel only)
    uint32_t sm_count = 148;       // SMs of the GPU (resident CTAs of the pipelined kernels)
    bool vec_ok = true;            // all pointers 16-byte aligned
    uint32_t max_ctas = 296;       // upper bound on CTAs per rank (co-residency for emulated ranks)
    uint32_t force_ctas = 0;       // >0: caller's CTA / lane count (still clamped to the limits)
    uint32_t force_slot_bytes = 0; // >0: caller's ring slot size (still clamped to the ring region)
};

struct Plan {
    Variant variant = Variant::Flash;
    uint32_t ctas = 1;          // CTAs (Flash, NVLS) or lanes (Stream) per rank
    uint32_t slot_bytes = 0;    // Stream
    uint64_t shard_elems = 0;   // Stream, NVLS two-shot
    uint32_t max_iters = 0;     // Stream: sequence numbers consumed by this call
    uint32_t stages = 0;        // FlashPull / StreamDirect: shared-memory stages per CTA
    uint32_t smem_bytes = 0;    // dynamic shared memory per CTA
    uint32_t flags = 0;         // CollFlags
};

// ---- the reference's tuning entry points, generalised to a world size ----
// Largest message (bytes) that takes the one-shot path.
uint64_t FlashCrossoverBytes(Dtype dt, int world = 2);
// Largest message (bytes) that takes the flag-in-data form of the one-shot kernel (YALI_LL_MAX_BYTES).
uint64_t LowLatencyMaxBytes(int world = 2);
// CTAs of the one-shot kernel.
int FlashLanePreset(uint64_t bytes, Dtype dt, int world = 2);
// Lanes of the two-shot kernel.
int StreamLanePreset(uint64_t bytes, Dtype dt, int world = 2);
// Ring slot size for a message.
uint64_t AutoSlotBytes(uint64_t bytes, int world = 2);
uint64_t ClampSlotBytes(uint64_t slot_bytes, uint64_t max_bytes);
// Flash: how many CTAs serve one lane's elements (>=1); Stream: always 1.
int AutoCtasPerLane(bool use_flash, int lanes, uint64_t max_lane_elems, uint64_t tile_elems);

// Largest message (bytes) for which the one-shot pull beats the two-shot direct form.
uint64_t PullCrossoverBytes(int world);
// Smallest message the copy-engine path takes in auto mode.
uint64_t CopyEngineMinBytes(int world);
// CTAs, bytes per source and stage, and stages of the pipelined kernels.
void DirectPreset(uint64_t bytes, int world, bool one_shot, uint32_t sm_count, uint32_t* ctas, uint32_t* chunk_bytes,
                  uint32_t* stages);

// NVLS kernels: multimem loads in flight per thread (4 or 8) and the block size the CTAs of a rank
// interleave over its shard (0: one contiguous slice per CTA).
uint32_t NvlsUnrollPreset(uint64_t bytes, int world);
uint32_t NvlsBlockBytesPreset(uint64_t bytes, int world);

// Elements per shard for a two-shot algorithm: ceil(count/world) rounded up to 16 elements.
uint64_t ShardElems(uint64_t count, int world);

// One measured row: for `world` ranks and element size `elem_bytes`, messages up
// to `max_bytes` use `variant` with `ctas` CTAs/lanes and `slot_bytes` slots.
struct TuningRow {
    int world = 0;
    int elem_bytes = 0;  // 0 matches any
    uint64_t max_bytes = 0;
    Variant variant = Variant::Flash;
    uint32_t ctas = 0;        // 0: heuristic
    uint32_t slot_bytes = 0;  // 0: heuristic
};
class TuningTable {
   public:
    // Parses the JSON written by the sweep tool: {"rows":[{"world":2,"elem_bytes":4,
    // "max_bytes":65536,"variant":"flash","ctas":8,"slot_bytes":0}, ...]}.
    static bool Parse(const std::string& json, TuningTable* out, std::string* err);
    static bool Load(const std::string& path, TuningTable* out, std::string* err);
    const TuningRow* Find(int world, int elem_bytes, uint64_t bytes) const;
    const std::vector<TuningRow>& rows() const { return rows_; }
    void Add(const TuningRow& r);

   private:
    std::vector<TuningRow> rows_;  // sorted by (world, elem_bytes, max_bytes)
};
// Table from YALI_TUNING_FILE, loaded once; nullptr when unset or unreadable.
const TuningTable* EnvTuningTable();

// The decision.  `forced` == Auto lets the table / heuristics choose.
Result MakePlan(int world, uint64_t count, Dtype in, Dtype out, int epilogue, KernelMode forced, const PlanCaps& caps,
                const TuningTable* table, Plan* plan, std::string* why);

}  // namespace yali
