#include "tuning.h"

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <mutex>
#include <sstream>

#include "../core/env.h"

namespace yali {

const char* VariantName(Variant v) {
    switch (v) {
        case Variant::Flash: return "flash";
        case Variant::Stream: return "stream";
        case Variant::NvlsOneShot: return "nvls1";
        case Variant::NvlsTwoShot: return "nvls2";
        case Variant::FlashPull: return "flash_pull";
        case Variant::StreamDirect: return "stream_direct";
        case Variant::CopyEngine: return "copy_engine";
    }
    return "?";
}

namespace {
uint64_t CeilDiv(uint64_t a, uint64_t b) { return (a + b - 1) / b; }
uint64_t RoundUp(uint64_t a, uint64_t b) { return CeilDiv(a, b) * b; }
}  // namespace

// One-shot sends (N-1)*S per rank, two-shot 2(N-1)/N*S: at N=2 they tie and the
// one-shot wins on latency up to its staging capacity; at larger N the one-shot
// only pays off while the message is latency-bound. Measured on 2 x B200 (CUDA graph): the staged
// one-shot leads at 16 MiB (36.5 us against 37.3 us for the pipelined two-shot) and trails it at
// 64 MiB.
uint64_t FlashCrossoverBytes(Dtype /*dt*/, int world) {
    if (world <= 2) return 32ull << 20;
    if (world <= 4) return 1ull << 20;
    return 256ull << 10;
}

uint64_t LowLatencyMaxBytes(int world) {
    const long long e = env::GetInt("YALI_LL_MAX_BYTES", -1);
    if (e >= 0) return static_cast<uint64_t>(e);
    // Measured on 2 x B200 in a CUDA graph: at 1 MiB the flag-in-data form on 128 CTAs takes 10.9 us,
    // the flagged one-shot 11.9 us; at 4 MiB the flagged form leads (16.0 us).  From four ranks on
    // the doubled traffic only pays up to 256 KiB.
    return world <= 2 ? (1ull << 20) : (256ull << 10);
}

int FlashLanePreset(uint64_t bytes, Dtype /*dt*/, int /*world*/) {
    // Measured on 2 x B200: about 32 KiB per CTA is best from 64 KiB to a few MiB (more CTAs
    // only add launch and flag traffic), 128 CTAs from 16 MiB, 256 for the largest messages.
    if (bytes <= (4ull << 10)) return 1;
    if (bytes <= (512ull << 10)) return static_cast<int>(std::min<uint64_t>(CeilDiv(bytes, 4ull << 10), 16));
    if (bytes < (32ull << 20)) return static_cast<int>(std::min<uint64_t>(std::max<uint64_t>(CeilDiv(bytes, 32ull << 10), 16), 128));
    return 256;
}

int StreamLanePreset(uint64_t bytes, Dtype /*dt*/, int /*world*/) {
    if (bytes >= (64ull << 20)) return 148;
    if (bytes >= (8ull << 20)) return 128;
    if (bytes >= (1ull << 20)) return 64;
    return 16;
}

uint64_t AutoSlotBytes(uint64_t bytes, int world) {
    // Slot = one rank's piece of one shard.  Keep at least ~2 pieces per lane so
    // the three pipeline stages overlap, and at most 256 KiB.
    const uint64_t shard = CeilDiv(bytes, static_cast<uint64_t>(std::max(world, 1)));
    uint64_t s = 256ull << 10;
    while (s > (8ull << 10) && shard / s < 256) s >>= 1;
    return s;
}

uint64_t ClampSlotBytes(uint64_t slot_bytes, uint64_t max_bytes) {
    uint64_t s = std::max<uint64_t>(256, std::min(slot_bytes, max_bytes));
    s = std::min<uint64_t>(s, 1ull << 30);
    return s / 256 * 256;
}

int AutoCtasPerLane(bool use_flash, int lanes, uint64_t max_lane_elems, uint64_t tile_elems) {
    if (!use_flash || lanes <= 0 || max_lane_elems == 0) return 1;
    if (tile_elems == 0) tile_elems = 1;
    return static_cast<int>(std::min<uint64_t>(std::max<uint64_t>(CeilDiv(max_lane_elems, tile_elems), 1), 32));
}

uint64_t PullCrossoverBytes(int /*world*/) {
    // The one-shot pull needs two link trips around its loads (peers ready, peers done) where the
    // staged push needs one, and loads in both directions at once reach 660-670 GB/s per direction on
    // 2 x B200 where stores reach 705: measured 16.4 us against 10.9-11.9 us at 1 MiB and 27.8 us
    // against 16.0 us at 4 MiB.  It is therefore never picked by size; YALI_PULL_MAX_BYTES or the forced
    // mode select it (it needs no staging, so it also serves messages beyond the one-shot staging).
    const long long e = env::GetInt("YALI_PULL_MAX_BYTES", -1);
    return e >= 0 ? static_cast<uint64_t>(e) : 0;
}

uint64_t CopyEngineMinBytes(int /*world*/) {
    // Off by size unless YALI_CE_MIN_BYTES says from where; the forced mode selects it at any size.
    const long long e = env::GetInt("YALI_CE_MIN_BYTES", -1);
    return e >= 0 ? static_cast<uint64_t>(e) : ~0ull;
}

void DirectPreset(uint64_t bytes, int world, bool one_shot, uint32_t sm_count, uint32_t* ctas, uint32_t* chunk_bytes,
                  uint32_t* stages) {
    // A stage holds one chunk of every rank's input.  Measured on 2 and 4 x B200: one CTA per SM is
    // best from 16 MiB on (651 GB/s at 128 MiB on 2 GPUs against 630 with two per SM); at 2 ranks large
    // messages like 32 KiB chunks in 3 stages, otherwise about 96 KiB of stages per CTA in chunks of
    // 8 KiB (4 KiB from three ranks on) so that two CTAs can share an SM for small messages.
    const uint64_t budget = 96ull << 10;
    uint32_t chunk = world <= 2 ? (8u << 10) : (4u << 10);
    uint32_t st = static_cast<uint32_t>(budget / (static_cast<uint64_t>(chunk) * std::max(world, 1)));
    if (world <= 2 && bytes >= (128ull << 20) && !one_shot) {
        chunk = 32u << 10;
        st = 3;
    }
    st = std::max<uint32_t>(2, std::min<uint32_t>(st, kMaxPipelineStages));
    const uint64_t range = one_shot ? bytes : CeilDiv(bytes, static_cast<uint64_t>(std::max(world, 1)));
    const uint64_t n_chunks = std::max<uint64_t>(CeilDiv(range, chunk), 1);
    const uint64_t cap = bytes >= (16ull << 20) ? std::max<uint32_t>(sm_count, 1) : 2ull * std::max<uint32_t>(sm_count, 1);
    *ctas = static_cast<uint32_t>(std::min<uint64_t>(n_chunks, cap));
    *chunk_bytes = chunk;
    *stages = st;
}

uint32_t NvlsUnrollPreset(uint64_t /*bytes*/, int /*world*/) { return 4; }
uint32_t NvlsBlockBytesPreset(uint64_t /*bytes*/, int /*world*/) { return 0; }

uint64_t ShardElems(uint64_t count, int world) {
    return RoundUp(CeilDiv(count, static_cast<uint64_t>(std::max(world, 1))), 16);
}

// ------------------------------------------------------------------ tuning table
namespace {

struct Cursor {
    const std::string& s;
    size_t i = 0;
    void ws() {
        while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i;
    }
    bool eat(char c) {
        ws();
        if (i < s.size() && s[i] == c) {
            ++i;
            return true;
        }
        return false;
    }
    bool str(std::string* out) {
        ws();
        if (i >= s.size() || s[i] != '"') return false;
        size_t j = s.find('"', i + 1);
        if (j == std::string::npos) return false;
        *out = s.substr(i + 1, j - i - 1);
        i = j + 1;
        return true;
    }
    bool num(double* out) {
        ws();
        char* end = nullptr;
        *out = std::strtod(s.c_str() + i, &end);
        if (end == s.c_str() + i) return false;
        i = static_cast<size_t>(end - s.c_str());
        return true;
    }
};

bool ParseVariant(const std::string& v, Variant* out) {
    if (v == "flash") *out = Variant::Flash;
    else if (v == "stream") *out = Variant::Stream;
    else if (v == "nvls1") *out = Variant::NvlsOneShot;
    else if (v == "nvls2") *out = Variant::NvlsTwoShot;
    else if (v == "flash_pull") *out = Variant::FlashPull;
    else if (v == "stream_direct") *out = Variant::StreamDirect;
    else if (v == "copy_engine") *out = Variant::CopyEngine;
    else return false;
    return true;
}

}  // namespace

void TuningTable::Add(const TuningRow& r) {
    rows_.push_back(r);
    std::stable_sort(rows_.begin(), rows_.end(), [](const TuningRow& a, const TuningRow& b) {
        if (a.world != b.world) return a.world < b.world;
        if (a.elem_bytes != b.elem_bytes) return a.elem_bytes > b.elem_bytes;  // specific before wildcard 0
        return a.max_bytes < b.max_bytes;
    });
}

bool TuningTable::Parse(const std::string& json, TuningTable* out, std::string* err) {
    Cursor c{json};
    auto fail = [&](const char* m) {
        if (err) *err = std::string("tuning table: ") + m + " at offset " + std::to_string(c.i);
        return false;
    };
    if (!c.eat('{')) return fail("expected '{'");
    std::string key;
    if (!c.str(&key) || key != "rows" || !c.eat(':') || !c.eat('[')) return fail("expected \"rows\": [");
    TuningTable t;
    if (!c.eat(']')) {
        do {
            if (!c.eat('{')) return fail("expected '{' of a row");
            TuningRow row;
            bool have_variant = false;
            if (!c.eat('}')) {
                do {
                    if (!c.str(&key) || !c.eat(':')) return fail("expected \"key\":");
                    if (key == "variant") {
                        std::string v;
                        if (!c.str(&v) || !ParseVariant(v, &row.variant)) return fail("bad variant");
                        have_variant = true;
                    } else {
                        double x;
                        if (!c.num(&x) || x < 0) return fail("expected a non-negative number");
                        if (key == "world") row.world = static_cast<int>(x);
                        else if (key == "elem_bytes") row.elem_bytes = static_cast<int>(x);
                        else if (key == "max_bytes") row.max_bytes = static_cast<uint64_t>(x);
                        else if (key == "ctas") row.ctas = static_cast<uint32_t>(x);
                        else if (key == "slot_bytes") row.slot_bytes = static_cast<uint32_t>(x);
                        // unknown numeric keys (measurements kept for the record) are ignored
                    }
                } while (c.eat(','));
                if (!c.eat('}')) return fail("expected '}' of a row");
            }
            if (!have_variant || row.world < 1 || row.world > kMaxRanks || row.max_bytes == 0)
                return fail("row needs world, max_bytes and variant");
            t.Add(row);
        } while (c.eat(','));
        if (!c.eat(']')) return fail("expected ']'");
    }
    *out = t;
    return true;
}

bool TuningTable::Load(const std::string& path, TuningTable* out, std::string* err) {
    std::ifstream f(path);
    if (!f) {
        if (err) *err = "cannot open " + path;
        return false;
    }
    std::stringstream ss;
    ss << f.rdbuf();
    return Parse(ss.str(), out, err);
}

const TuningRow* TuningTable::Find(int world, int elem_bytes, uint64_t bytes) const {
    for (const TuningRow& r : rows_) {
        if (r.world != world) continue;
        if (r.elem_bytes != 0 && r.elem_bytes != elem_bytes) continue;
        if (bytes <= r.max_bytes) return &r;
    }
    return nullptr;
}

const TuningTable* EnvTuningTable() {
    static TuningTable table;
    static bool ok = false;
    static std::once_flag once;
    std::call_once(once, [] {
        std::string path = env::TuningFile();
        if (path.empty()) return;
        std::string err;
        ok = TuningTable::Load(path, &table, &err);
        if (!ok && env::DebugLevel() > 0) std::fprintf(stderr, "[yali] %s\n", err.c_str());
    });
    return ok ? &table : nullptr;
}

// ------------------------------------------------------------------ the plan
Result MakePlan(int world, uint64_t count, Dtype in, Dtype out, int epilogue, KernelMode forced, const PlanCaps& caps,
                const TuningTable* table, Plan* plan, std::string* why) {
    if (world < 1 || world > kMaxRanks) {
        if (why) *why = "world size out of range";
        return Result::InvalidArg;
    }
    const uint64_t in_b = DtypeSize(in), out_b = DtypeSize(out);
    const uint64_t bytes = count * in_b;
    const uint32_t max_ctas = std::max<uint32_t>(1, caps.max_ctas);
    Plan p;
    if (caps.vec_ok) p.flags |= kFlagVecOk;

    // Which variants can run this call at all.
    const bool rows = epilogue == kEpiResidualRmsNorm;
    const bool flash_ok = bytes <= caps.flash_cap || world == 1;
    const bool stream_ok = !rows && world > 1 && caps.ring_bytes > 0;
    // A rank's own alignment must not influence which kernel runs: with one GPU per process it is a
    // local fact, and ranks that chose differently would wait for each other until the deadline.  The
    // staged forms (one-shot, flag-in-data, ring, staged NVLS) therefore cope with buffers that are
    // aligned to their element type only; alignment matters for the plan only where all ranks share
    // it (symmetric buffers sit at one heap offset everywhere, ranks of one process are all known).
    const bool nvls_ok = !rows && world > 1 && caps.has_multicast && in == out && (bytes % 16 == 0) &&
                         (caps.symmetric ? caps.vec_ok : bytes <= caps.nvls_cap);
    // The pipelined kernels read every rank's input and (two-shot) write every rank's output in
    // place: all of them must be addressable and 16-byte aligned.  The one-shot pull overwrites
    // its output while peers may still read their inputs, so it cannot run in place.
    const bool direct_ok = !rows && world > 1 && caps.peer_send && caps.peer_recv && caps.vec_ok &&
                           !caps.half_collective;
    const bool pull_ok = direct_ok && !caps.in_place;
    // The copy-engine path: one GPU per rank, plain sum, every rank's shard non-empty.
    const bool ce_ok = direct_ok && caps.one_gpu_per_rank && in == out && epilogue == kEpiIdentity &&
                       static_cast<uint64_t>(world - 1) * ShardElems(count, world) < count;

    Variant v;
    const TuningRow* row = (table && forced == KernelMode::Auto) ? table->Find(world, static_cast<int>(in_b), bytes)
                                                                 : nullptr;
    if (forced == KernelMode::Flash) v = Variant::Flash;
    else if (forced == KernelMode::Stream) v = Variant::Stream;
    else if (forced == KernelMode::NVLS) v = bytes <= (128ull << 10) ? Variant::NvlsOneShot : Variant::NvlsTwoShot;
    else if (forced == KernelMode::FlashPull) v = Variant::FlashPull;
    else if (forced == KernelMode::StreamDirect) v = Variant::StreamDirect;
    else if (forced == KernelMode::CopyEngine) v = Variant::CopyEngine;
    else if (row) v = row->variant;
    // Measured on 8 x B200 with symmetric buffers: the flag-in-data one-shot wins up to 64 KiB
    // (8.3-13.5 us against 11-15 us), the in-switch forms from 128 KiB (16 us against 16-21 us).
    else if (nvls_ok && caps.symmetric && world > 4 && bytes > (64ull << 10))
        v = bytes <= (128ull << 10) ? Variant::NvlsOneShot : Variant::NvlsTwoShot;
    else if (bytes <= LowLatencyMaxBytes(world) && bytes <= caps.ll_cap) v = Variant::Flash;
    else if (pull_ok && bytes <= PullCrossoverBytes(world)) v = Variant::FlashPull;
    // With addressable buffers the pipelined two-shot overtakes the staged one-shot earlier: measured
    // on 2 x B200 (events) 8 MiB 26.5 against 36.4 us, 16 MiB 40.6 against 40.0, 32 MiB 71.2 against 64.2.
    else if (bytes <= (direct_ok && world == 2 ? std::min<uint64_t>(12ull << 20, FlashCrossoverBytes(in, world))
                                               : FlashCrossoverBytes(in, world)))
        v = Variant::Flash;
    else if (ce_ok && bytes >= CopyEngineMinBytes(world)) v = Variant::CopyEngine;
    else if (nvls_ok && world > 2) v = Variant::NvlsTwoShot;
    else if (direct_ok) v = Variant::StreamDirect;
    else v = Variant::Stream;

    // In place on symmetric buffers the in-switch one-shot would overwrite operands of the peers'
    // ld_reduce; the two-shot form reads and writes every element from one CTA of one rank only.
    if (v == Variant::NvlsOneShot && caps.symmetric && caps.in_place) v = Variant::NvlsTwoShot;

    // Fall back when the chosen variant cannot run; a forced mode that cannot run is an error.
    auto runnable = [&](Variant x) {
        switch (x) {
            case Variant::Flash: return flash_ok;
            case Variant::Stream: return stream_ok;
            case Variant::FlashPull: return pull_ok;
            case Variant::StreamDirect: return direct_ok;
            case Variant::CopyEngine: return ce_ok;
            default: return nvls_ok;
        }
    };
    if (!runnable(v)) {
        if (forced != KernelMode::Auto) {
            if (why)
                *why = std::string("kernel mode '") + KernelModeName(forced) +
                       "' cannot run this call (size, alignment, epilogue or missing multicast)";
            return Result::Unsupported;
        }
        if (direct_ok && v != Variant::StreamDirect) v = Variant::StreamDirect;
        else if (stream_ok) v = Variant::Stream;
        else if (flash_ok) v = Variant::Flash;
        else {
            if (why) *why = "message exceeds the one-shot staging capacity and no two-shot path is available";
            return Result::Unsupported;
        }
    }
    p.variant = v;

    // Per-call overrides win over the environment knobs.
    const int dev_ctas = caps.force_ctas ? static_cast<int>(caps.force_ctas) : env::DevCtas();
    const int dev_lanes = caps.force_ctas ? static_cast<int>(caps.force_ctas) : env::DevLanes();
    const long long dev_slot = caps.force_slot_bytes ? static_cast<long long>(caps.force_slot_bytes)
                                                      : env::DevSlotBytes();
    switch (v) {
        case Variant::Flash: {
            uint32_t c = row && row->ctas ? row->ctas : static_cast<uint32_t>(FlashLanePreset(bytes, in, world));
            if (dev_ctas > 0) c = dev_ctas;
            // Small messages of equal in/out type take the flag-in-data form (twice the bytes on
            // the wire, but no flag round trip).
            if (!rows && world > 1 && in == out && bytes % 16 == 0 && bytes <= caps.ll_cap &&
                bytes <= LowLatencyMaxBytes(world)) {
                p.flags |= kFlagLowLatency;
                if (!(row && row->ctas) && dev_ctas <= 0)
                    // about 16 KiB of pushes per CTA (each CTA pushes its slice to world-1 peers); from
                    // 512 KiB one 16-byte vector per thread (128 CTAs at 1 MiB measured fastest)
                    c = bytes > (512ull << 10)
                            ? 128u
                            : static_cast<uint32_t>(std::min<uint64_t>(
                                  std::max<uint64_t>(CeilDiv(bytes * (world - 1), 16ull << 10), 1), 64));
            }
            p.ctas = std::max<uint32_t>(1, std::min<uint32_t>(std::min<uint32_t>(c, max_ctas), kMaxFlashCtas));
            break;
        }
        case Variant::Stream: {
            const uint64_t elem = std::max(in_b, out_b);
            p.shard_elems = ShardElems(count, world);
            uint64_t slot = row && row->slot_bytes ? row->slot_bytes : AutoSlotBytes(count * elem, world);
            if (dev_slot > 0) slot = static_cast<uint64_t>(dev_slot);
            uint32_t lanes = row && row->ctas ? row->ctas : static_cast<uint32_t>(StreamLanePreset(bytes, in, world));
            if (dev_lanes > 0) lanes = dev_lanes;
            lanes = std::max<uint32_t>(1, std::min<uint32_t>(std::min<uint32_t>(lanes, max_ctas), kMaxLanes));
            // The rings of all lanes must fit: lanes * (world-1) * kRingCap * 2 * slot <= ring_bytes.
            const uint64_t per_lane_slots = static_cast<uint64_t>(world - 1) * kRingCap * 2;
            slot = ClampSlotBytes(slot, std::max<uint64_t>(256, caps.ring_bytes / (per_lane_slots * lanes)));
            if (slot * per_lane_slots * lanes > caps.ring_bytes) {
                lanes = static_cast<uint32_t>(std::max<uint64_t>(1, caps.ring_bytes / (per_lane_slots * slot)));
            }
            const uint64_t piece = slot / elem;
            const uint64_t n_pieces = CeilDiv(p.shard_elems, std::max<uint64_t>(piece, 1));
            lanes = static_cast<uint32_t>(std::min<uint64_t>(lanes, std::max<uint64_t>(n_pieces, 1)));
            p.ctas = lanes;
            p.slot_bytes = static_cast<uint32_t>(slot);
            p.max_iters = static_cast<uint32_t>(CeilDiv(n_pieces, lanes));
            if (caps.peer_recv) p.flags |= kFlagDirectAg;
            break;
        }
        case Variant::FlashPull:
        case Variant::StreamDirect: {
            const bool one_shot = v == Variant::FlashPull;
            p.shard_elems = ShardElems(count, world);
            uint32_t c, chunk, st;
            DirectPreset(bytes, world, one_shot, caps.sm_count, &c, &chunk, &st);
            if (row && row->ctas) c = row->ctas;
            if (row && row->slot_bytes) chunk = row->slot_bytes;
            if (dev_ctas > 0) c = dev_ctas;
            if (dev_slot > 0) chunk = static_cast<uint32_t>(dev_slot);
            const long long dev_stages = env::GetInt("YALI_DEV_STAGES", 0);
            chunk = std::max<uint32_t>(1024, std::min<uint32_t>(chunk, 64u << 10)) / 1024 * 1024;
            if (dev_stages > 0) st = static_cast<uint32_t>(dev_stages);
            // At most 200 KiB of stages per CTA.
            const uint32_t per_stage = chunk * static_cast<uint32_t>(world);
            st = std::max<uint32_t>(2, std::min<uint32_t>(std::min<uint32_t>(st, kMaxPipelineStages), (200u << 10) / per_stage));
            p.smem_bytes = st * per_stage;
            const uint32_t per_sm = std::max<uint32_t>(1, std::min<uint32_t>(2, (220u << 10) / (p.smem_bytes + 1024)));
            const uint32_t resident = per_sm * std::max<uint32_t>(caps.sm_count, 1);
            // `max_ctas` counts two CTAs per SM (emulated ranks share one GPU and one cooperative launch):
            // with stages so large that only one CTA fits an SM, half of that.
            const uint32_t share = std::max<uint32_t>(1, per_sm >= 2 ? max_ctas : max_ctas / 2);
            p.ctas = std::max<uint32_t>(1, std::min<uint32_t>(std::min<uint32_t>(c, share), std::min<uint32_t>(resident, kBarSlots)));
            p.slot_bytes = chunk;
            p.stages = st;
            if (one_shot) p.flags |= kFlagPullOneShot;
            break;
        }
        case Variant::CopyEngine: {
            // Two ranks: every rank copies the peer's whole input (S bytes per direction, one phase).
            // More ranks: two-shot over shards.  About eight chunks per rank keep the host's work per call
            // (six to twenty API calls per chunk) well below the time the copies take.
            const bool one_shot = world == 2;
            p.shard_elems = ShardElems(count, world);
            const uint64_t region = one_shot ? bytes : p.shard_elems * in_b;
            uint64_t chunk = std::min<uint64_t>(std::max<uint64_t>(RoundUp(CeilDiv(region, 8), 1ull << 20), 1ull << 20), 16ull << 20);
            if (dev_slot > 0) chunk = RoundUp(static_cast<uint64_t>(dev_slot), 16);
            chunk = std::max<uint64_t>(chunk, RoundUp(CeilDiv(region, 64), 16));  // at most 64 chunks per rank
            p.slot_bytes = static_cast<uint32_t>(chunk);
            p.stages = 3;  // staging slots per source
            if (env::GetInt("YALI_DEV_STAGES", 0) > 1) p.stages = static_cast<uint32_t>(std::min<long long>(env::GetInt("YALI_DEV_STAGES", 0), 8));
            uint32_t c = 2 * std::max<uint32_t>(caps.sm_count, 1);
            if (dev_ctas > 0) c = dev_ctas;
            p.ctas = std::max<uint32_t>(1, static_cast<uint32_t>(std::min<uint64_t>(c, CeilDiv(chunk, 16 * 512))));
            if (one_shot) p.flags |= kFlagPullOneShot;
            break;
        }
        case Variant::NvlsOneShot:
        case Variant::NvlsTwoShot: {
            p.shard_elems = ShardElems(count, world);
            // Measured on 8 x B200: the switch-side reduction saturates with few CTAs; 32 CTAs give
            // 843 GB/s bus bandwidth at 1 GiB where 148 give 725 and 296 give 636.
            // On 4 x B200 16 CTAs lead up to 128 MiB (658 against 650 GB/s at 128 MiB, 23.5 against 24.8 us
            // at 4 MiB); from 512 MiB 32 and 64 CTAs are level.
            const uint64_t nvls_cap_ctas = (world <= 4 && bytes < (256ull << 20)) ? 16 : 32;
            uint32_t c = row && row->ctas ? row->ctas
                                          : static_cast<uint32_t>(std::min<uint64_t>(
                                                std::max<uint64_t>(CeilDiv(bytes, 64ull << 10), 1), nvls_cap_ctas));
            if (v == Variant::NvlsTwoShot)
                c = static_cast<uint32_t>(std::min<uint64_t>(c, std::max<uint64_t>(CeilDiv(bytes / world, 8192), 1)));
            if (dev_ctas > 0) c = dev_ctas;
            p.ctas = std::max<uint32_t>(1, std::min<uint32_t>(std::min<uint32_t>(c, max_ctas), kBarSlots));
            if (caps.symmetric) p.flags |= kFlagSymmetric;
            // Loads in flight per thread (4 or 8) and, for symmetric two-shot calls, the size of the
            // blocks the CTAs interleave over the shard (0: one contiguous slice per CTA).
            p.stages = NvlsUnrollPreset(bytes, world);
            p.slot_bytes = caps.symmetric && v == Variant::NvlsTwoShot ? NvlsBlockBytesPreset(bytes, world) : 0;
            if (env::GetInt("YALI_DEV_STAGES", 0) > 0) p.stages = env::GetInt("YALI_DEV_STAGES", 0) >= 8 ? 8 : 4;
            if (dev_slot > 0 && caps.symmetric && v == Variant::NvlsTwoShot)
                p.slot_bytes = static_cast<uint32_t>(dev_slot) / 16 * 16;
            break;
        }
    }
    *plan = p;
    return Result::Success;
}

}  // namespace yali
