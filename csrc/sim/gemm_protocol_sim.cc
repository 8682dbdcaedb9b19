// Host-thread model of the fused GEMM layer's cross-rank protocol (yali_c.h,
// yali_c_simulate_fused).  One host thread plays one CTA of one rank.  What it
// models is everything of kernels/gemm_ar_rmsnorm.cu that involves another rank:
// the walk over the tiles (rotated per rank), the push of partial rows into the
// owner's landing zone of the call's parity, the arrival counters with the
// host-computed targets (ops/fused_linear.cc, FusedLinearCounts), the reduction of
// the owned rows, the delivery into every rank's output, the delivered-row counters
// and the call words that the last CTA of a launch advances.  A "row segment" is one
// float per (row, column tile); the GEMM itself is a formula of (rank, call, row,
// column tile).  Calls follow one another with no barrier between ranks; CTAs of one
// rank meet between calls, as kernels of one stream do.
//
// Every landing cell and every output cell carries a stamp that is NOT part of the
// protocol: a producer that finds a cell still FULL, or a consumer that finds the
// stamp of another call, has caught the protocol reusing memory too early (the two
// call parities, or an output that a fast peer overwrites before the slow rank's
// stream has consumed it), which on the device would be silent corruption.
//
// Parity: the reference has neither the fused layer nor a protocol model.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../capi/yali_c.h"
#include "../comm/layout.h"
#include "../kernels/gemm_ar_rmsnorm.h"
#include "../ops/fused_linear.h"

namespace {

using Clock = std::chrono::steady_clock;

struct RankBarrier {
    std::mutex m;
    std::condition_variable cv;
    int count, waiting = 0, gen = 0;
    explicit RankBarrier(int n) : count(n) {}
    void wait() {
        std::unique_lock<std::mutex> l(m);
        int g = gen;
        if (++waiting == count) {
            waiting = 0;
            ++gen;
            cv.notify_all();
        } else {
            cv.wait(l, [&] { return g != gen; });
        }
    }
};

struct Cell {
    std::atomic<uint64_t> stamp{0};  // 0 = FREE, else call + 1
    float value = 0.f;
};

struct FusedShared {
    YaliFusedSimConfig cfg;
    int W, C;
    uint32_t T, ntn, ntm, bm, Rs;
    // landing[on_rank]: [parity][src][row_local][nt]
    std::vector<std::unique_ptr<Cell[]>> landing;
    // out[on_rank]: [row][nt]
    std::vector<std::unique_ptr<Cell[]>> out;
    // counters per rank: arrivals[src], delivered[owner]; call words: epoch, cnt target, done targets
    struct Words {
        std::atomic<uint32_t> cnt[yali::kMaxRanks], done[yali::kMaxRanks];
        std::atomic<uint32_t> epoch{0}, cnt_base{0}, done_base[yali::kMaxRanks], checked_out{0};
    };
    std::unique_ptr<Words[]> words;
    std::vector<std::unique_ptr<RankBarrier>> barrier;
    std::atomic<uint64_t> timeouts{0}, violations{0}, mismatches{0}, counter_writes{0};
    std::atomic<int> t_rank{-1}, t_peer{-1}, t_site{0};
    std::atomic<bool> abort{false};

    size_t ImageIndex(uint32_t parity, uint32_t row, uint32_t nt) const {
        return (static_cast<size_t>(parity) * T + row) * ntn + nt;
    }
    size_t LandingIndex(uint32_t parity, int src, uint32_t row_local, uint32_t nt) const {
        return ((static_cast<size_t>(parity) * W + src) * Rs + row_local) * ntn + nt;
    }
};

float Partial(int rank, int call, uint32_t row, uint32_t nt) {
    return static_cast<float>((rank * 131 + call * 17 + row * 7 + nt * 3) % 251) * 0.125f - 9.0f;
}

bool Reached(uint32_t seen, uint32_t wanted) { return static_cast<int32_t>(seen - wanted) >= 0; }

bool WaitCounter(FusedShared& s, std::atomic<uint32_t>& w, uint32_t wanted, int rank, int peer, int site) {
    const auto deadline = Clock::now() + std::chrono::milliseconds(s.cfg.timeout_ms);
    uint32_t spins = 0;
    while (!Reached(w.load(std::memory_order_acquire), wanted)) {
        if ((++spins & 255u) == 0) {
            if (s.abort.load() || Clock::now() > deadline) {
                if (s.timeouts.fetch_add(1) == 0) {
                    s.t_rank = rank;
                    s.t_peer = peer;
                    s.t_site = site;
                }
                s.abort = true;
                return false;
            }
            std::this_thread::yield();
        }
    }
    return true;
}

struct RankStop {
    std::atomic<int> v{0};
};

void FusedCta(FusedShared& s, std::vector<RankStop>& stop, int r, int c) {
    const int W = s.W, C = s.C;
    const bool oneshot = s.cfg.oneshot != 0;
    const uint32_t T = s.T, ntn = s.ntn, ntm = s.ntm, bm = s.bm, Rs = s.Rs;
    uint32_t arrivals[yali::kMaxRanks], rows_of[yali::kMaxRanks];
    yali::FusedLinearCounts(T, ntn * yali::kGemmTileN, W, oneshot, arrivals, rows_of);
    FusedShared::Words& mine = s.words[r];
    const uint32_t shift = oneshot ? 0u : (((static_cast<uint32_t>(r) + 1u) % W) * Rs / bm) % ntm;
    for (int call = 0; call < s.cfg.calls; ++call) {
        if (s.cfg.fault == 1 && r == s.cfg.fault_rank && call >= s.cfg.fault_call) break;  // stops launching
        // Call words as the previous launch of this rank left them.
        const uint32_t epoch = mine.epoch.load(std::memory_order_acquire);
        const uint32_t parity = s.cfg.single_parity ? 0u : ((epoch + 1u) & 1u);
        const uint32_t cnt_wanted = mine.cnt_base.load() + arrivals[r];
        const uint64_t stamp = static_cast<uint64_t>(call) + 1;
        bool ok = true;
        // ---- phase 1: tiles -> owners' landing zones, then one announcement per owner touched
        for (uint32_t tile = c; tile < ntm * ntn; tile += C) {
            const uint32_t mt = (tile / ntn + shift) % ntm, nt = tile % ntn;
            const uint32_t lo = mt * bm, hi = std::min(T, lo + bm);
            for (uint32_t row = lo; row < hi; ++row) {
                const float v = Partial(r, call, row, nt);
                if (s.cfg.in_switch) {
                    // In-switch form: the partial row stays in this rank's own image of the call parity.
                    Cell& cell = s.landing[r][s.ImageIndex(parity, row, nt)];
                    if (cell.stamp.load(std::memory_order_acquire) != 0) s.violations.fetch_add(1);  // still unread
                    cell.value = v;
                    cell.stamp.store(stamp, std::memory_order_release);
                    continue;
                }
                for (int d = 0; d < W; ++d) {
                    if (!oneshot && static_cast<uint32_t>(d) != row / Rs) continue;
                    Cell& cell = s.landing[d][s.LandingIndex(parity, r, oneshot ? row : row - d * Rs, nt)];
                    if (cell.stamp.load(std::memory_order_acquire) != 0) s.violations.fetch_add(1);  // still unread
                    cell.value = v;
                    cell.stamp.store(stamp, std::memory_order_release);
                }
            }
            for (int q = 0; q < W; ++q) {
                const bool touched = oneshot || (static_cast<uint32_t>(q) * Rs < hi && (static_cast<uint32_t>(q) + 1) * Rs > lo);
                if (!touched) continue;
                if (s.cfg.fault == 2 && r == s.cfg.fault_rank && call == s.cfg.fault_call && tile == static_cast<uint32_t>(c))
                    continue;  // this announcement is lost
                s.words[q].cnt[r].fetch_add(1, std::memory_order_release);
                s.counter_writes.fetch_add(1, std::memory_order_relaxed);
            }
        }
        if (r == s.cfg.slow_rank) std::this_thread::sleep_for(std::chrono::milliseconds(2));
        // ---- phase 2: reduce the owned rows, deliver them
        const uint32_t row_lo = oneshot ? 0u : std::min(T, static_cast<uint32_t>(r) * Rs);
        const uint32_t row_hi = oneshot ? T : std::min(T, row_lo + Rs);
        const uint32_t my_rows = row_hi - row_lo;
        if (my_rows > 0) {
            for (int src = 0; src < W && ok; ++src) ok = WaitCounter(s, mine.cnt[src], cnt_wanted, r, src, 1);
            uint32_t rows_done = 0;
            for (uint32_t lr = c; ok && lr < my_rows; lr += C) {
                const uint32_t grow = row_lo + lr;
                for (uint32_t nt = 0; nt < ntn; ++nt) {
                    float sum = 0.f;
                    for (int src = 0; src < W; ++src) {
                        // in-switch form: the switch reads every rank's own image at the row's offset
                        Cell& cell = s.cfg.in_switch ? s.landing[src][s.ImageIndex(parity, grow, nt)]
                                                     : s.landing[r][s.LandingIndex(parity, src, lr, nt)];
                        if (cell.stamp.load(std::memory_order_acquire) != stamp) s.violations.fetch_add(1);
                        sum += cell.value;
                        cell.stamp.store(0, std::memory_order_release);
                    }
                    for (int d = 0; d < W; ++d) {
                        if (oneshot && d != r) continue;
                        Cell& o = s.out[d][static_cast<size_t>(grow) * ntn + nt];
                        if (o.stamp.load(std::memory_order_acquire) != 0) s.violations.fetch_add(1);  // not consumed yet
                        o.value = sum;
                        o.stamp.store(stamp, std::memory_order_release);
                    }
                }
                ++rows_done;
            }
            if (!oneshot && rows_done > 0)
                for (int q = 0; q < W; ++q) {
                    s.words[q].done[r].fetch_add(rows_done, std::memory_order_release);
                    s.counter_writes.fetch_add(1, std::memory_order_relaxed);
                }
        }
        if (!oneshot && c == 0)
            for (int q = 0; q < W && ok; ++q)
                ok = WaitCounter(s, mine.done[q], mine.done_base[q].load() + rows_of[q], r, q, 2);
        // ---- the launch ends when all its CTAs have; the last one advances the call words, then the
        // rank's stream consumes the output before it launches the next call.
        s.barrier[r]->wait();
        if (c == 0) {
            const bool aborted = s.abort.load();
            if (!aborted) {
                mine.epoch.fetch_add(1, std::memory_order_release);
                mine.cnt_base.fetch_add(arrivals[r]);
                for (int q = 0; q < W; ++q) mine.done_base[q].fetch_add(rows_of[q]);
                for (uint32_t row = 0; row < T; ++row)
                    for (uint32_t nt = 0; nt < ntn; ++nt) {
                        Cell& o = s.out[r][static_cast<size_t>(row) * ntn + nt];
                        float want = 0.f;
                        for (int q = 0; q < W; ++q) want += Partial(q, call, row, nt);
                        if (o.stamp.load(std::memory_order_acquire) != stamp) s.violations.fetch_add(1);
                        else if (std::fabs(o.value - want) > 1e-3f) s.mismatches.fetch_add(1);
                        o.stamp.store(0, std::memory_order_release);
                    }
            }
            stop[r].v.store(aborted ? 1 : 0);
        }
        s.barrier[r]->wait();
        if (stop[r].v.load()) break;
    }
}

// ---- the few-token form (kernels/gemm_ar_decode.cu): flag-in-data lines, no counters.
// A line is one 64-bit word {call number, value}: the device writes 16 bytes with one store, so the
// number and the payload arrive together.  Source (rank, K split) owns one landing zone per call
// parity on every rank.  A work item is (column tile, K split); CTA c takes items c, c + C, ...,
// pushes the partial of every row to every rank, then CTA t < T sums row t over all sources.
struct DecodeShared {
    YaliFusedSimConfig cfg;
    int W, C;
    uint32_t T, ntn, ks;
    // lines[on_rank]: [parity][src rank][split][row][tile]
    std::vector<std::unique_ptr<std::atomic<uint64_t>[]>> lines;
    std::vector<std::unique_ptr<Cell[]>> out;  // [row][tile]
    std::unique_ptr<std::atomic<uint32_t>[]> call_word;  // per rank: calls completed
    std::vector<std::unique_ptr<RankBarrier>> barrier;
    std::atomic<uint64_t> timeouts{0}, violations{0}, mismatches{0}, line_writes{0};
    std::atomic<int> t_rank{-1}, t_peer{-1}, t_site{0};
    std::atomic<bool> abort{false};
    size_t Line(uint32_t parity, int src, uint32_t split, uint32_t row, uint32_t tile) const {
        return ((((static_cast<size_t>(parity) * W + src) * ks + split) * T + row) * ntn + tile);
    }
};

float PartialSplit(int rank, int call, uint32_t row, uint32_t nt, uint32_t split) {
    return static_cast<float>((rank * 131 + call * 17 + row * 7 + nt * 3 + split * 29) % 251) * 0.125f - 9.0f;
}

void DecodeCta(DecodeShared& s, std::vector<RankStop>& stop, int r, int c) {
    const int W = s.W, C = s.C;
    const uint32_t T = s.T, ntn = s.ntn, ks = s.ks;
    for (int call = 0; call < s.cfg.calls; ++call) {
        if (s.cfg.fault == 1 && r == s.cfg.fault_rank && call >= s.cfg.fault_call) break;  // stops launching
        const uint32_t number = s.call_word[r].load(std::memory_order_acquire) + 1u;  // this call, never 0
        const uint32_t parity = s.cfg.single_parity ? 0u : (number & 1u);
        // ---- phase 1: every row of every item of this CTA to every rank
        for (uint32_t item = c; item < ntn * ks; item += C) {
            const uint32_t tile = item / ks, split = item % ks;
            if (s.cfg.fault == 2 && r == s.cfg.fault_rank && call == s.cfg.fault_call && item == static_cast<uint32_t>(c))
                continue;  // the lines of this item are lost
            for (int k = 0; k < W; ++k) {
                const int d = (r + k) % W;
                for (uint32_t row = 0; row < T; ++row) {
                    float v = PartialSplit(r, call, row, tile, split);
                    uint32_t bits;
                    std::memcpy(&bits, &v, 4);
                    s.lines[d][s.Line(parity, r, split, row, tile)].store((static_cast<uint64_t>(number) << 32) | bits,
                                                                         std::memory_order_release);
                    s.line_writes.fetch_add(1, std::memory_order_relaxed);
                }
            }
        }
        if (r == s.cfg.slow_rank) std::this_thread::sleep_for(std::chrono::milliseconds(2));
        // ---- phase 2: CTA t sums row t on this rank
        bool ok = true;
        const auto deadline = Clock::now() + std::chrono::milliseconds(s.cfg.timeout_ms);
        for (uint32_t row = c; ok && row < T; row += C) {
            for (uint32_t tile = 0; ok && tile < ntn; ++tile) {
                float sum = 0.f;
                for (int src = 0; ok && src < W; ++src) {
                    for (uint32_t split = 0; ok && split < ks; ++split) {
                        std::atomic<uint64_t>& line = s.lines[r][s.Line(parity, src, split, row, tile)];
                        uint32_t spins = 0;
                        uint64_t w;
                        while (static_cast<uint32_t>((w = line.load(std::memory_order_acquire)) >> 32) != number) {
                            // A later call's number here means that the zone was reused before this reader was done.
                            if (static_cast<int32_t>(static_cast<uint32_t>(w >> 32) - number) > 0 && (w >> 32) != 0) {
                                s.violations.fetch_add(1);
                                ok = false;
                                break;
                            }
                            if ((++spins & 255u) == 0) {
                                if (s.abort.load() || Clock::now() > deadline) {
                                    if (s.timeouts.fetch_add(1) == 0) {
                                        s.t_rank = r;
                                        s.t_peer = src;
                                        s.t_site = 1;
                                    }
                                    s.abort = true;
                                    ok = false;
                                    break;
                                }
                                std::this_thread::yield();
                            }
                        }
                        if (!ok) break;
                        const uint32_t bits = static_cast<uint32_t>(w);
                        float v;
                        std::memcpy(&v, &bits, 4);
                        sum += v;
                    }
                }
                if (!ok) break;
                Cell& o = s.out[r][static_cast<size_t>(row) * ntn + tile];
                if (o.stamp.load(std::memory_order_acquire) != 0) s.violations.fetch_add(1);  // not consumed yet
                o.value = sum;
                o.stamp.store(static_cast<uint64_t>(call) + 1, std::memory_order_release);
            }
        }
        // ---- end of the launch: the last CTA advances the call word; the stream consumes the output
        s.barrier[r]->wait();
        if (c == 0) {
            const bool aborted = s.abort.load();
            if (!aborted) {
                s.call_word[r].fetch_add(1, std::memory_order_release);
                for (uint32_t row = 0; row < T; ++row)
                    for (uint32_t tile = 0; tile < ntn; ++tile) {
                        Cell& o = s.out[r][static_cast<size_t>(row) * ntn + tile];
                        float want = 0.f;
                        for (int q = 0; q < W; ++q)
                            for (uint32_t split = 0; split < ks; ++split) want += PartialSplit(q, call, row, tile, split);
                        if (o.stamp.load(std::memory_order_acquire) != static_cast<uint64_t>(call) + 1) s.violations.fetch_add(1);
                        else if (std::fabs(o.value - want) > 1e-3f) s.mismatches.fetch_add(1);
                        o.stamp.store(0, std::memory_order_release);
                    }
            }
            stop[r].v.store(aborted ? 1 : 0);
        }
        s.barrier[r]->wait();
        if (stop[r].v.load()) break;
    }
}

int SimulateDecode(const YaliFusedSimConfig* cfg, YaliSimReport* rep) {
    if (cfg->rows > yali::kGemmDecodeMaxRows || cfg->ksplit > static_cast<int>(yali::kGemmDecodeMaxSplit)) return -1;
    DecodeShared s;
    s.cfg = *cfg;
    s.W = cfg->world;
    s.C = cfg->ctas;
    s.T = cfg->rows;
    s.ntn = cfg->col_tiles;
    s.ks = static_cast<uint32_t>(cfg->ksplit);
    const size_t nlines = 2ull * s.W * s.ks * s.T * s.ntn;
    s.call_word.reset(new std::atomic<uint32_t>[s.W]);
    for (int r = 0; r < s.W; ++r) {
        s.lines.emplace_back(new std::atomic<uint64_t>[nlines]);
        for (size_t i = 0; i < nlines; ++i) s.lines[r][i].store(0);
        s.out.emplace_back(new Cell[static_cast<size_t>(s.T) * s.ntn]);
        s.call_word[r].store(0);
        s.barrier.emplace_back(new RankBarrier(s.C));
    }
    std::vector<RankStop> stop(s.W);
    std::vector<std::thread> threads;
    for (int r = 0; r < s.W; ++r)
        for (int c = 0; c < s.C; ++c) threads.emplace_back(DecodeCta, std::ref(s), std::ref(stop), r, c);
    for (auto& t : threads) t.join();
    rep->timeouts = s.timeouts.load();
    rep->flag_writes = s.line_writes.load();
    rep->timeout_rank = s.t_rank.load();
    rep->timeout_peer = s.t_peer.load();
    rep->timeout_site = s.t_site.load();
    if (s.violations.load()) {
        rep->mismatches = s.violations.load();
        return rep->status = 3;
    }
    if (rep->timeouts) return rep->status = 2;
    rep->mismatches = s.mismatches.load();
    return rep->status = rep->mismatches ? 1 : 0;
}

}  // namespace

extern "C" int yali_c_simulate_fused(const YaliFusedSimConfig* cfg, YaliSimReport* rep) {
    std::memset(rep, 0, sizeof(*rep));
    rep->timeout_rank = rep->timeout_peer = -1;
    if (!cfg || cfg->world < 1 || cfg->world > yali::kMaxRanks || cfg->ctas < 1 || cfg->ctas > 64 || cfg->rows == 0 ||
        cfg->col_tiles == 0 || cfg->calls < 1)
        return -1;
    if (cfg->ksplit > 0) return SimulateDecode(cfg, rep);
    FusedShared s;
    s.cfg = *cfg;
    s.W = cfg->world;
    s.C = cfg->ctas;
    s.T = cfg->rows;
    s.ntn = cfg->col_tiles;
    s.bm = yali::kGemmTileM;
    s.ntm = (s.T + s.bm - 1) / s.bm;
    s.Rs = cfg->oneshot ? s.T : (s.T + s.W - 1) / s.W;
    if (cfg->in_switch && cfg->oneshot) return -1;  // the in-switch form is a two-shot form
    const size_t nland = std::max<size_t>(2ull * s.W * s.Rs * s.ntn, 2ull * s.T * s.ntn);
    const size_t nout = static_cast<size_t>(s.T) * s.ntn;
    s.words.reset(new FusedShared::Words[s.W]);
    for (int r = 0; r < s.W; ++r) {
        s.landing.emplace_back(new Cell[nland]);
        s.out.emplace_back(new Cell[nout]);
        for (int q = 0; q < yali::kMaxRanks; ++q) {
            s.words[r].cnt[q].store(0);
            s.words[r].done[q].store(0);
            s.words[r].done_base[q].store(0);
        }
        s.barrier.emplace_back(new RankBarrier(s.C));
    }
    std::vector<RankStop> stop(s.W);
    std::vector<std::thread> threads;
    for (int r = 0; r < s.W; ++r)
        for (int c = 0; c < s.C; ++c) threads.emplace_back(FusedCta, std::ref(s), std::ref(stop), r, c);
    for (auto& t : threads) t.join();
    rep->timeouts = s.timeouts.load();
    rep->flag_writes = s.counter_writes.load();
    rep->timeout_rank = s.t_rank.load();
    rep->timeout_peer = s.t_peer.load();
    rep->timeout_site = s.t_site.load();
    if (s.violations.load()) {
        rep->mismatches = s.violations.load();
        return rep->status = 3;
    }
    if (rep->timeouts) return rep->status = 2;
    rep->mismatches = s.mismatches.load();
    return rep->status = rep->mismatches ? 1 : 0;
}
