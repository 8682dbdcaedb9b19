// Host-thread model of the kernels' cross-rank protocols (see yali_c.h,
// yali_c_simulate).  One host thread plays one CTA (a lane of the two-shot ring
// kernel or a CTA of the one-shot kernel) of one rank; all "device memory" is host
// memory and flags are std::atomic with release/acquire ordering, which is what
// st.release.sys / ld.acquire.sys give the device code.  Calls follow one another
// without any barrier between ranks; lanes of one rank meet between calls, as
// kernels of one stream do.  Every slot and staging slice carries a FULL/FREE stamp
// that is NOT part of the protocol: a producer that finds FULL, or a consumer that
// finds a stamp of the wrong iteration, has caught the protocol reusing memory too
// early, which the real kernels could only show as silent corruption.
//
// Parity: the reference has no such model; its protocol is described in comments
// only (src/kernels/ring.cuh:18-34, src/kernels/stream.cuh:8-37,140-145).
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
#include "../ops/buffer_ops.h"
#include "../ops/host_oracle.h"
#include "../ops/tuning.h"

namespace {

using Clock = std::chrono::steady_clock;

struct Barrier {
    std::mutex m;
    std::condition_variable cv;
    int count, waiting = 0, gen = 0;
    explicit Barrier(int n) : count(n) {}
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

struct Shared {
    YaliSimConfig cfg;
    int W, L;
    // flags[rank][kind][lane][src]
    std::vector<std::unique_ptr<std::atomic<uint32_t>[]>> flags;
    // slots[rank][lane][srcslot][cap][which] -> data + stamp
    std::vector<std::vector<float>> ring;          // per rank
    std::vector<std::unique_ptr<std::atomic<uint64_t>[]>> ring_stamp;  // per rank, one per slot; 0 = FREE
    std::vector<std::vector<float>> stage;         // one-shot staging per rank: [2][W-1][count]
    std::vector<std::unique_ptr<std::atomic<uint64_t>[]>> stage_stamp;  // [2][W-1][ctas]
    // flag-in-data form: one 64-bit word per element = {call number, value bits}, [2][W-1][count] per rank
    std::vector<std::unique_ptr<std::atomic<uint64_t>[]>> ll;
    std::vector<std::vector<float>> send, recv;
    std::vector<std::unique_ptr<Barrier>> rank_barrier;
    std::unique_ptr<std::atomic<int>[]> rank_abort;  // agreed between the lanes of a rank at the barrier
    std::atomic<uint64_t> timeouts{0}, violations{0}, flag_writes{0}, max_outstanding{0};
    std::atomic<int> t_rank{-1}, t_peer{-1}, t_site{0};
    std::atomic<bool> abort{false};
    int dropped = 0;
    std::mutex drop_m;
};

enum Kind { kRs = 0, kAg = 1, kCr = 2, kFlash = 3, kKinds = 4 };

std::atomic<uint32_t>& Flag(Shared& s, int on_rank, int kind, int lane, int src) {
    return s.flags[on_rank][(static_cast<size_t>(kind) * s.L + lane) * yali::kMaxRanks + src];
}

bool SeqReached(uint32_t seen, uint32_t wanted) { return static_cast<int32_t>(seen - wanted) >= 0; }

// Waits for the flags of all peers; false on timeout or global abort.
bool WaitPeers(Shared& s, int rank, int kind, int lane, uint32_t wanted, int site) {
    auto deadline = Clock::now() + std::chrono::milliseconds(s.cfg.timeout_ms);
    for (int p = 0; p < s.W; ++p) {
        if (p == rank) continue;
        uint32_t spins = 0;
        while (!SeqReached(Flag(s, rank, kind, lane, p).load(std::memory_order_acquire), wanted)) {
            if ((++spins & 255u) == 0) {
                if (s.abort.load() || Clock::now() > deadline) {
                    if (s.timeouts.fetch_add(1) == 0) {
                        s.t_rank = rank;
                        s.t_peer = p;
                        s.t_site = site;
                    }
                    s.abort = true;
                    return false;
                }
                std::this_thread::yield();
            }
        }
    }
    return true;
}

void SignalPeers(Shared& s, int rank, int kind, int lane, uint32_t value, int call) {
    for (int p = 0; p < s.W; ++p) {
        if (p == rank) continue;
        if (s.cfg.fault == 2 && rank == s.cfg.fault_rank && call == s.cfg.fault_call) {
            std::lock_guard<std::mutex> l(s.drop_m);
            if (s.dropped == 0) {
                s.dropped = 1;
                continue;  // this publication is lost
            }
        }
        Flag(s, p, kind, lane, rank).store(value, std::memory_order_release);
        s.flag_writes.fetch_add(1, std::memory_order_relaxed);
    }
}

size_t SlotIndex(const Shared& s, int on_rank, int src, int lane, int slot, int which) {
    return ((static_cast<size_t>(lane) * (s.W - 1) + yali::SrcSlot(src, on_rank)) * yali::kRingCap + slot) * 2 + which;
}

void ProducerStamp(Shared& s, int on_rank, size_t idx, uint64_t stamp) {
    uint64_t expect = 0;
    if (!s.ring_stamp[on_rank][idx].compare_exchange_strong(expect, stamp)) s.violations.fetch_add(1);
}
void ConsumerCheck(Shared& s, int on_rank, size_t idx, uint64_t stamp) {
    uint64_t expect = stamp;
    if (!s.ring_stamp[on_rank][idx].compare_exchange_strong(expect, 0)) s.violations.fetch_add(1);
}

void StreamLane(Shared& s, int r, int lane) {
    const YaliSimConfig& c = s.cfg;
    const int W = s.W;
    const uint64_t shard = yali::ShardElems(c.count, W);
    const uint64_t piece = c.slot_elems;
    uint32_t seq_base = 0;
    const uint64_t n_pieces = (shard + piece - 1) / piece;
    const uint32_t max_iters = static_cast<uint32_t>((n_pieces + s.L - 1) / s.L);
    for (int call = 0; call < c.calls; ++call) {
        if (c.fault == 1 && r == c.fault_rank && call >= c.fault_call) return;  // this rank never launches
        const uint32_t n_it = yali::oracle::StreamIters(shard, piece, s.L, lane);
        const float* send = s.send[r].data();
        float* recv = s.recv[r].data();
        bool ok = true;
        for (uint32_t step = 0; ok && step < n_it + 2; ++step) {
            if (step < n_it) {  // stage A
                const uint32_t i = step, slot = i % yali::kRingCap;
                if (i >= yali::kRingCap) ok = WaitPeers(s, r, kCr, lane, seq_base + (i - yali::kRingCap) + 1, 2);
                if (!ok) break;
                for (int k = 1; k < W; ++k) {
                    const int p = (r + k) % W;
                    uint64_t eb, ee;
                    yali::oracle::StreamPiece(c.count, shard, piece, s.L, lane, i, p, &eb, &ee);
                    const size_t idx = SlotIndex(s, p, r, lane, slot, 0);
                    ProducerStamp(s, p, idx, (static_cast<uint64_t>(call + 1) << 32) | (i + 1));
                    std::memcpy(&s.ring[p][idx * piece], send + eb, (ee - eb) * sizeof(float));
                }
                SignalPeers(s, r, kRs, lane, seq_base + i + 1, call);
            }
            if (step >= 1 && step - 1 < n_it) {  // stage B
                const uint32_t i = step - 1, slot = i % yali::kRingCap;
                ok = WaitPeers(s, r, kRs, lane, seq_base + i + 1, 3);
                if (!ok) break;
                uint64_t eb, ee;
                yali::oracle::StreamPiece(c.count, shard, piece, s.L, lane, i, r, &eb, &ee);
                std::vector<float> red(ee - eb);
                for (uint64_t e = 0; e < ee - eb; ++e) {
                    float acc = 0.f;
                    for (int q = 0; q < W; ++q)
                        acc += (q == r) ? send[eb + e] : s.ring[r][SlotIndex(s, r, q, lane, slot, 0) * piece + e];
                    red[e] = acc;
                }
                for (int q = 0; q < W; ++q)
                    if (q != r)
                        ConsumerCheck(s, r, SlotIndex(s, r, q, lane, slot, 0),
                                      (static_cast<uint64_t>(call + 1) << 32) | (i + 1));
                std::memcpy(recv + eb, red.data(), red.size() * sizeof(float));
                for (int k = 1; k < W; ++k) {
                    const int p = (r + k) % W;
                    if (c.direct_ag) {
                        std::memcpy(s.recv[p].data() + eb, red.data(), red.size() * sizeof(float));
                    } else {
                        const size_t idx = SlotIndex(s, p, r, lane, slot, 1);
                        ProducerStamp(s, p, idx, (static_cast<uint64_t>(call + 1) << 32) | (i + 1));
                        std::memcpy(&s.ring[p][idx * piece], red.data(), red.size() * sizeof(float));
                    }
                }
                SignalPeers(s, r, kAg, lane, seq_base + i + 1, call);
                if (c.direct_ag) SignalPeers(s, r, kCr, lane, seq_base + i + 1, call);
            }
            if (!c.direct_ag && step >= 2 && step - 2 < n_it) {  // stage C
                const uint32_t i = step - 2, slot = i % yali::kRingCap;
                ok = WaitPeers(s, r, kAg, lane, seq_base + i + 1, 4);
                if (!ok) break;
                for (int k = 1; k < W; ++k) {
                    const int q = (r + k) % W;
                    uint64_t eb, ee;
                    yali::oracle::StreamPiece(c.count, shard, piece, s.L, lane, i, q, &eb, &ee);
                    const size_t idx = SlotIndex(s, r, q, lane, slot, 1);
                    std::memcpy(recv + eb, &s.ring[r][idx * piece], (ee - eb) * sizeof(float));
                    ConsumerCheck(s, r, idx, (static_cast<uint64_t>(call + 1) << 32) | (i + 1));
                }
                SignalPeers(s, r, kCr, lane, seq_base + i + 1, call);
            }
        }
        if (ok && c.direct_ag && n_it > 0) ok = WaitPeers(s, r, kAg, lane, seq_base + n_it, 5);
        if (!ok) {
            s.abort = true;
        }
        seq_base += max_iters;
        // Stream order: the next kernel of this rank starts when all CTAs of this one are done.
        if (s.abort.load()) s.rank_abort[r].store(1);
        s.rank_barrier[r]->wait();
        if (s.rank_abort[r].load()) return;
    }
}

void FlashCta(Shared& s, int r, int cta) {
    const YaliSimConfig& c = s.cfg;
    const int W = s.W;
    for (int call = 0; call < c.calls; ++call) {
        if (c.fault == 1 && r == c.fault_rank && call >= c.fault_call) return;
        const uint32_t epoch = call + 1, parity = epoch & 1u;
        uint64_t vb, ve, tb, te;
        yali::oracle::FlashSlice(c.count, 4, s.L, cta, true, &vb, &ve, &tb, &te);
        const uint64_t eb = vb * 4, ee = (cta == s.L - 1) ? c.count : ve * 4;
        const float* send = s.send[r].data();
        for (int k = 1; k < W; ++k) {
            const int p = (r + k) % W;
            const size_t sidx = (static_cast<size_t>(parity) * (W - 1) + yali::SrcSlot(r, p));
            uint64_t expect = 0;
            if (!s.stage_stamp[p][sidx * s.L + cta].compare_exchange_strong(expect, epoch)) s.violations.fetch_add(1);
            std::memcpy(&s.stage[p][sidx * c.count + eb], send + eb, (ee - eb) * sizeof(float));
        }
        SignalPeers(s, r, kFlash, cta, epoch, call);
        bool ok = WaitPeers(s, r, kFlash, cta, epoch, 1);
        if (ok) {
            float* recv = s.recv[r].data();
            for (uint64_t e = eb; e < ee; ++e) {
                float acc = 0.f;
                for (int q = 0; q < W; ++q) {
                    if (q == r) acc += send[e];
                    else acc += s.stage[r][(static_cast<size_t>(parity) * (W - 1) + yali::SrcSlot(q, r)) * c.count + e];
                }
                recv[e] = acc;
            }
            for (int q = 0; q < W; ++q) {
                if (q == r) continue;
                const size_t sidx = (static_cast<size_t>(parity) * (W - 1) + yali::SrcSlot(q, r));
                uint64_t expect = epoch;
                if (!s.stage_stamp[r][sidx * s.L + cta].compare_exchange_strong(expect, 0)) s.violations.fetch_add(1);
            }
        } else {
            s.abort = true;
        }
        if (s.abort.load()) s.rank_abort[r].store(1);
        s.rank_barrier[r]->wait();
        if (s.rank_abort[r].load()) return;
    }
}

// Flag-in-data form of the one-shot (small messages): no flags at all.  Every pushed word carries the
// call number beside the payload, and a reader polls the word itself until the number is the current
// call's.  Two staging parities; what keeps a writer two calls ahead from overwriting unread words is
// only that it cannot finish the call in between without this rank's data for it.
void FlashLLCta(Shared& s, int r, int cta) {
    const YaliSimConfig& c = s.cfg;
    const int W = s.W;
    for (int call = 0; call < c.calls; ++call) {
        if (c.fault == 1 && r == c.fault_rank && call >= c.fault_call) return;
        const uint32_t epoch = call + 1, parity = epoch & 1u;
        uint64_t vb, ve, tb, te;
        yali::oracle::FlashSlice(c.count, 4, s.L, cta, true, &vb, &ve, &tb, &te);
        const uint64_t eb = vb * 4, ee = (cta == s.L - 1) ? c.count : ve * 4;
        const float* send = s.send[r].data();
        for (int k = 1; k < W; ++k) {
            const int p = (r + k) % W;
            const size_t sidx = (static_cast<size_t>(parity) * (W - 1) + yali::SrcSlot(r, p));
            uint64_t expect = 0;
            if (!s.stage_stamp[p][sidx * s.L + cta].compare_exchange_strong(expect, epoch)) s.violations.fetch_add(1);
            const bool lose = c.fault == 2 && r == c.fault_rank && call == c.fault_call && k == 1 && cta == 0;
            for (uint64_t e = eb; e < ee; ++e) {
                if (lose && e == eb) continue;  // one pushed word never arrives
                uint32_t bits;
                std::memcpy(&bits, send + e, 4);
                s.ll[p][sidx * c.count + e].store((static_cast<uint64_t>(epoch) << 32) | bits, std::memory_order_release);
            }
            s.flag_writes.fetch_add(ee - eb, std::memory_order_relaxed);
        }
        bool ok = true;
        float* recv = s.recv[r].data();
        const auto deadline = Clock::now() + std::chrono::milliseconds(c.timeout_ms);
        for (uint64_t e = eb; e < ee && ok; ++e) {
            float acc = 0.f;
            for (int q = 0; q < W && ok; ++q) {
                if (q == r) {
                    acc += send[e];
                    continue;
                }
                std::atomic<uint64_t>& w = s.ll[r][(static_cast<size_t>(parity) * (W - 1) + yali::SrcSlot(q, r)) * c.count + e];
                uint64_t v;
                uint32_t spins = 0;
                while (static_cast<uint32_t>((v = w.load(std::memory_order_acquire)) >> 32) != epoch) {
                    if ((++spins & 255u) == 0) {
                        if (s.abort.load() || Clock::now() > deadline) {
                            if (s.timeouts.fetch_add(1) == 0) {
                                s.t_rank = r;
                                s.t_peer = q;
                                s.t_site = 3;
                            }
                            s.abort = true;
                            ok = false;
                            break;
                        }
                        std::this_thread::yield();
                    }
                }
                if (!ok) break;
                const uint32_t bits = static_cast<uint32_t>(v);
                float f;
                std::memcpy(&f, &bits, 4);
                acc += f;
            }
            if (ok) recv[e] = acc;
        }
        if (ok)
            for (int q = 0; q < W; ++q) {
                if (q == r) continue;
                const size_t sidx = (static_cast<size_t>(parity) * (W - 1) + yali::SrcSlot(q, r));
                uint64_t expect = epoch;
                if (!s.stage_stamp[r][sidx * s.L + cta].compare_exchange_strong(expect, 0)) s.violations.fetch_add(1);
            }
        if (s.abort.load()) s.rank_abort[r].store(1);
        s.rank_barrier[r]->wait();
        if (s.rank_abort[r].load()) return;
    }
}

// Two-shot through the switch on staged (non-symmetric) buffers: copy in, per-CTA barrier across the
// ranks, every rank sums its shard over all ranks' staging and writes the result back into EVERY rank's
// staging (multimem.ld_reduce / multimem.st), second barrier, copy out.  The staging half alternates per
// call.  Every staged element has a stamp: 2*call+1 = input, 2*call+2 = result, 0 = free.
void NvlsCta(Shared& s, int r, int cta) {
    const YaliSimConfig& c = s.cfg;
    const int W = s.W, C = s.L;
    const uint64_t S = ((c.count + W - 1) / W + 3) / 4 * 4;  // shard elements
    const uint64_t per = (S + C - 1) / C;
    auto slice = [&](int q, uint64_t* b, uint64_t* e) {
        *b = std::min<uint64_t>(c.count, q * S + std::min(S, cta * per));
        *e = std::max(*b, std::min<uint64_t>(c.count, q * S + std::min(S, cta * per + per)));
    };
    auto stamp_at = [&](int rank, uint32_t parity, uint64_t e) -> std::atomic<uint64_t>& {
        return s.ll[rank][static_cast<size_t>(parity) * c.count + e];
    };
    auto stage_at = [&](int rank, uint32_t parity, uint64_t e) -> float& {
        return s.stage[rank][static_cast<size_t>(parity) * c.count + e];
    };
    for (int call = 0; call < c.calls; ++call) {
        if (c.fault == 1 && r == c.fault_rank && call >= c.fault_call) return;
        const uint32_t epoch = 2u * call, parity = call & 1u;
        const uint64_t in_stamp = 2ull * call + 1, out_stamp = 2ull * call + 2;
        for (int q = 0; q < W; ++q) {  // copy in: slice `cta` of every shard
            uint64_t b, e;
            slice(q, &b, &e);
            for (uint64_t i = b; i < e; ++i) {
                uint64_t expect = 0;
                if (!stamp_at(r, parity, i).compare_exchange_strong(expect, in_stamp)) s.violations.fetch_add(1);
                stage_at(r, parity, i) = s.send[r][i];
            }
        }
        SignalPeers(s, r, kFlash, cta, epoch + 1, call);
        bool ok = WaitPeers(s, r, kFlash, cta, epoch + 1, 1);
        if (ok) {
            uint64_t b, e;
            slice(r, &b, &e);
            for (uint64_t i = b; i < e; ++i) {
                float acc = 0.f;
                for (int q = 0; q < W; ++q) {
                    if (stamp_at(q, parity, i).load(std::memory_order_acquire) != in_stamp) s.violations.fetch_add(1);
                    acc += stage_at(q, parity, i);
                }
                for (int q = 0; q < W; ++q) {
                    stage_at(q, parity, i) = acc;
                    stamp_at(q, parity, i).store(out_stamp, std::memory_order_release);
                }
            }
            // the second barrier uses the other flag word of the pair in the kernels; here a second kind
            for (int p = 0; p < W; ++p)
                if (p != r) Flag(s, p, kAg, cta, r).store(epoch + 2, std::memory_order_release);
            ok = WaitPeers(s, r, kAg, cta, epoch + 2, 2);
        }
        if (ok) {
            for (int q = 0; q < W; ++q) {  // copy out
                uint64_t b, e;
                slice(q, &b, &e);
                for (uint64_t i = b; i < e; ++i) {
                    uint64_t expect = out_stamp;
                    if (!stamp_at(r, parity, i).compare_exchange_strong(expect, 0)) s.violations.fetch_add(1);
                    s.recv[r][i] = stage_at(r, parity, i);
                }
            }
        } else {
            s.abort = true;
        }
        if (s.abort.load()) s.rank_abort[r].store(1);
        s.rank_barrier[r]->wait();
        if (s.rank_abort[r].load()) return;
    }
}

// Pipelined direct forms (direct_pipeline.cu).  mode 4, two-shot IN PLACE: buf[r] is rank r's input and
// output; CTA c of rank r sums chunk c, c+C, ... of shard r over all ranks' buffers and writes the sum into
// every rank's buffer.  mode 5, one-shot pull: CTA c of rank r sums chunk c, c+C, ... of the whole message
// over all ranks' inputs into its own output.  Two per-CTA barriers per call are the only synchronisation.
// Between calls every rank overwrites its input with the next call's data (what a user or the next kernel
// does), which is only safe if the second barrier really means "all peers are done with this rank's
// buffer".  Stamps per element: 2*call+1 = input of the call, 2*call+2 = result of the call (mode 4).
void DirectCta(Shared& s, int r, int cta) {
    const YaliSimConfig& c = s.cfg;
    const int W = s.W, C = s.L;
    const bool one_shot = c.mode == 5;
    const uint64_t S = ((c.count + W - 1) / W + 3) / 4 * 4;  // shard elements
    const uint64_t chunk = std::max<uint64_t>(4, c.slot_elems ? c.slot_elems : 64);
    const uint64_t range_b = one_shot ? 0 : std::min<uint64_t>(c.count, r * S);
    const uint64_t range_e = one_shot ? c.count : std::min<uint64_t>(c.count, range_b + S);
    auto stamp_at = [&](int rank, uint64_t e) -> std::atomic<uint64_t>& { return s.ll[rank][e]; };
    for (int call = 0; call < c.calls; ++call) {
        if (c.fault == 1 && r == c.fault_rank && call >= c.fault_call) return;
        const uint32_t epoch = 2u * call;
        const uint64_t in_stamp = 2ull * call + 1, out_stamp = 2ull * call + 2;
        SignalPeers(s, r, kFlash, cta, epoch + 1, call);
        bool ok = WaitPeers(s, r, kFlash, cta, epoch + 1, 1);
        if (ok) {
            for (uint64_t b = range_b + cta * chunk; b < range_e; b += static_cast<uint64_t>(C) * chunk) {
                const uint64_t e = std::min(range_e, b + chunk);
                for (uint64_t i = b; i < e; ++i) {
                    float acc = 0.f;
                    for (int q = 0; q < W; ++q) {  // the bulk copies of the stage: every rank's input
                        if (stamp_at(q, i).load(std::memory_order_acquire) != in_stamp) s.violations.fetch_add(1);
                        acc += s.send[q][i];
                    }
                    if (one_shot) {
                        s.recv[r][i] = acc;
                    } else {
                        for (int q = 0; q < W; ++q) {
                            s.send[q][i] = acc;  // in place: input and output are one buffer
                            stamp_at(q, i).store(out_stamp, std::memory_order_release);
                        }
                    }
                }
            }
            for (int p = 0; p < W; ++p)
                if (p != r) Flag(s, p, kAg, cta, r).store(epoch + 2, std::memory_order_release);
            ok = WaitPeers(s, r, kAg, cta, epoch + 2, 2);
        }
        if (!ok) s.abort = true;
        if (s.abort.load()) s.rank_abort[r].store(1);
        s.rank_barrier[r]->wait();  // the kernel of this rank is complete
        if (s.rank_abort[r].load()) return;
        if (cta == 0) {
            // The stream's next operation on this rank: check the results and write the next call's input.
            const bool last = call + 1 == c.calls;
            for (uint64_t i = 0; i < c.count; ++i) {
                if (!one_shot) {
                    if (stamp_at(r, i).load(std::memory_order_acquire) != out_stamp) s.violations.fetch_add(1);
                    if (last) s.recv[r][i] = s.send[r][i];
                }
                if (!last) {
                    s.send[r][i] = yali::RandomValue(yali::kDistNormal, c.seed + r + 1000ull * (call + 1), i);
                    stamp_at(r, i).store(in_stamp + 2, std::memory_order_release);
                }
            }
        }
        s.rank_barrier[r]->wait();
    }
}

// Copy-engine path (comm/copy_engine_path.cc), IN PLACE.  Two threads per rank: lane 0 is the caller's
// stream (enter kernel, one reduce kernel per chunk, the outgoing copies of the two-shot form, exit
// kernel), lane 1 the stream of the incoming copies.  mode 6, one-shot: every rank copies every peer's
// whole buffer chunk by chunk into staging, announces each chunk as read, and overwrites its own chunk
// with the sum only after every peer has announced the same.  mode 7, two-shot: rank r copies shard r of
// every peer, writes the sums over its own shard and into every peer's shard r, then says "done".
// Flags on rank p written by src: kFlash = call src has entered, kAg = (call << 8) | chunks src has read
// on p, kRs = call src has finished with p.  Chunks are ordered between the two threads of a rank by the
// `copied` / `reduced` words (the events of the real path); `lanes` staging slots per source.
// direct_ag = 1 is the negative control of mode 6: no wait before overwriting, and rank 1 copies slowly.
// Stamps per element as in the pipelined forms: 2*call+1 = input of the call, 2*call+2 = its result.
struct CeRankState {
    std::unique_ptr<std::atomic<uint32_t>[]> copied, reduced;  // per chunk: call number when done
    std::vector<float> staging;                                // [W-1][slots][chunk]
};
std::vector<std::unique_ptr<CeRankState>> g_ce;  // set up by yali_c_simulate for modes 6 and 7

bool CeWaitWord(Shared& s, std::atomic<uint32_t>& w, uint32_t wanted, int rank, int peer, int site) {
    auto deadline = Clock::now() + std::chrono::milliseconds(s.cfg.timeout_ms);
    uint32_t spins = 0;
    while (!SeqReached(w.load(std::memory_order_acquire), wanted)) {
        if ((++spins & 255u) == 0) {
            if (s.abort.load() || Clock::now() > deadline) {
                // A wait between the two streams of one rank (events on the device) only passes the failure on:
                // the record names the cross-rank wait that caused it.
                if (peer != rank && s.timeouts.fetch_add(1) == 0) {
                    s.t_rank = rank;
                    s.t_peer = peer;
                    s.t_site = site;
                }
                if (peer != rank) s.abort = true;
                if (peer == rank && !s.abort.load()) {  // give the cross-rank waiter time to report first
                    std::this_thread::sleep_for(std::chrono::milliseconds(20));
                    s.abort = true;
                }
                return false;
            }
            std::this_thread::yield();
        }
    }
    return true;
}

void CopyEngineRank(Shared& s, int r, int lane) {
    const YaliSimConfig& c = s.cfg;
    const int W = s.W;
    const bool one_shot = c.mode == 6;
    constexpr uint32_t kSlots = 3;
    const uint64_t S = ((c.count + W - 1) / W + 3) / 4 * 4;  // shard elements
    const uint64_t chunk = std::max<uint64_t>(4, c.slot_elems ? c.slot_elems : 64);
    const uint64_t range_b = one_shot ? 0 : std::min<uint64_t>(c.count, r * S);
    const uint64_t range_e = one_shot ? c.count : std::min<uint64_t>(c.count, range_b + S);
    const uint32_t chunks = static_cast<uint32_t>((range_e - range_b + chunk - 1) / chunk);
    CeRankState& me = *g_ce[r];
    auto stamp_at = [&](int rank, uint64_t e) -> std::atomic<uint64_t>& { return s.ll[rank][e]; };
    auto slot_of = [&](int q, uint32_t ch) { return (static_cast<size_t>(yali::SrcSlot(q, r)) * kSlots + ch % kSlots) * chunk; };
    for (int call = 0; call < c.calls; ++call) {
        if (c.fault == 1 && r == c.fault_rank && call >= c.fault_call) return;
        const uint32_t number = static_cast<uint32_t>(call) + 1;
        const uint64_t in_stamp = 2ull * call + 1, out_stamp = 2ull * call + 2;
        bool ok = true;
        if (lane == 1) {
            // ---- the stream of the incoming copies
            for (int q = 0; q < W && ok; ++q)
                if (q != r) ok = CeWaitWord(s, Flag(s, r, kFlash, 0, q), number, r, q, 1);
            for (uint32_t ch = 0; ok && ch < chunks; ++ch) {
                if (ch >= kSlots) ok = CeWaitWord(s, me.reduced[ch - kSlots], number, r, r, 5);  // the slot is free again
                if (!ok) break;
                if (c.direct_ag == 1 && r == 1) std::this_thread::sleep_for(std::chrono::microseconds(300));
                const uint64_t b = range_b + ch * chunk, e = std::min(range_e, b + chunk);
                for (int q = 0; q < W; ++q) {
                    if (q == r) continue;
                    for (uint64_t i = b; i < e; ++i) {
                        // The peer's chunk must still hold this call's input: not yet its result, not the next input.
                        if (stamp_at(q, i).load(std::memory_order_acquire) != in_stamp) s.violations.fetch_add(1);
                        me.staging[slot_of(q, ch) + (i - b)] = s.send[q][i];
                    }
                }
                me.copied[ch].store(number, std::memory_order_release);
            }
        } else {
            // ---- the caller's stream
            SignalPeers(s, r, kFlash, 0, number, call);  // enter
            for (uint32_t ch = 0; ok && ch < chunks; ++ch) {
                ok = CeWaitWord(s, me.copied[ch], number, r, r, 4);
                if (!ok) break;
                const uint64_t b = range_b + ch * chunk, e = std::min(range_e, b + chunk);
                if (one_shot) {
                    const uint32_t word = (number << 8) | (ch + 1);
                    for (int p = 0; p < W; ++p)
                        if (p != r) {
                            Flag(s, p, kAg, 0, r).store(word, std::memory_order_release);  // chunk ch of p has been read
                            s.flag_writes.fetch_add(1, std::memory_order_relaxed);
                        }
                    if (c.direct_ag != 1)
                        for (int q = 0; q < W && ok; ++q)
                            if (q != r) ok = CeWaitWord(s, Flag(s, r, kAg, 0, q), word, r, q, 2);
                    if (!ok) break;
                }
                for (uint64_t i = b; i < e; ++i) {
                    float acc = 0.f;
                    for (int q = 0; q < W; ++q) {
                        if (q == r) {
                            if (stamp_at(r, i).load(std::memory_order_acquire) != in_stamp) s.violations.fetch_add(1);
                            acc += s.send[r][i];
                        } else {
                            acc += me.staging[slot_of(q, ch) + (i - b)];
                        }
                    }
                    s.send[r][i] = acc;  // in place
                    stamp_at(r, i).store(out_stamp, std::memory_order_release);
                    if (!one_shot) {
                        for (int q = 0; q < W; ++q) {  // the outgoing copies: shard r of every peer
                            if (q == r) continue;
                            if (stamp_at(q, i).load(std::memory_order_acquire) != in_stamp) s.violations.fetch_add(1);
                            s.send[q][i] = acc;
                            stamp_at(q, i).store(out_stamp, std::memory_order_release);
                        }
                    }
                }
                me.reduced[ch].store(number, std::memory_order_release);
            }
            if (ok && !one_shot) SignalPeers(s, r, kRs, 0, number, call);  // done
            // exit: every peer has read all of this rank's buffer (one-shot) or is done with this rank (two-shot)
            for (int q = 0; q < W && ok; ++q) {
                if (q == r) continue;
                // every rank cuts the same message into the same number of chunks in the one-shot form
                ok = one_shot ? CeWaitWord(s, Flag(s, r, kAg, 0, q), (number << 8) | chunks, r, q, 3)
                              : CeWaitWord(s, Flag(s, r, kRs, 0, q), number, r, q, 3);
            }
        }
        if (!ok) s.abort = true;
        if (s.abort.load()) s.rank_abort[r].store(1);
        s.rank_barrier[r]->wait();  // both streams of this rank are through the call
        if (s.rank_abort[r].load()) return;
        if (lane == 0) {
            const bool last = call + 1 == c.calls;
            for (uint64_t i = 0; i < c.count; ++i) {
                if (stamp_at(r, i).load(std::memory_order_acquire) != out_stamp) s.violations.fetch_add(1);
                if (last) s.recv[r][i] = s.send[r][i];
                if (!last) {
                    s.send[r][i] = yali::RandomValue(yali::kDistNormal, c.seed + r + 1000ull * (call + 1), i);
                    stamp_at(r, i).store(in_stamp + 2, std::memory_order_release);
                }
            }
        }
        s.rank_barrier[r]->wait();
    }
}

}  // namespace

extern "C" int yali_c_simulate(const YaliSimConfig* cfg, YaliSimReport* rep) {
    std::memset(rep, 0, sizeof(*rep));
    rep->timeout_rank = rep->timeout_peer = -1;
    if (!cfg || cfg->world < 2 || cfg->world > yali::kMaxRanks || cfg->lanes < 1 || cfg->lanes > 64 ||
        cfg->count == 0 || cfg->calls < 1 || (cfg->mode == 1 && (cfg->slot_elems == 0 || cfg->slot_elems % 4)))
        return -1;
    const bool ce = cfg->mode == 6 || cfg->mode == 7;
    if (ce && cfg->lanes != 2) return -1;  // the caller's stream and the stream of the incoming copies
    Shared s;
    s.cfg = *cfg;
    s.W = cfg->world;
    s.L = cfg->lanes;
    const int W = s.W;
    const size_t nflags = static_cast<size_t>(kKinds) * s.L * yali::kMaxRanks;
    const size_t nslots = static_cast<size_t>(s.L) * (W - 1) * yali::kRingCap * 2;
    for (int r = 0; r < W; ++r) {
        s.flags.emplace_back(new std::atomic<uint32_t>[nflags]);
        for (size_t i = 0; i < nflags; ++i) s.flags[r][i].store(0);
        s.send.emplace_back(cfg->count);
        s.recv.emplace_back(cfg->count, -12345.f);
        for (uint64_t i = 0; i < cfg->count; ++i)
            s.send[r][i] = yali::RandomValue(yali::kDistNormal, cfg->seed + r, i);
        if (cfg->mode == 1) {
            s.ring.emplace_back(nslots * cfg->slot_elems);
            s.ring_stamp.emplace_back(new std::atomic<uint64_t>[nslots]);
            for (size_t i = 0; i < nslots; ++i) s.ring_stamp[r][i].store(0);
        } else {
            if (cfg->mode == 4 || cfg->mode == 5 || ce) {
                s.ll.emplace_back(new std::atomic<uint64_t>[cfg->count]);
                for (size_t i = 0; i < cfg->count; ++i) s.ll[r][i].store(1);  // input of call 0
            } else if (cfg->mode == 2 || cfg->mode == 3) {
                const size_t nw = 2ull * std::max(W - 1, 1) * cfg->count;
                s.ll.emplace_back(new std::atomic<uint64_t>[nw]);
                for (size_t i = 0; i < nw; ++i) s.ll[r][i].store(0);
            }
            s.stage.emplace_back(2ull * (W - 1) * cfg->count);
            s.stage_stamp.emplace_back(new std::atomic<uint64_t>[2ull * (W - 1) * s.L]);
            for (size_t i = 0; i < 2ull * (W - 1) * s.L; ++i) s.stage_stamp[r][i].store(0);
        }
        s.rank_barrier.emplace_back(new Barrier(s.L));
    }
    s.rank_abort.reset(new std::atomic<int>[W]);
    for (int r = 0; r < W; ++r) s.rank_abort[r].store(0);
    g_ce.clear();
    if (ce) {
        const uint64_t chunk = std::max<uint64_t>(4, cfg->slot_elems ? cfg->slot_elems : 64);
        const size_t nchunks = static_cast<size_t>((cfg->count + chunk - 1) / chunk) + 1;
        for (int r = 0; r < W; ++r) {
            g_ce.emplace_back(new CeRankState());
            g_ce[r]->copied.reset(new std::atomic<uint32_t>[nchunks]);
            g_ce[r]->reduced.reset(new std::atomic<uint32_t>[nchunks]);
            for (size_t i = 0; i < nchunks; ++i) {
                g_ce[r]->copied[i].store(0);
                g_ce[r]->reduced[i].store(0);
            }
            g_ce[r]->staging.assign(static_cast<size_t>(W - 1) * 3 * chunk, 0.f);
        }
    }
    std::vector<std::thread> threads;
    for (int r = 0; r < W; ++r)
        for (int l = 0; l < s.L; ++l)
            threads.emplace_back(cfg->mode == 1   ? StreamLane
                                 : cfg->mode == 2 ? FlashLLCta
                                 : cfg->mode == 3 ? NvlsCta
                                 : (cfg->mode == 4 || cfg->mode == 5) ? DirectCta
                                 : ce                                 ? CopyEngineRank
                                                                      : FlashCta,
                                 std::ref(s), r, l);
    // A rank that stops launching leaves its lanes' barrier short-handed only for itself.
    for (auto& t : threads) t.join();

    rep->timeouts = s.timeouts.load();
    rep->flag_writes = s.flag_writes.load();
    rep->timeout_rank = s.t_rank.load();
    rep->timeout_peer = s.t_peer.load();
    rep->timeout_site = s.t_site.load();
    if (s.violations.load()) {
        rep->mismatches = s.violations.load();
        rep->status = 3;
        return 3;
    }
    if (rep->timeouts) {
        rep->status = 2;
        return 2;
    }
    // Oracle: fp64 sum; fp32 rank-order accumulation differs from it by rounding only.
    uint64_t bad = 0;
    const bool direct = cfg->mode == 4 || cfg->mode == 5 || ce;
    for (int r = 0; r < W; ++r) {
        for (uint64_t i = 0; i < cfg->count; ++i) {
            double e = 0.0;
            for (int q = 0; q < W; ++q)  // the pipelined forms get fresh inputs every call: the last call's count
                e += direct ? yali::RandomValue(yali::kDistNormal, cfg->seed + q + 1000ull * (cfg->calls - 1), i) : s.send[q][i];
            if (!(std::fabs(s.recv[r][i] - e) <= 1e-5 * W + 1e-5 * std::fabs(e))) ++bad;
        }
    }
    rep->mismatches = bad;
    rep->status = bad ? 1 : 0;
    return rep->status;
}
