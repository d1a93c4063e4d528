// Host-side thread model of the fused all-reduce protocols (gemm_sm100.cu): W threads play W ranks, each with a "heap"
// of 64-bit words, and run the same protocol steps with the same index arithmetic (csrc/cuda/comm_layout.h):
//
//   * two-hop packets   - hop 1: every piece to its owner as (data, tag) words; the owner sums in rank order;
//                         hop 2: the finished piece to every rank as (data, tag) words; everybody collects the tile.
//   * one-shot packets  - every partial to every rank, every rank sums everything in rank order.
//   * fence + flags     - plain data words, a release store of the step number into a flag, acquire loads on the other side.
//   * in-switch barrier - one "multicast" store of the step number into the same word of every rank, bounded local polling.
//
// What the model checks (built with -fsanitize=thread by tests/test_sanitizers.py, so a missing happens-before edge in
// the flag protocol is reported as a race): all ranks end with the same, correct sums for W = 2, 4, 8 over several
// steps and both staging buffers; a rank that skips a step makes the others run out of their bounded polls and report
// a time-out status instead of hanging; the step after that works again (tags and flags carry the step number, so
// nothing has to be reset).
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include "comm_layout.h"

using namespace ovb;

namespace {

constexpr int kStatusOk = 0, kStatusPeerTimeout = 2;

struct World {
    int W, tiles, pieces;                                   // pieces of 16 bytes per tile
    size_t stage_words, flags_words;
    std::vector<std::vector<std::atomic<uint64_t>>> stage;  // [rank][parity * stage_words + word]: packets are two 64-bit words per 8 data bytes
    std::vector<std::vector<std::atomic<int>>> flags;       // [rank][...]
    std::vector<std::vector<uint32_t>> plain;               // [rank]: plain (non-atomic) data area of the fence + flag protocol
    World(int w, int t, int p) : W(w), tiles(t), pieces(p) {
        stage_words = 2 * (size_t)W * tiles * pieces * (kPacketBytes / 8);
        flags_words = (size_t)tiles * kNvlsFlagStride + (size_t)tiles * (W + 1);
        for (int r = 0; r < W; ++r) {
            stage.emplace_back(2 * stage_words);
            flags.emplace_back(flags_words);
            plain.emplace_back((size_t)W * tiles * pieces * 4);
            for (auto& x : stage.back()) x.store(0, std::memory_order_relaxed);
            for (auto& x : flags.back()) x.store(0, std::memory_order_relaxed);
        }
    }
};

// A packet in the model: four 64-bit units (data word, tag), like the two 16-byte stores of the kernel.
inline void put_packet(std::atomic<uint64_t>* at, const uint32_t d[4], uint32_t tag) {
    for (int j = 0; j < 4; ++j) at[j].store(((uint64_t)tag << 32) | d[j], std::memory_order_relaxed);
}
inline bool get_packet(const std::atomic<uint64_t>* at, uint32_t tag, uint32_t d[4], int max_polls) {
    for (int poll = 0; poll < max_polls; ++poll) {
        bool ok = true;
        for (int j = 0; j < 4; ++j) {
            const uint64_t v = at[j].load(std::memory_order_relaxed);
            if ((uint32_t)(v >> 32) != tag) { ok = false; break; }
            d[j] = (uint32_t)v;
        }
        if (ok) return true;
        std::this_thread::yield();
    }
    return false;
}

// The "partial" of rank r for data word j of piece i of a tile in step s: small integers, so sums are exact.
inline uint32_t partial_word(int r, int step, int tile, int i, int j) { return (uint32_t)((r + 1) * 7 + step * 3 + tile * 5 + i + j) & 0xFFFF; }
inline uint32_t expected_word(int W, int step, int tile, int i, int j) {
    uint32_t s = 0;
    for (int r = 0; r < W; ++r) s += partial_word(r, step, tile, i, j);
    return s;
}

// ---- two-hop packets
int twohop(World& w, int rank, int step, int site, int max_polls, std::vector<uint32_t>& out) {
    const int W = w.W, share = w.pieces / W;
    const uint32_t tag = packet_tag(step, site);
    const size_t par = (size_t)(site & 1) * w.stage_words;
    for (int tile = 0; tile < w.tiles; ++tile) {
        for (int i = 0; i < w.pieces; ++i) {                               // hop 1
            const int owner = twohop_owner(i, share);
            if (owner == rank) continue;
            uint32_t d[4];
            for (int j = 0; j < 4; ++j) d[j] = partial_word(rank, step, tile, i, j);
            put_packet(&w.stage[owner][par + twohop_hop1_offset(rank, w.tiles, tile, share, i - owner * share) / 8], d, tag);
        }
    }
    for (int tile = 0; tile < w.tiles; ++tile) {
        for (int k = 0; k < share; ++k) {                                  // the owner reduces its share in rank order, hop 2
            const int i = rank * share + k;
            uint32_t sum[4] = {0, 0, 0, 0};
            for (int r = 0; r < W; ++r) {
                uint32_t d[4];
                if (r == rank) {
                    for (int j = 0; j < 4; ++j) d[j] = partial_word(rank, step, tile, i, j);
                } else if (!get_packet(&w.stage[rank][par + twohop_hop1_offset(r, w.tiles, tile, share, k) / 8], tag, d, max_polls)) {
                    return kStatusPeerTimeout;
                }
                for (int j = 0; j < 4; ++j) sum[j] += d[j];
            }
            for (int r = 0; r < W; ++r) put_packet(&w.stage[r][par + twohop_hop2_offset(w.tiles, w.pieces, tile, i) / 8], sum, tag);
        }
    }
    for (int tile = 0; tile < w.tiles; ++tile)
        for (int i = 0; i < w.pieces; ++i) {
            uint32_t d[4];
            if (!get_packet(&w.stage[rank][par + twohop_hop2_offset(w.tiles, w.pieces, tile, i) / 8], tag, d, max_polls)) return kStatusPeerTimeout;
            for (int j = 0; j < 4; ++j) out[((size_t)tile * w.pieces + i) * 4 + j] = d[j];
        }
    return kStatusOk;
}

// ---- one-shot packets
int oneshot(World& w, int rank, int step, int site, int max_polls, std::vector<uint32_t>& out) {
    const int W = w.W;
    const uint32_t tag = packet_tag(step, site);
    const size_t par = (size_t)(site & 1) * w.stage_words;
    for (int tile = 0; tile < w.tiles; ++tile)
        for (int i = 0; i < w.pieces; ++i) {
            uint32_t d[4];
            for (int j = 0; j < 4; ++j) d[j] = partial_word(rank, step, tile, i, j);
            for (int r = 0; r < W; ++r)
                if (r != rank) put_packet(&w.stage[r][par + (oneshot_slot_offset(rank, w.tiles, tile, w.pieces) + (size_t)i * kPacketBytes) / 8], d, tag);
        }
    for (int tile = 0; tile < w.tiles; ++tile)
        for (int i = 0; i < w.pieces; ++i) {
            uint32_t sum[4] = {0, 0, 0, 0};
            for (int r = 0; r < W; ++r) {
                uint32_t d[4];
                if (r == rank) {
                    for (int j = 0; j < 4; ++j) d[j] = partial_word(rank, step, tile, i, j);
                } else if (!get_packet(&w.stage[rank][par + (oneshot_slot_offset(r, w.tiles, tile, w.pieces) + (size_t)i * kPacketBytes) / 8], tag, d, max_polls)) {
                    return kStatusPeerTimeout;
                }
                for (int j = 0; j < 4; ++j) sum[j] += d[j];
            }
            for (int j = 0; j < 4; ++j) out[((size_t)tile * w.pieces + i) * 4 + j] = sum[j];
        }
    return kStatusOk;
}

// ---- plain data + release / acquire flags (one flag per tile and source rank, holding the step number)
int fence_flags(World& w, int rank, int step, int max_polls, std::vector<uint32_t>& out) {
    const int W = w.W;
    const size_t flag_base = (size_t)w.tiles * kNvlsFlagStride;
    for (int tile = 0; tile < w.tiles; ++tile) {
        for (int r = 0; r < W; ++r) {
            uint32_t* dst = &w.plain[r][(((size_t)rank * w.tiles + tile) * w.pieces) * 4];
            for (int i = 0; i < w.pieces; ++i)
                for (int j = 0; j < 4; ++j) dst[i * 4 + j] = partial_word(rank, step, tile, i, j);   // plain stores
        }
        for (int r = 0; r < W; ++r) w.flags[r][flag_base + (size_t)tile * (W + 1) + rank].store(step, std::memory_order_release);
    }
    for (int tile = 0; tile < w.tiles; ++tile) {
        for (int r = 0; r < W; ++r) {
            int poll = 0;
            while (w.flags[rank][flag_base + (size_t)tile * (W + 1) + r].load(std::memory_order_acquire) < step) {
                if (++poll > max_polls) return kStatusPeerTimeout;
                std::this_thread::yield();
            }
        }
        for (int i = 0; i < w.pieces; ++i)
            for (int j = 0; j < 4; ++j) {
                uint32_t s = 0;
                for (int r = 0; r < W; ++r) s += w.plain[rank][(((size_t)r * w.tiles + tile) * w.pieces + i) * 4 + j];
                out[((size_t)tile * w.pieces + i) * 4 + j] = s;
            }
    }
    return kStatusOk;
}

// ---- in-switch barrier: a "multicast" store of the step number, bounded polling of the local words
bool nvls_barrier(World& w, int rank, int tile, int phase, int step, int max_polls) {
    for (int r = 0; r < w.W; ++r) w.flags[r][nvls_barrier_word(tile, phase, rank)].store(step, std::memory_order_release);
    for (int poll = 0; poll < max_polls; ++poll) {
        bool all = true;
        for (int r = 0; r < w.W; ++r) all = all && w.flags[rank][nvls_barrier_word(tile, phase, r)].load(std::memory_order_acquire) >= step;
        if (all) return true;
        std::this_thread::yield();
    }
    return false;
}

struct Result { int status; bool correct; };

// Runs `steps` steps of one protocol on W threads; in step `skip_step` rank `skip_rank` stays away (-1: nobody).
bool run(const char* name, int protocol, int W, int steps, int skip_step, int skip_rank) {
    World w(W, /*tiles=*/3, /*pieces=*/16);
    std::vector<std::vector<Result>> res(W, std::vector<Result>(steps, Result{0, true}));
    // Steps are separated by a host-side barrier, the way a serving loop learns on the host that a rank has left a step:
    // the model is about what happens INSIDE a step.
    std::atomic<int> arrived{0};
    auto host_barrier = [&](int gen) {
        arrived.fetch_add(1, std::memory_order_acq_rel);
        while (arrived.load(std::memory_order_acquire) < gen * W) std::this_thread::yield();
    };
    std::vector<std::thread> th;
    for (int rank = 0; rank < W; ++rank)
        th.emplace_back([&, rank] {
            std::vector<uint32_t> out((size_t)w.tiles * w.pieces * 4);
            for (int s = 0; s < steps; ++s) {
                const int step = s + 1, site = s % 5;
                const bool away = (s == skip_step && rank == skip_rank);
                const int max_polls = (s == skip_step && skip_rank >= 0) ? 2000 : 50000000;
                int st = kStatusOk;
                if (!away) {
                    std::fill(out.begin(), out.end(), 0u);
                    if (protocol == 0) st = twohop(w, rank, step, site, max_polls, out);
                    else if (protocol == 1) st = oneshot(w, rank, step, site, max_polls, out);
                    else if (protocol == 2) st = fence_flags(w, rank, step, max_polls, out);
                    else {
                        for (int tile = 0; tile < w.tiles && st == kStatusOk; ++tile)
                            for (int phase = 0; phase < 2 && st == kStatusOk; ++phase)
                                if (!nvls_barrier(w, rank, tile, phase, step, max_polls)) st = kStatusPeerTimeout;
                    }
                    bool good = true;
                    if (st == kStatusOk && protocol < 3)
                        for (int tile = 0; tile < w.tiles; ++tile)
                            for (int i = 0; i < w.pieces; ++i)
                                for (int j = 0; j < 4; ++j)
                                    good = good && out[((size_t)tile * w.pieces + i) * 4 + j] == expected_word(W, step, tile, i, j);
                    res[rank][s] = Result{st, good};
                }
                host_barrier(s + 1);
            }
        });
    for (auto& t : th) t.join();
    bool ok = true;
    for (int rank = 0; rank < W; ++rank)
        for (int s = 0; s < steps; ++s) {
            const Result r = res[rank][s];
            if (s == skip_step && skip_rank >= 0) {
                // the rank that stayed away reports nothing; everybody else must have given up with the time-out status
                if (rank != skip_rank && r.status != kStatusPeerTimeout) { std::printf("%s W=%d: rank %d did not time out in step %d\n", name, W, rank, s); ok = false; }
            } else if (r.status != kStatusOk || !r.correct) {
                std::printf("%s W=%d: rank %d step %d status %d correct %d\n", name, W, rank, s, r.status, (int)r.correct);
                ok = false;
            }
        }
    return ok;
}

}  // namespace

int main() {
    const char* names[4] = {"two-hop packets", "one-shot packets", "fence + flags", "in-switch barrier"};
    bool ok = true;
    for (int protocol = 0; protocol < 4; ++protocol)
        for (int W : {2, 4, 8}) {
            ok = run(names[protocol], protocol, W, 6, -1, -1) && ok;          // everybody takes part
            ok = run(names[protocol], protocol, W, 6, 2, W - 1) && ok;        // the last rank skips step 2; steps 3.. work again
        }
    std::printf(ok ? "COMM_MODEL_OK\n" : "COMM_MODEL_FAILED\n");
    return ok ? 0 : 1;
}
