// Host model of the dispatch data plane (and, with --combine 1, of the combine that follows it): ranks are threads, segments are plain memory, every flag is a
// std::atomic_ref on the same offsets the kernels use (SegmentLayout and make_seq come from the kernels' own
// header).  It exists for two reasons.  It is an executable statement of the protocol's rules -- single-writer
// epoch-valued flags, local polling, counts before rows, credit before a ring slot is reused, `done` before the next
// epoch's first remote write, bounded waits that end in an error code and an abort every peer sees -- that runs
// under ThreadSanitizer, which no GPU tool on hand can do for the kernels.  And failure scenarios that must not be
// staged on a shared GPU (a rank that never sends its counts, never returns credit, never hands its staging area
// back, writes a wrong sequence, never signals that its combine rows are out, never hands the landing area back) run
// here instead.
//
// Combine (--combine 1; with --relay 1 the one-kernel form instead, whose per-row flags the relay forwards: a flag per
// (expert rank, token) follows each landing row and the owner waits for the flags of the rows it reads), by default
// the form with a separate owner-side sum: the rank that received a token's row for epoch e
// writes one result row into the owner's landing area [rank][token], behind the reuse guard `cdone >= e - 1` of every
// owner; when all its rows are out it releases `csig = e` to every owner.  An owner acquires every peer's `csig`,
// reads the landing rows of the ranks each token went to, and releases `cdone = e` to every peer.
//
// Publication of a row, selectable so that the rule can be seen to matter:
//   release   payload by ordinary stores, flag by a release store (what `st.release.sys` is on the GPU);
//   fenced    payload by ordinary stores, a fence, then a relaxed flag store (the send warps' chain: completion
//             wait, `fence.acq_rel.sys`, `st.relaxed.sys`);
//   relaxed   payload, then a relaxed flag with nothing in between -- wrong, and ThreadSanitizer says so.
//
// With --relay 1 the ranks do not write into each other's segments: rank r writes what it would send to rank d into an
// outbox O(r->d) of its own, and the product's CPU relay (csrc/comm/numa_relay.hpp, the very class the host-staged
// transport runs) forwards it into d's segment.  The relay's threads then run under ThreadSanitizer together with the
// scripted ranks: counts, rows, bounded rings with credit, acknowledgements and hand-backs all pass through it.
//
// Build: g++ -std=c++20 -O1 -g -pthread [-fsanitize=thread] -I<csrc> -I<cuda include> protocol_model.cpp
// Output: one JSON object per rank on stdout; exit status 0 when every rank ended as the scenario expects
// (--expect CODE, default 0).
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#include "comm/numa_relay.hpp"
#include "kernels/protocol.cuh"

namespace {

using Clock = std::chrono::steady_clock;
using bep::SegmentLayout;

struct Options {
    int ranks = 4, channels = 2, tokens = 48, hidden = 64, slots = 2, epochs = 6;
    int timeout_ms = 2000;
    int delay_us = 0;            // random delays up to this long before publications and consumptions
    int withhold_counts = -1;    // this rank never sends its counts message
    int withhold_credit = -1;    // this rank never acknowledges rows (ring mode)
    int skip_done = -1;          // this rank never hands its staging area back
    int corrupt_sequence = -1;   // this rank writes a wrong sequence into its rows
    int combine = 0;             // 1: every epoch's dispatch is followed by its combine
    int withhold_signal = -1;    // this rank never signals that its combine rows are out
    int skip_combine_done = -1;  // this rank never hands the combine landing area back
    int relay = 0;               // 1: remote writes go into outboxes that the product's CPU relay forwards
    int expect = 0;              // error code every failing rank is expected to end with (0: nobody fails)
    std::string publish = "release";
    unsigned seed = 1;
};

struct Rank {
    std::vector<std::uint8_t> segment;
    std::atomic<int> error{0};    // first error of this rank (the sticky latch)
    std::atomic<int> context{0};
    long long rows_received = 0;
    long long rows_sent = 0;
    long long rows_combined = 0;  // landing rows this rank read as an owner
};

struct World {
    Options opt;
    SegmentLayout lay;
    std::vector<Rank> rank;
    std::vector<std::vector<std::uint8_t>> outbox;  // relay mode: [source * ranks + destination], laid out like a segment
    std::vector<std::unique_ptr<bep::NumaRelay>> relays;
};

// Where rank `me` writes what is meant for rank `d`: d's segment, or (relay mode) me's outbox for d.
std::vector<std::uint8_t>& remote(World& w, int me, int d) {
    return (w.opt.relay && d != me) ? w.outbox[static_cast<std::size_t>(me) * w.opt.ranks + d] : w.rank[d].segment;
}

std::atomic_ref<std::uint64_t> flag_at(std::vector<std::uint8_t>& seg, std::size_t off) {
    return std::atomic_ref<std::uint64_t>(*reinterpret_cast<std::uint64_t*>(seg.data() + off));
}

// destinations of token t of rank s in epoch e (bit d), deterministic; about half of the ranks, never empty
unsigned route_mask(const Options& o, int s, int t, int e) {
    std::uint32_t h = static_cast<std::uint32_t>(s) * 2654435761u ^ static_cast<std::uint32_t>(t) * 40503u ^ static_cast<std::uint32_t>(e) * 97u ^ o.seed;
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    unsigned mask = h & ((1u << o.ranks) - 1u);
    if (mask == 0) mask = 1u << (t % o.ranks);
    return mask;
}

std::uint16_t payload_word(int s, int t, int e, int col) {
    return static_cast<std::uint16_t>((s * 131 + t * 7 + e * 29 + col * 3) % 251);
}

void random_delay(const Options& o, std::uint32_t& state) {
    if (o.delay_us <= 0) return;
    state = state * 1664525u + 1013904223u;
    const int us = static_cast<int>((state >> 8) % static_cast<unsigned>(o.delay_us + 1));
    if (us > 0) std::this_thread::sleep_for(std::chrono::microseconds(us));
}

// First error of a rank: latched locally, then published to every peer (this rank is the only writer of its flag).
void fail(World& w, int me, int code, int context) {
    int expected = 0;
    if (w.rank[me].error.compare_exchange_strong(expected, code)) {
        w.rank[me].context.store(context);
        for (int p = 0; p < w.opt.ranks; ++p)
            flag_at(remote(w, me, p), w.lay.abort_off + static_cast<std::size_t>(me) * bep::kFlagStride).store(static_cast<std::uint64_t>(code), std::memory_order_release);
    }
}

// One probe of a bounded wait: true when the wait has to end (own failure, a peer's abort, the deadline).
bool give_up(World& w, int me, Clock::time_point deadline, int code, int context) {
    if (w.rank[me].error.load() != 0) return true;
    for (int p = 0; p < w.opt.ranks; ++p) {
        if (p == me) continue;
        const std::uint64_t a = flag_at(w.rank[me].segment, w.lay.abort_off + static_cast<std::size_t>(p) * bep::kFlagStride).load(std::memory_order_acquire);
        if (a != 0) {
            fail(w, me, bep::kErrPeerAbort, p);
            return true;
        }
    }
    if (Clock::now() > deadline) {
        fail(w, me, code, context);
        return true;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(20));  // (a probe of a bounded wait backs off, like the kernels' waits)
    return false;
}

// row index of token t among the tokens of (source s, channel c) that go to destination d: the plan's `slot`
struct Plan {
    std::vector<int> slot;          // [T][P], -1 when the token does not go there
    std::vector<int> chan_count;    // [C][P]
};

Plan make_plan(const Options& o, int s, int e) {
    Plan p;
    const int tc = (o.tokens + o.channels - 1) / o.channels;
    p.slot.assign(static_cast<std::size_t>(o.tokens) * o.ranks, -1);
    p.chan_count.assign(static_cast<std::size_t>(o.channels) * o.ranks, 0);
    for (int t = 0; t < o.tokens; ++t) {
        const int c = t / tc;
        const unsigned mask = route_mask(o, s, t, e);
        for (int d = 0; d < o.ranks; ++d)
            if (mask >> d & 1u) p.slot[static_cast<std::size_t>(t) * o.ranks + d] = p.chan_count[static_cast<std::size_t>(c) * o.ranks + d]++;
    }
    return p;
}

// Owner side of the combine of one epoch: every peer's rows have landed (its signal says so), then every token's rows
// are read from the ranks the token went to.  False when the rank has failed.
bool combine_owner(World& w, int me, int epoch) {
    const Options& o = w.opt;
    const SegmentLayout& lay = w.lay;
    // between the expert side's reuse guard (which a missing signal may be the consequence of) and the next epoch's
    // counts wait (which is the consequence of an owner stuck here)
    const auto deadline = Clock::now() + std::chrono::milliseconds(o.timeout_ms + o.timeout_ms / 16);
    if (!o.relay) {
        for (int r = 0; r < o.ranks; ++r) {
            auto sig = flag_at(w.rank[me].segment, lay.csig_off + static_cast<std::size_t>(r) * bep::kFlagStride);
            while (sig.load(std::memory_order_acquire) < static_cast<std::uint64_t>(epoch))
                if (give_up(w, me, deadline, bep::kErrFusedSignalWait, r)) return false;
        }
    }
    for (int t = 0; t < o.tokens; ++t) {
        const unsigned mask = route_mask(o, me, t, epoch);
        for (int r = 0; r < o.ranks; ++r) {
            if (!(mask >> r & 1u)) continue;
            if (o.relay) {
                // the one-kernel form of the combine, the one the relay forwards: a flag per (expert rank, token)
                auto ready = flag_at(w.rank[me].segment, lay.cready_off + (static_cast<std::size_t>(r) * o.tokens + t) * 8);
                while (ready.load(std::memory_order_acquire) < static_cast<std::uint64_t>(epoch))
                    if (give_up(w, me, deadline, bep::kErrRowWait, r)) return false;
            }
            const auto* row = reinterpret_cast<const std::uint16_t*>(w.rank[me].segment.data() + lay.cstage_off +
                                                                     (static_cast<std::size_t>(r) * o.tokens + t) * lay.crow_stride);
            for (int col = 0; col < o.hidden; ++col) {
                if (row[col] != static_cast<std::uint16_t>(payload_word(me, t, epoch, col) + r)) {
                    fail(w, me, 98, r);  // a landing row that is not what the expert's rank made of this token: never expected
                    return false;
                }
            }
            ++w.rank[me].rows_combined;
        }
    }
    if (me != o.skip_combine_done)
        for (int p = 0; p < o.ranks; ++p)
            flag_at(remote(w, me, p), lay.cdone_off + static_cast<std::size_t>(me) * bep::kFlagStride).store(static_cast<std::uint64_t>(epoch), std::memory_order_release);
    return true;
}

void sender(World& w, int me) {
    const Options& o = w.opt;
    const SegmentLayout& lay = w.lay;
    std::uint32_t rng = o.seed * 7919u + static_cast<unsigned>(me);
    const int tc = (o.tokens + o.channels - 1) / o.channels;
    for (int epoch = 1; epoch <= o.epochs && w.rank[me].error.load() == 0; ++epoch) {
        // Deadlines are staggered in the order in which an epoch's waits depend on one another -- reuse guard, counts,
        // rows and credit -- so that the wait that is closest to the cause names it (the kernel's receive warps get a
        // quarter of the timeout more than its control warp for the same reason).
        const auto guard_deadline = Clock::now() + std::chrono::milliseconds(o.timeout_ms);
        const auto deadline = guard_deadline + std::chrono::milliseconds(o.timeout_ms / 4);
        // reuse guard: every destination has finished reading the previous epoch out of its staging area
        for (int d = 0; d < o.ranks; ++d) {
            auto done = flag_at(w.rank[me].segment, lay.done_off + static_cast<std::size_t>(d) * bep::kFlagStride);
            while (done.load(std::memory_order_acquire) + 1 < static_cast<std::uint64_t>(epoch))
                if (give_up(w, me, guard_deadline, bep::kErrReuseGuardWait, d)) return;
        }
        const Plan plan = make_plan(o, me, epoch);
        // counts first: a destination learns how many rows to expect per channel before (or while) they arrive
        if (me != o.withhold_counts) {
            for (int d = 0; d < o.ranks; ++d) {
                int* msg = reinterpret_cast<int*>(remote(w, me, d).data() + lay.counts_off) + static_cast<std::size_t>(me) * lay.counts_stride;
                for (int c = 0; c < o.channels; ++c) msg[o.ranks + lay.num_local_experts + c] = plan.chan_count[static_cast<std::size_t>(c) * o.ranks + d];
                random_delay(o, rng);
                flag_at(remote(w, me, d), lay.counts_flag_off + static_cast<std::size_t>(me) * bep::kFlagStride).store(static_cast<std::uint64_t>(epoch), std::memory_order_release);
            }
        }
        for (int t = 0; t < o.tokens; ++t) {
            const int c = t / tc;
            const unsigned mask = route_mask(o, me, t, epoch);
            for (int d = 0; d < o.ranks; ++d) {
                if (!(mask >> d & 1u)) continue;
                const int j = plan.slot[static_cast<std::size_t>(t) * o.ranks + d];
                const std::size_t ring = (static_cast<std::size_t>(me) * o.channels + c) * lay.slots + static_cast<std::size_t>(j % lay.slots);
                if (j >= lay.slots) {
                    // credit: the destination has acknowledged the row that used this ring slot before
                    auto ack = flag_at(w.rank[me].segment, lay.ack_off + ((static_cast<std::size_t>(d) * o.channels + c) * lay.slots + static_cast<std::size_t>(j % lay.slots)) * 8);
                    const std::uint64_t want = bep::make_seq(static_cast<std::uint64_t>(epoch), static_cast<std::uint32_t>(j - lay.slots + 1));
                    while (ack.load(std::memory_order_acquire) != want)
                        if (give_up(w, me, deadline, bep::kErrCreditWait, d)) return;
                }
                std::uint8_t* row = remote(w, me, d).data() + lay.stage_off + ring * lay.row_stride;
                auto* payload = reinterpret_cast<std::uint16_t*>(row);
                for (int col = 0; col < o.hidden; ++col) payload[col] = payload_word(me, t, epoch, col);
                auto* meta = reinterpret_cast<std::uint32_t*>(row + lay.meta_off);
                meta[0] = static_cast<std::uint32_t>(t);
                meta[2] = static_cast<std::uint32_t>(epoch) + (me == o.corrupt_sequence ? 1u : 0u);
                meta[3] = static_cast<std::uint32_t>(t) + 1u;
                random_delay(o, rng);
                auto ready = flag_at(remote(w, me, d), lay.ready_off + ring * 8);
                const std::uint64_t value = bep::make_seq(static_cast<std::uint64_t>(epoch), static_cast<std::uint32_t>(j + 1));
                if (o.publish == "release") {
                    ready.store(value, std::memory_order_release);
                } else if (o.publish == "fenced") {
                    std::atomic_thread_fence(std::memory_order_acq_rel);
                    ready.store(value, std::memory_order_relaxed);
                } else {
                    ready.store(value, std::memory_order_relaxed);  // the broken chain
                }
                ++w.rank[me].rows_sent;
            }
        }
        if (o.combine && !combine_owner(w, me, epoch)) return;
    }
}

void receiver(World& w, int me) {
    const Options& o = w.opt;
    const SegmentLayout& lay = w.lay;
    std::uint32_t rng = o.seed * 104729u + static_cast<unsigned>(me);
    for (int epoch = 1; epoch <= o.epochs && w.rank[me].error.load() == 0; ++epoch) {
        const auto counts_deadline = Clock::now() + std::chrono::milliseconds(o.timeout_ms + o.timeout_ms / 8);
        const auto deadline = counts_deadline + std::chrono::milliseconds(o.timeout_ms / 4);  // rows: after the senders' credit waits
        std::vector<int> expected(static_cast<std::size_t>(o.ranks) * o.channels, 0);
        for (int s = 0; s < o.ranks; ++s) {
            auto flag = flag_at(w.rank[me].segment, lay.counts_flag_off + static_cast<std::size_t>(s) * bep::kFlagStride);
            while (flag.load(std::memory_order_acquire) != static_cast<std::uint64_t>(epoch))
                if (give_up(w, me, counts_deadline, bep::kErrCountsWait, s)) return;
            const int* msg = reinterpret_cast<const int*>(w.rank[me].segment.data() + lay.counts_off) + static_cast<std::size_t>(s) * lay.counts_stride;
            for (int c = 0; c < o.channels; ++c) expected[static_cast<std::size_t>(s) * o.channels + c] = msg[o.ranks + lay.num_local_experts + c];
        }
        // rows of every (source, channel) in row order; sources are visited round-robin like the receive warps do
        std::vector<int> next(static_cast<std::size_t>(o.ranks) * o.channels, 0);
        std::vector<std::pair<int, int>> received;  // (source, token) of every row, for the combine
        bool pending = true;
        while (pending) {
            pending = false;
            for (int s = 0; s < o.ranks; ++s) {
                for (int c = 0; c < o.channels; ++c) {
                    int& j = next[static_cast<std::size_t>(s) * o.channels + c];
                    if (j >= expected[static_cast<std::size_t>(s) * o.channels + c]) continue;
                    pending = true;
                    const std::size_t ring = (static_cast<std::size_t>(s) * o.channels + c) * lay.slots + static_cast<std::size_t>(j % lay.slots);
                    auto ready = flag_at(w.rank[me].segment, lay.ready_off + ring * 8);
                    if (ready.load(std::memory_order_acquire) != bep::make_seq(static_cast<std::uint64_t>(epoch), static_cast<std::uint32_t>(j + 1))) {
                        if (give_up(w, me, deadline, bep::kErrRowWait, s)) return;
                        continue;
                    }
                    random_delay(o, rng);
                    const std::uint8_t* row = w.rank[me].segment.data() + lay.stage_off + ring * lay.row_stride;
                    const auto* meta = reinterpret_cast<const std::uint32_t*>(row + lay.meta_off);
                    const int token = static_cast<int>(meta[0]);
                    if (meta[2] != static_cast<std::uint32_t>(epoch) || meta[3] != static_cast<std::uint32_t>(token) + 1u || token < 0 || token >= o.tokens) {
                        fail(w, me, bep::kErrSequence, s);
                        return;
                    }
                    const auto* payload = reinterpret_cast<const std::uint16_t*>(row);
                    for (int col = 0; col < o.hidden; ++col) {
                        if (payload[col] != payload_word(s, token, epoch, col)) {
                            fail(w, me, 99, s);  // a row that does not carry what its header says: never expected
                            return;
                        }
                    }
                    ++w.rank[me].rows_received;
                    if (o.combine) received.emplace_back(s, token);
                    if (lay.slots < lay.slots_full && me != o.withhold_credit) {
                        // credit back to the source (in the source's segment, written by this rank only)
                        auto ack = flag_at(remote(w, me, s), lay.ack_off + ((static_cast<std::size_t>(me) * o.channels + c) * lay.slots + static_cast<std::size_t>(j % lay.slots)) * 8);
                        ack.store(bep::make_seq(static_cast<std::uint64_t>(epoch), static_cast<std::uint32_t>(j + 1)), std::memory_order_release);
                    }
                    ++j;
                }
            }
        }
        // the staging area of this epoch has been read: hand it back to every source
        if (me != o.skip_done)
            for (int s = 0; s < o.ranks; ++s)
                flag_at(remote(w, me, s), lay.done_off + static_cast<std::size_t>(me) * bep::kFlagStride).store(static_cast<std::uint64_t>(epoch), std::memory_order_release);
        if (!o.combine) continue;
        // expert side of the combine.  Reuse guard: every owner has read the previous epoch out of its landing area
        const auto guard_deadline = Clock::now() + std::chrono::milliseconds(o.timeout_ms);
        for (int p = 0; p < o.ranks; ++p) {
            auto done = flag_at(w.rank[me].segment, lay.cdone_off + static_cast<std::size_t>(p) * bep::kFlagStride);
            while (done.load(std::memory_order_acquire) + 1 < static_cast<std::uint64_t>(epoch))
                if (give_up(w, me, guard_deadline, bep::kErrReuseGuardWait, p)) return;
        }
        for (const auto& [s, token] : received) {
            auto* row = reinterpret_cast<std::uint16_t*>(remote(w, me, s).data() + lay.cstage_off +
                                                         (static_cast<std::size_t>(me) * o.tokens + token) * lay.crow_stride);
            for (int col = 0; col < o.hidden; ++col) row[col] = static_cast<std::uint16_t>(payload_word(s, token, epoch, col) + me);
            random_delay(o, rng);
            if (o.relay && me != o.withhold_signal)  // per-row flag: the relay forwards the row, then the flag
                flag_at(remote(w, me, s), lay.cready_off + (static_cast<std::size_t>(me) * o.tokens + token) * 8).store(static_cast<std::uint64_t>(epoch), std::memory_order_release);
        }
        if (!o.relay && me != o.withhold_signal)
            for (int p = 0; p < o.ranks; ++p)
                flag_at(w.rank[p].segment, lay.csig_off + static_cast<std::size_t>(me) * bep::kFlagStride).store(static_cast<std::uint64_t>(epoch), std::memory_order_release);
    }
}

int to_int(const char* s) { return std::atoi(s); }

}  // namespace

int main(int argc, char** argv) {
    World w;
    Options& o = w.opt;
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string key = argv[i];
        const char* v = argv[i + 1];
        if (key == "--ranks") o.ranks = to_int(v);
        else if (key == "--channels") o.channels = to_int(v);
        else if (key == "--tokens") o.tokens = to_int(v);
        else if (key == "--hidden") o.hidden = to_int(v);
        else if (key == "--slots") o.slots = to_int(v);
        else if (key == "--epochs") o.epochs = to_int(v);
        else if (key == "--timeout-ms") o.timeout_ms = to_int(v);
        else if (key == "--delay-us") o.delay_us = to_int(v);
        else if (key == "--withhold-counts") o.withhold_counts = to_int(v);
        else if (key == "--withhold-credit") o.withhold_credit = to_int(v);
        else if (key == "--skip-done") o.skip_done = to_int(v);
        else if (key == "--corrupt-sequence") o.corrupt_sequence = to_int(v);
        else if (key == "--combine") o.combine = to_int(v);
        else if (key == "--withhold-signal") o.withhold_signal = to_int(v);
        else if (key == "--skip-combine-done") o.skip_combine_done = to_int(v);
        else if (key == "--relay") o.relay = to_int(v);
        else if (key == "--expect") o.expect = to_int(v);
        else if (key == "--publish") o.publish = v;
        else if (key == "--seed") o.seed = static_cast<unsigned>(to_int(v));
        else {
            std::fprintf(stderr, "unknown option %s\n", key.c_str());
            return 2;
        }
    }
    if (o.ranks < 1 || o.ranks > bep::kMaxRanks || o.channels < 1 || o.tokens < 1 || o.hidden < 8 || o.hidden % 8 != 0 ||
        (o.publish != "release" && o.publish != "fenced" && o.publish != "relaxed")) {
        std::fprintf(stderr, "bad arguments\n");
        return 2;
    }
    // experts only size the counts message here: one local expert per rank
    w.lay = bep::make_segment_layout(o.ranks, o.channels, o.ranks, 1, o.hidden, o.tokens, o.slots, o.combine != 0);
    w.rank = std::vector<Rank>(static_cast<std::size_t>(o.ranks));
    for (auto& r : w.rank) r.segment.assign(w.lay.size_bytes + 64, 0);
    if (o.relay) {
        w.outbox.assign(static_cast<std::size_t>(o.ranks) * o.ranks, std::vector<std::uint8_t>());
        for (int s = 0; s < o.ranks; ++s)
            for (int d = 0; d < o.ranks; ++d)
                if (s != d) w.outbox[static_cast<std::size_t>(s) * o.ranks + d].assign(w.lay.size_bytes + 64, 0);
        bep::RelayOptions ro;
        ro.num_ranks = o.ranks;
        ro.channels = o.channels;
        ro.num_experts = o.ranks;
        ro.num_topk = 1;
        ro.hidden = o.hidden;
        ro.num_max_tokens = o.tokens;
        ro.payload_slots = o.slots;
        ro.enable_combine = o.combine != 0;
        for (int r = 0; r < o.ranks; ++r) {
            std::vector<std::int64_t> outboxes, targets;
            for (int d = 0; d < o.ranks; ++d) {
                outboxes.push_back(d == r ? 0 : reinterpret_cast<std::int64_t>(w.outbox[static_cast<std::size_t>(r) * o.ranks + d].data()));
                targets.push_back(reinterpret_cast<std::int64_t>(w.rank[d].segment.data()));
            }
            w.relays.push_back(std::make_unique<bep::NumaRelay>(ro, outboxes, targets, r));
            w.relays.back()->start();
        }
    }
    std::vector<std::thread> threads;
    for (int r = 0; r < o.ranks; ++r) {
        threads.emplace_back(sender, std::ref(w), r);
        threads.emplace_back(receiver, std::ref(w), r);
    }
    for (auto& t : threads) t.join();
    long long relayed = 0;
    int relay_failures = 0;
    for (auto& relay : w.relays) {
        relay->stop();
        for (const bep::RelayFlowState& flow : relay->flow_states()) {
            relayed += static_cast<long long>(flow.rows_copied);
            // (199 = stopped with rows pending: what a relay reports when its ranks gave up in a failure scenario)
            if (flow.failure != 0 && flow.failure != 199) ++relay_failures;
        }
    }
    if (o.relay) std::printf("{\"relay_rows\": %lld, \"relay_failures\": %d}\n", relayed, relay_failures);
    bool as_expected = relay_failures == 0;
    int failed = 0;
    for (int r = 0; r < o.ranks; ++r) {
        const int code = w.rank[r].error.load();
        std::printf("{\"rank\": %d, \"error\": %d, \"context\": %d, \"rows_sent\": %lld, \"rows_received\": %lld, \"rows_combined\": %lld}\n", r, code,
                    w.rank[r].context.load(), w.rank[r].rows_sent, w.rank[r].rows_received, w.rank[r].rows_combined);
        if (code != 0) ++failed;
        // a scenario names the code of the rank that found the fault; the others may end with it, with "a peer
        // aborted", or -- if they were done before the fault mattered to them -- without an error
        if (o.expect == 0 ? code != 0 : (code != 0 && code != o.expect && code != bep::kErrPeerAbort)) as_expected = false;
    }
    if (o.expect != 0 && failed == 0) as_expected = false;
    return as_expected ? 0 : 1;
}
