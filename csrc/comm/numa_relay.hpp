// CPU relay of the host-staged transport (numa_mode = "relay").
//
// Direct host-staged mode lets a GPU store straight into the destination's host segment, wherever
// that memory lives.  In relay mode a GPU only ever touches host memory placed next to itself: rank r
// writes what it would send to rank d into an *outbox* O(r->d) of its own (same layout as a segment),
// and CPU threads of rank r's process forward it into d's real segment S(d), then publish the same
// flags there.  The GPU kernels are unchanged -- only the pointer table differs -- and the hand-off
// between GPU and CPU uses the very flags of the protocol: the GPU's st.release.sys is the CPU's
// acquire load, the CPU's release store is the destination GPU's ld.acquire.sys.
//
// Parity: the reference's NumaRelay (csrc/comm/numa_relay.hpp:59-366: pinned worker threads per target NUMA
// domain that copy payload + metadata and republish descriptors, credit recycling, a drained epoch, page-placement
// query), re-expressed for the push protocol: a worker follows one or more flows (r->d) and per flow forwards, in
// this order, the abort flag, the counts message, staged rows channel by channel as their READY flags appear (in
// bounded-ring mode only into slots the destination has acknowledged), the acknowledgements this rank's GPU wrote
// for rows it received, the done/cdone hand-backs and the combine rows.
//
// Workers are grouped by the NUMA node of the destination GPU: `workers` threads per node, each pinned to that
// node's CPUs (or to `cpu_affinity` when given), so that a copy runs next to the memory it writes.
//
// Failure codes (reported through diagnostics() and, where possible, as the rank's abort flag):
//   101 a flow's READY sequence went backwards, 102 counts announce more rows than a channel can ever hold,
//   199 the relay was stopped while rows were still pending.
#pragma once

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include <pthread.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cstdio>
#include <map>

#include "../kernels/protocol.cuh"

namespace bep {

// What a relay is built from.  Plain data: the Python binding fills it from the options dictionary, the host model
// of the protocol (csrc/model/protocol_model.cpp) fills it directly and runs the relay under ThreadSanitizer.
struct RelayOptions {
    int num_ranks = 0, channels = 0, num_experts = 0, num_topk = 0, hidden = 0, num_max_tokens = 0, payload_slots = 0;
    bool enable_combine = false;
    int workers = 1;                    // threads per NUMA node that has destinations
    std::vector<int> cpu_affinity;      // allowed CPUs (empty: the CPUs of the destination's NUMA node)
    std::vector<int> target_numa_nodes; // NUMA node of every rank's GPU (empty: node 0 for all)
};

// Progress of one flow (this rank -> dest), as diagnostics() reports it.
struct RelayFlowState {
    int dest = 0, numa_node = 0, failure = 0, worker_cpu = -1;
    std::uint64_t rows_copied = 0, bytes_copied = 0, counts_epoch = 0, combine_rows_copied = 0, acks_forwarded = 0, credit_waits = 0,
                  drained_epoch = 0;
};

class NumaRelay {
   public:
    // outboxes[d] / targets[d]: host addresses of O(rank->d) and S(d); entries for d == rank are ignored.
    NumaRelay(const RelayOptions& options, const std::vector<std::int64_t>& outboxes, const std::vector<std::int64_t>& targets, int rank)
        : rank_(rank) {
        const int P = options.num_ranks;
        lay_ = make_segment_layout(P, options.channels, options.num_experts, options.num_topk, options.hidden, options.num_max_tokens,
                                   options.payload_slots, options.enable_combine);
        ring_mode_ = lay_.slots < lay_.slots_full;
        if (static_cast<int>(outboxes.size()) != P || static_cast<int>(targets.size()) != P)
            throw std::invalid_argument("one outbox and one target per rank");
        own_segment_ = reinterpret_cast<std::uint8_t*>(targets[rank]);
        if (ring_mode_ && own_segment_ == nullptr) throw std::invalid_argument("bounded rings need this rank's own segment (credit checks)");
        std::vector<int> nodes(P, 0);
        if (!options.target_numa_nodes.empty()) {
            nodes = options.target_numa_nodes;
            if (static_cast<int>(nodes.size()) != P) throw std::invalid_argument("one NUMA node per rank");
        }
        workers_ = std::max(1, options.workers);
        affinity_ = options.cpu_affinity;
        // Explicit CPUs are a restriction, not a wish: for every NUMA node that has destinations, the CPUs named, the
        // CPUs of that node (where the platform tells) and the CPUs this process may run on must have one in common.
        if (!affinity_.empty()) {
            for (int d = 0; d < P; ++d) {
                if (d == rank) continue;
                const int node = nodes[d] < 0 ? 0 : nodes[d];
                if (worker_cpus(node).empty())
                    throw std::invalid_argument("relay_cpu_affinity leaves no usable CPU for the workers of NUMA node " + std::to_string(node));
            }
        }
        for (int d = 0; d < P; ++d) {
            if (d == rank) continue;
            auto flow = std::make_unique<Flow>();
            flow->dest = d;
            flow->outbox = reinterpret_cast<std::uint8_t*>(outboxes[d]);
            flow->target = reinterpret_cast<std::uint8_t*>(targets[d]);
            flow->numa_node = nodes[d] < 0 ? 0 : nodes[d];
            flow->acks_seen.assign(ring_mode_ ? static_cast<std::size_t>(lay_.num_channels) * lay_.slots : 0, 0);
            flow->forwarded.assign(lay_.num_channels, 0);
            flow->expected.assign(lay_.num_channels, 0);
            flow->combine_epoch.assign(lay_.has_combine ? lay_.num_max_tokens : 0, 0);
            flows_.push_back(std::move(flow));
        }
    }

    ~NumaRelay() { stop(); }

    void start() {
        if (running_) return;
        stopping_.store(false);
        running_ = true;
        // `workers_` threads per NUMA node that has destinations; a thread serves every workers_-th flow of its node
        std::map<int, std::vector<std::size_t>> by_node;
        for (std::size_t i = 0; i < flows_.size(); ++i) by_node[flows_[i]->numa_node].push_back(i);
        int ordinal = 0;
        for (const auto& [node, members] : by_node) {
            const int count = std::min<int>(workers_, static_cast<int>(members.size()));
            for (int w = 0; w < count; ++w) {
                std::vector<std::size_t> mine;
                for (std::size_t k = w; k < members.size(); k += count) mine.push_back(members[k]);
                threads_.emplace_back([this, node, ordinal, mine] { run(node, ordinal, mine); });
                ++ordinal;
            }
        }
    }

    void stop() {
        if (!running_) return;
        stopping_.store(true);
        for (auto& t : threads_) t.join();
        threads_.clear();
        running_ = false;
        for (auto& flow : flows_)
            if (flow->rows_pending() && flow->failure == 0) flow->failure = 199;
    }

    void set_delay_ns(std::uint64_t ns) { delay_ns_.store(ns); }

    std::vector<RelayFlowState> flow_states() const {
        std::vector<RelayFlowState> states;
        for (const auto& flow : flows_) {
            RelayFlowState f;
            f.dest = flow->dest;
            f.numa_node = flow->numa_node;
            f.failure = flow->failure.load();
            f.worker_cpu = flow->worker_cpu.load();
            f.rows_copied = flow->rows_copied.load();
            f.bytes_copied = flow->bytes_copied.load();
            f.counts_epoch = flow->counts_epoch.load();
            f.combine_rows_copied = flow->combine_rows.load();
            f.acks_forwarded = flow->acks_forwarded.load();
            f.credit_waits = flow->credit_waits.load();
            f.drained_epoch = flow->drained_epoch.load();
            states.push_back(f);
        }
        return states;
    }
    int worker_count() const { return static_cast<int>(threads_.size()); }
    bool running() const { return running_; }
    bool ring_mode() const { return ring_mode_; }

   private:
    struct Flow {
        int dest = 0;
        std::uint8_t* outbox = nullptr;
        std::uint8_t* target = nullptr;
        int numa_node = 0;                         // of the destination GPU
        std::vector<std::uint64_t> acks_seen;      // ring mode: last acknowledgement forwarded per (channel, slot)
        std::atomic<std::uint64_t> acks_forwarded{0}, credit_waits{0}, drained_epoch{0};
        std::vector<int> forwarded, expected;      // per channel, for the current counts epoch
        std::vector<std::uint64_t> combine_epoch;  // per token: last combine epoch forwarded
        std::uint64_t last_done = 0, last_cdone = 0, last_abort = 0;
        std::atomic<std::uint64_t> counts_epoch{0}, rows_copied{0}, bytes_copied{0}, combine_rows{0};
        std::atomic<int> failure{0}, worker_cpu{-1};
        bool rows_pending() const {
            for (std::size_t c = 0; c < forwarded.size(); ++c)
                if (forwarded[c] < expected[c]) return true;
            return false;
        }
    };

    static std::uint64_t load_acquire(const std::uint8_t* p) {
        return __atomic_load_n(reinterpret_cast<const std::uint64_t*>(p), __ATOMIC_ACQUIRE);
    }
    static void store_release(std::uint8_t* p, std::uint64_t v) {
        __atomic_store_n(reinterpret_cast<std::uint64_t*>(p), v, __ATOMIC_RELEASE);
    }

    // CPUs of one NUMA node, from sysfs ("0-15,32-47"); empty when the platform does not say
    static std::vector<int> node_cpus(int node) {
        std::vector<int> cpus;
        char path[96];
        std::snprintf(path, sizeof(path), "/sys/devices/system/node/node%d/cpulist", node);
        std::FILE* f = std::fopen(path, "r");
        if (f == nullptr) return cpus;
        char text[4096] = {0};
        const std::size_t got = std::fread(text, 1, sizeof(text) - 1, f);
        std::fclose(f);
        text[got] = 0;
        const char* p = text;
        while (*p) {
            char* end = nullptr;
            const long lo = std::strtol(p, &end, 10);
            if (end == p) break;
            long hi = lo;
            p = end;
            if (*p == '-') {
                hi = std::strtol(p + 1, &end, 10);
                p = end;
            }
            for (long c = lo; c <= hi && c < CPU_SETSIZE; ++c) cpus.push_back(static_cast<int>(c));
            while (*p == ',' || *p == '\n' || *p == ' ') ++p;
        }
        return cpus;
    }

    // Can a thread of this process be pinned to this CPU?  Tried on a short-lived thread of its own, so that nobody's
    // affinity changes (the calling thread may itself be bound to a few CPUs, which says nothing about what is permitted).
    static bool cpu_permitted(int cpu) {
        if (cpu < 0 || cpu >= CPU_SETSIZE) return false;
        bool ok = false;
        std::thread([&ok, cpu] {
            cpu_set_t set;
            CPU_ZERO(&set);
            CPU_SET(cpu, &set);
            ok = pthread_setaffinity_np(pthread_self(), sizeof(set), &set) == 0;
        }).join();
        return ok;
    }

    // Where the workers of one NUMA node run.  With explicit CPUs (`cpu_affinity`): those of them that lie on the node
    // (where the platform names the node's CPUs) and that this process may use.  Without: the node's CPUs.
    std::vector<int> worker_cpus(int node) const {
        const std::vector<int> of_node = node_cpus(node);
        if (affinity_.empty()) return of_node;
        std::vector<int> cpus;
        for (int c : affinity_) {
            if (!of_node.empty() && std::find(of_node.begin(), of_node.end(), c) == of_node.end()) continue;
            if (cpu_permitted(c)) cpus.push_back(c);
        }
        return cpus;
    }

    // Pin the calling worker.  With explicit CPUs: to one of them, the workers taking turns.  Without: to the CPUs of
    // the destination's NUMA node as a set.  Best effort: a refused call leaves the thread where it is.
    void pin(int node, int ordinal) {
        const std::vector<int> cpus = worker_cpus(node);
        if (cpus.empty()) return;
        cpu_set_t set;
        CPU_ZERO(&set);
        if (!affinity_.empty()) {
            CPU_SET(cpus[static_cast<std::size_t>(ordinal) % cpus.size()], &set);
        } else {
            for (int c : cpus) CPU_SET(c, &set);
        }
        pthread_setaffinity_np(pthread_self(), sizeof(set), &set);
    }

    void run(int node, int ordinal, const std::vector<std::size_t>& mine) {
        pin(node, ordinal);
        const int cpu = sched_getcpu();
        unsigned idle = 0;
        while (!stopping_.load(std::memory_order_relaxed)) {
            bool progressed = false;
            for (std::size_t i : mine) {
                flows_[i]->worker_cpu.store(cpu);
                progressed |= progress(*flows_[i]);
            }
            if (progressed) {
                idle = 0;
            } else if (++idle > 2000) {
                std::this_thread::sleep_for(std::chrono::microseconds(20));
            }
        }
    }

    // One pass over one flow; true if anything moved.
    bool progress(Flow& f) {
        if (f.failure.load() != 0) return false;
        bool moved = false;
        const int me = rank_;
        const std::size_t flag = static_cast<std::size_t>(me) * kFlagStride;
        // 1. abort
        const std::uint64_t abort_value = load_acquire(f.outbox + lay_.abort_off + flag);
        if (abort_value != f.last_abort) {
            store_release(f.target + lay_.abort_off + flag, abort_value);
            f.last_abort = abort_value;
            moved = true;
        }
        // 2. counts message of a new epoch
        const std::uint64_t epoch = load_acquire(f.outbox + lay_.counts_flag_off + flag);
        if (epoch > f.counts_epoch.load()) {
            const std::size_t bytes = static_cast<std::size_t>(lay_.counts_stride) * 4;
            const std::size_t at = lay_.counts_off + static_cast<std::size_t>(me) * bytes;
            std::memcpy(f.target + at, f.outbox + at, bytes);
            const int* message = reinterpret_cast<const int*>(f.outbox + at);
            const int* chan = message + lay_.num_ranks + lay_.num_local_experts;
            for (int c = 0; c < lay_.num_channels; ++c) {
                if (chan[c] > lay_.slots_full) {
                    f.failure.store(102);
                    return true;
                }
                f.expected[c] = chan[c];
                f.forwarded[c] = 0;
            }
            store_release(f.target + lay_.counts_flag_off + flag, epoch);
            f.counts_epoch.store(epoch);
            moved = true;
        }
        // 3. staged rows, in channel order, as far as their READY flags have appeared
        const std::uint64_t current = f.counts_epoch.load();
        if (current != 0) {
            const std::uint64_t delay = delay_ns_.load(std::memory_order_relaxed);
            for (int c = 0; c < lay_.num_channels; ++c) {
                while (f.forwarded[c] < f.expected[c]) {
                    const int j = f.forwarded[c];
                    const std::size_t ring = (static_cast<std::size_t>(me) * lay_.num_channels + c) * lay_.slots + j % lay_.slots;
                    const std::uint64_t want = make_seq(current, static_cast<std::uint32_t>(j + 1));
                    const std::uint64_t seen = load_acquire(f.outbox + lay_.ready_off + ring * 8);
                    if (seen != want) {
                        if ((seen >> 32) > current) f.failure.store(101);
                        break;
                    }
                    if (ring_mode_ && j >= lay_.slots) {
                        // the destination's slot is free once its GPU has acknowledged row j - slots; that
                        // acknowledgement arrives in this rank's own segment (forwarded by the destination's relay)
                        const std::size_t credit = (static_cast<std::size_t>(f.dest) * lay_.num_channels + c) * lay_.slots + j % lay_.slots;
                        if (load_acquire(own_segment_ + lay_.ack_off + credit * 8) != make_seq(current, static_cast<std::uint32_t>(j - lay_.slots + 1))) {
                            f.credit_waits.fetch_add(1, std::memory_order_relaxed);
                            break;
                        }
                    }
                    if (delay) std::this_thread::sleep_for(std::chrono::nanoseconds(delay));
                    const std::size_t row = lay_.stage_off + ring * lay_.row_stride;
                    const std::size_t bytes = static_cast<std::size_t>(lay_.meta_off) + lay_.meta_bytes;
                    std::memcpy(f.target + row, f.outbox + row, bytes);
                    store_release(f.target + lay_.ready_off + ring * 8, want);
                    ++f.forwarded[c];
                    f.rows_copied.fetch_add(1, std::memory_order_relaxed);
                    f.bytes_copied.fetch_add(bytes, std::memory_order_relaxed);
                    moved = true;
                }
            }
            // everything the counts message of this epoch announced has been forwarded
            if (!f.rows_pending() && f.drained_epoch.load() != current) f.drained_epoch.store(current);
        }
        // 4. ring mode: acknowledgements this rank's GPU wrote (as a destination) for rows that came from f.dest
        if (ring_mode_) {
            const std::size_t base = static_cast<std::size_t>(me) * lay_.num_channels * lay_.slots;
            for (std::size_t i = 0; i < f.acks_seen.size(); ++i) {
                const std::uint64_t value = load_acquire(f.outbox + lay_.ack_off + (base + i) * 8);
                if (value != f.acks_seen[i]) {
                    store_release(f.target + lay_.ack_off + (base + i) * 8, value);
                    f.acks_seen[i] = value;
                    f.acks_forwarded.fetch_add(1, std::memory_order_relaxed);
                    moved = true;
                }
            }
        }
        {
        // 5. hand-backs
        const std::uint64_t done = load_acquire(f.outbox + lay_.done_off + flag);
        if (done != f.last_done) {
            store_release(f.target + lay_.done_off + flag, done);
            f.last_done = done;
            moved = true;
        }
        if (lay_.has_combine) {
            const std::uint64_t cdone = load_acquire(f.outbox + lay_.cdone_off + flag);
            if (cdone != f.last_cdone) {
                store_release(f.target + lay_.cdone_off + flag, cdone);
                f.last_cdone = cdone;
                moved = true;
            }
            // 6. combine rows: one flag per (this rank, token)
            const std::size_t flags = lay_.cready_off + static_cast<std::size_t>(me) * lay_.num_max_tokens * 8;
            const std::size_t rows = lay_.cstage_off + static_cast<std::size_t>(me) * lay_.num_max_tokens * lay_.crow_stride;
            for (int t = 0; t < lay_.num_max_tokens; ++t) {
                const std::uint64_t e = load_acquire(f.outbox + flags + static_cast<std::size_t>(t) * 8);
                if (e > f.combine_epoch[t]) {
                    const std::size_t at = rows + static_cast<std::size_t>(t) * lay_.crow_stride;
                    std::memcpy(f.target + at, f.outbox + at, static_cast<std::size_t>(lay_.hidden) * 2);
                    store_release(f.target + flags + static_cast<std::size_t>(t) * 8, e);
                    f.combine_epoch[t] = e;
                    f.combine_rows.fetch_add(1, std::memory_order_relaxed);
                    moved = true;
                }
            }
        }
        }
        return moved;
    }

    int rank_;
    bool ring_mode_ = false;
    std::uint8_t* own_segment_ = nullptr;
    SegmentLayout lay_{};
    int workers_ = 1;
    std::vector<int> affinity_;
    std::vector<std::unique_ptr<Flow>> flows_;
    std::vector<std::thread> threads_;
    std::atomic<bool> stopping_{false};
    std::atomic<std::uint64_t> delay_ns_{0};
    bool running_ = false;
};

// Which NUMA node holds each page of [address, address + bytes)?  node -> page count; -1 collects pages the kernel
// could not place (not yet touched, or the call is not permitted here).  Uses move_pages(2) in its query form
// (no node list): nothing is moved.
inline std::map<int, long> query_numa_pages(std::uintptr_t address, std::size_t bytes) {
    std::map<int, long> per_node;
    const long page = sysconf(_SC_PAGESIZE);
    if (bytes == 0 || page <= 0) return per_node;
    const std::uintptr_t first = address & ~static_cast<std::uintptr_t>(page - 1);
    const std::size_t count = (address + bytes - first + page - 1) / page;
    constexpr std::size_t kBatch = 4096;
    std::vector<void*> pages(kBatch);
    std::vector<int> status(kBatch);
    for (std::size_t done = 0; done < count; done += kBatch) {
        const std::size_t n = std::min(kBatch, count - done);
        for (std::size_t i = 0; i < n; ++i) pages[i] = reinterpret_cast<void*>(first + (done + i) * page);
        const long rc = syscall(SYS_move_pages, 0, static_cast<unsigned long>(n), pages.data(), nullptr, status.data(), 0);
        for (std::size_t i = 0; i < n; ++i) per_node[rc == 0 && status[i] >= 0 ? status[i] : -1] += 1;
    }
    return per_node;
}

}  // namespace bep
