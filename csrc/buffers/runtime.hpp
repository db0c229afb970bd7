// Native runtime of one (virtual) EP rank: owns the device-resident rank constants, the result
// pools, the routing-plan pool and the launch logic (parity: the reference's AdvancedRuntime,
// csrc/buffers/advanced.hpp:43-550, for the peer-memory transport).
//
// Result pools: `output_pool_size` eager sets
// plus one graph set are allocated up front.  A set is busy while any of its tensors -- or a view of
// one -- is still referenced from Python; when every set is busy, dispatch fails with "pool exhausted"
// instead of waiting or allocating.  Routing plans come from a pool of the same size (+1 for graphs).
#pragma once

#include <cstdint>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../comm/peer_memory.hpp"
#include "../kernels/expert_gemm.hpp"
#include "../kernels/launch.hpp"

namespace bep {

namespace py = pybind11;

// True when nothing outside this runtime can still reach the tensor's memory.  Pool tensors are never
// handed out themselves: Python only ever receives aliases (distinct tensor objects sharing the
// storage), so "some result tensor or a view of it is alive" is exactly "the storage has another
// owner".  This needs nothing of PyTorch's Python-object bookkeeping.
inline bool tensor_unowned(const at::Tensor& t) {
    if (!t.defined()) return true;
    return t.use_count() == 1 && t.unsafeGetTensorImpl()->unsafe_storage().use_count() == 1;
}

struct TensorRefs {
    std::int64_t tensor_use_count, storage_use_count;
};
inline TensorRefs tensor_refs(const at::Tensor& t) {
    return {static_cast<std::int64_t>(t.use_count()),
            static_cast<std::int64_t>(t.unsafeGetTensorImpl()->unsafe_storage().use_count())};
}

struct RuntimeOptions {
    int channels = 32;
    int payload_slots = 0;
    int timeout_ms = 30000;
    bool wire_fp8 = false;
    bool recv_fp8 = false;
    bool use_tma = true;
    bool host_segments = false;  // the segments are registered host memory (transport "host_staged")
    bool force_scalar = false;  // ablation: 2-byte register copies even where 16-byte accesses would be legal
    int tx_warps = 2;
    int rx_warps = 8;
    int send_stages = 3;
    int send_ctas = -1;  // dedicated sender CTAs; -1: by channel count with more than one rank, none with one
    int output_pool_size = 3;
    bool enable_graph = false;
    bool enable_combine = true;
    bool enable_fused = false;
    std::string combine_reduce = "auto";  // owner-side sum of combine: "separate" launch, "inline", or "auto" by rank count
    std::uint64_t delay_meta_ns = 0, delay_tx_ns = 0, delay_rx_ns = 0, delay_scatter_ns = 0;

    static RuntimeOptions parse(const py::dict& d) {
        RuntimeOptions o;
        auto get = [&d](const char* key, auto fallback) {
            using T = decltype(fallback);
            return d.contains(key) ? d[key].cast<T>() : fallback;
        };
        o.channels = get("channels", o.channels);
        o.payload_slots = get("payload_slots", o.payload_slots);
        o.timeout_ms = get("timeout_ms", o.timeout_ms);
        o.wire_fp8 = get("wire_dtype", std::string("bf16")) == "fp8_e4m3";
        o.recv_fp8 = get("recv_dtype", std::string("bf16")) == "fp8_e4m3";
        if (o.recv_fp8 && !o.wire_fp8) throw std::invalid_argument("recv_dtype fp8_e4m3 needs wire_dtype fp8_e4m3");
        o.use_tma = get("copy_engine", std::string("tma")) == "tma";
        o.force_scalar = get("force_scalar", false);
        o.host_segments = get("segment_kind", std::string("peer")) == "host_staged";
        o.tx_warps = get("tx_warps", o.tx_warps);
        o.rx_warps = get("rx_warps", o.rx_warps);
        o.send_stages = get("pipeline_stages", o.send_stages);
        o.send_ctas = get("send_ctas", o.send_ctas);
        o.output_pool_size = get("output_pool_size", o.output_pool_size);
        o.enable_graph = get("enable_graph", o.enable_graph);
        o.enable_combine = get("enable_combine", o.enable_combine);
        o.enable_fused = get("fused_expert_combine", o.enable_fused);
        o.combine_reduce = get("combine_reduce", std::string("auto"));
        o.delay_meta_ns = get("metadata_delay_ns", std::uint64_t{0});
        o.delay_tx_ns = get("tx_delay_ns", std::uint64_t{0});
        o.delay_rx_ns = get("rx_delay_ns", std::uint64_t{0});
        o.delay_scatter_ns = get("scatter_delay_ns", std::uint64_t{0});
        if (o.channels < 1 || o.channels > kMaxChannels) throw std::invalid_argument("channels out of range");
        if (o.tx_warps < 1 || o.rx_warps < 1 || 1 + o.tx_warps + o.rx_warps > kMaxWarps)
            throw std::invalid_argument("1 + tx_warps + rx_warps must not exceed 16");
        if (o.send_ctas < -1 || o.send_ctas > 64) throw std::invalid_argument("send_ctas must be -1 (automatic) or in [0,64]");
        if (o.send_stages < 2 || o.send_stages > kMaxSendStages) throw std::invalid_argument("pipeline_stages must be 2, 3 or 4");
        if (o.output_pool_size < 2 || o.output_pool_size > 8) throw std::invalid_argument("output_pool_size must be in [2,8]");
        if (o.timeout_ms < 1) throw std::invalid_argument("timeout_ms must be positive");
        return o;
    }
};

// One routing plan: what the layout phase computed for one topk_idx, reusable while the routing
// tensor is unchanged.
struct Layout {
    at::Tensor mask, slot, expert_ord, counts;
    int num_tokens = -1;
    int alignment = 0;
    bool expand = false;
    bool valid = false;  // filled by a completed (enqueued) dispatch
};

struct OutputSet {
    at::Tensor recv_x, recv_idx, recv_w, recv_scale, source_meta, comb_map, recv_chan_counts;
    at::Tensor unique_count, expanded_count, expert_counts, expert_offsets, expert_prefix, source_offsets;
    at::Tensor source_expert_prefix, error, stats, timestamps, prefix_tx_ts;
    at::Tensor combine_error, combine_stats, profile, combine_profile, role_profile;

    std::vector<const at::Tensor*> all() const {
        return {&recv_x, &recv_idx, &recv_w, &recv_scale, &source_meta, &comb_map, &recv_chan_counts, &unique_count,
                &expanded_count, &expert_counts, &expert_offsets, &expert_prefix, &source_offsets,
                &source_expert_prefix, &error, &stats, &timestamps, &prefix_tx_ts, &combine_error, &combine_stats, &profile, &combine_profile,
                &role_profile};
    }
    bool free() const {
        for (const at::Tensor* t : all())
            if (!tensor_unowned(*t)) return false;
        return true;
    }
};

// What dispatch returns to Python: a dict-like lease on one result pool.  Tensors are created on
// first access (as aliases of the pool's tensors, never the pool tensors themselves) and cached, so a
// dispatch costs no per-field work on the CPU.  The pool is busy while this object, or any tensor it
// handed out, or a view of one, is alive.
class DispatchResult {
   public:
    DispatchResult(std::shared_ptr<OutputSet> set, std::shared_ptr<Layout> layout, bool expand, int num_tokens,
                   int unique_cap, int expanded_cap, int topk, bool recv_fp8 = false)
        : set_(std::move(set)), layout_(std::move(layout)), expand_(expand), num_tokens_(num_tokens),
          unique_cap_(unique_cap), expanded_cap_(expanded_cap), topk_(topk), recv_fp8_(recv_fp8) {}

    static const std::vector<std::string>& tensor_keys() {
        static const std::vector<std::string> keys = {
            "recv_x", "recv_topk_idx", "recv_topk_weights", "source_meta", "comb_map", "recv_chan_counts",
            "unique_count", "expanded_count", "expert_counts", "expert_offsets", "expert_prefix", "source_offsets",
            "source_expert_prefix", "error", "stats", "transport_timestamps_ns", "prefix_tx_timestamps_ns",
            "combine_error", "combine_stats", "profiling", "combine_profiling", "recv_x_scales", "role_profiling"};
        return keys;
    }

    bool contains(const std::string& key) const {
        if (overrides_.contains(key.c_str())) return true;
        if (key == "_layout" || key == "_expand" || key == "_num_tokens") return true;
        for (const auto& k : tensor_keys())
            if (k == key) return true;
        return false;
    }

    py::object get(const std::string& key) {
        if (overrides_.contains(key.c_str())) return overrides_[key.c_str()];
        if (key == "_layout") return py::cast(layout_);
        if (key == "_expand") return py::cast(expand_);
        if (key == "_num_tokens") return py::cast(num_tokens_);
        auto hit = cache_.find(key);
        if (hit != cache_.end()) return py::cast(hit->second);
        at::Tensor t = make(key);
        cache_.emplace(key, t);
        return py::cast(t);
    }
    void set(const std::string& key, py::object value) { overrides_[key.c_str()] = std::move(value); }
    py::list keys() const {
        py::list out;
        for (const auto& k : tensor_keys()) out.append(k);
        out.append("_layout");
        out.append("_expand");
        out.append("_num_tokens");
        return out;
    }

    const OutputSet& set_ref() const { return *set_; }
    const std::shared_ptr<Layout>& layout() const { return layout_; }
    bool expand() const { return expand_; }
    int num_tokens() const { return num_tokens_; }

   private:
    at::Tensor make(const std::string& key) const {
        const OutputSet& s = *set_;
        const std::int64_t K = topk_;
        if (key == "recv_x") {
            const std::int64_t cap = expand_ ? expanded_cap_ : unique_cap_;
            if (!recv_fp8_) return s.recv_x.narrow(0, 0, cap);
            // E4M3 rows occupy the first half of the BF16-sized pool tensor, one byte per element
            const std::int64_t hidden = s.recv_x.size(1);
            return s.recv_x.view(at::kByte).reshape({-1}).narrow(0, 0, cap * hidden).view({cap, hidden}).view(at::kFloat8_e4m3fn);
        }
        if (key == "recv_x_scales") return recv_fp8_ ? s.recv_scale.narrow(0, 0, expand_ ? expanded_cap_ : unique_cap_) : at::alias(s.recv_scale);
        if (key == "source_meta") return s.source_meta.narrow(0, 0, expand_ ? expanded_cap_ : unique_cap_);
        if (key == "recv_topk_idx")
            return expand_ ? s.recv_idx.narrow(0, 0, expanded_cap_) : s.recv_idx.narrow(0, 0, unique_cap_ * K).view({unique_cap_, K});
        if (key == "recv_topk_weights")
            return expand_ ? s.recv_w.narrow(0, 0, expanded_cap_) : s.recv_w.narrow(0, 0, unique_cap_ * K).view({unique_cap_, K});
        if (key == "comb_map") return at::alias(s.comb_map);
        if (key == "recv_chan_counts") return at::alias(s.recv_chan_counts);
        if (key == "unique_count") return at::alias(s.unique_count);
        if (key == "expanded_count") return at::alias(s.expanded_count);
        if (key == "expert_counts") return at::alias(s.expert_counts);
        if (key == "expert_offsets") return at::alias(s.expert_offsets);
        if (key == "expert_prefix") return at::alias(s.expert_prefix);
        if (key == "source_offsets") return at::alias(s.source_offsets);
        if (key == "source_expert_prefix") return at::alias(s.source_expert_prefix);
        if (key == "error") return at::alias(s.error);
        if (key == "stats") return at::alias(s.stats);
        if (key == "transport_timestamps_ns") return at::alias(s.timestamps);
        if (key == "prefix_tx_timestamps_ns") return at::alias(s.prefix_tx_ts);
        if (key == "combine_error") return at::alias(s.combine_error);
        if (key == "combine_stats") return at::alias(s.combine_stats);
        if (key == "profiling") return at::alias(s.profile);
        if (key == "combine_profiling") return at::alias(s.combine_profile);
        if (key == "role_profiling") return at::alias(s.role_profile);
        throw py::key_error(key);
    }

    std::shared_ptr<OutputSet> set_;
    std::shared_ptr<Layout> layout_;
    bool expand_;
    int num_tokens_, unique_cap_, expanded_cap_, topk_;
    bool recv_fp8_ = false;
    std::unordered_map<std::string, at::Tensor> cache_;
    py::dict overrides_;
};

struct PreparedDispatch {
    DispatchArgs args;
    std::shared_ptr<DispatchResult> result;
};

struct PreparedCombine {
    CombineArgs args;          // cooperative kernel (combine_reduce="inline")
    at::Tensor out;
    bool inline_kernel = false;  // one cooperative launch does both sides
    CombinePushArgs push{};    // expert side as an ordinary launch (the default)
    bool reduce_needed = false;  // more than one rank: the owner-side sum follows as a second ordinary launch
    FusedReduceArgs reduce{};
};

class Runtime {
   public:
    Runtime(int rank, int num_ranks, int num_max_tokens, int hidden, int num_topk, int num_experts,
            const py::dict& options, const std::vector<std::int64_t>& segment_pointers, int device)
        : rank_(rank), device_(device), options_(RuntimeOptions::parse(options)) {
        if (num_ranks < 1 || num_ranks > kMaxRanks) throw std::invalid_argument("num_ranks must be in [1,16]");
        if (rank < 0 || rank >= num_ranks) throw std::invalid_argument("rank out of range");
        if (num_topk < 1 || num_topk > kMaxTopk) throw std::invalid_argument("num_topk must be in [1,32]");
        if (num_experts < num_ranks || num_experts > kMaxExperts || num_experts % num_ranks)
            throw std::invalid_argument("num_experts must be a multiple of num_ranks, at most 4096");
        if (hidden < 1 || num_max_tokens < 1) throw std::invalid_argument("hidden and num_max_tokens must be positive");
        if (static_cast<int>(segment_pointers.size()) != num_ranks) throw std::invalid_argument("one segment pointer per rank");
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        lay_ = make_segment_layout(num_ranks, options_.channels, num_experts, num_topk, hidden, num_max_tokens,
                                   options_.payload_slots, options_.enable_combine, options_.enable_fused);
        // automatic choice: one sender CTA per eight channels, at most sixteen (sixteen SMs saturate NVLink)
        if (options_.send_ctas < 0) options_.send_ctas = num_ranks > 1 ? std::min(16, std::max(1, options_.channels / 8)) : 0;
        if (num_ranks == 1) options_.send_ctas = 0;  // nothing leaves a single rank
        const bool vec_ok = (hidden * 2) % 16 == 0 && !options_.force_scalar;
        use_tma_ = options_.use_tma && vec_ok && !(options_.recv_fp8 && hidden % 16 != 0);
        if (dispatch_row_buffer_count(options_.tx_warps, options_.rx_warps, options_.send_stages, options_.send_ctas) > kMaxRowBuffers)
            throw std::invalid_argument("tx_warps * pipeline_stages + rx_warps exceeds the row buffers a CTA can manage");
        if (dispatch_cta_warps(options_.tx_warps, options_.rx_warps, options_.send_ctas) > kMaxWarps)
            throw std::invalid_argument("too many warps per CTA: at most 16");
        smem_ = dispatch_shared_bytes(lay_, options_.tx_warps, options_.rx_warps, use_tma_, options_.send_stages, options_.send_ctas);
        int max_optin = 0;
        cuda_check(cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device), "query shared memory");
        // too many row buffers for this hidden size: give up send stages first, then receive warps, and only
        // then fall back to the register path
        while (use_tma_ && smem_ > static_cast<std::size_t>(max_optin)) {
            if (options_.send_stages > 2) --options_.send_stages;
            else if (options_.send_ctas > 0 && options_.tx_warps * options_.send_stages > options_.rx_warps && options_.tx_warps > 1) --options_.tx_warps;
            else if (options_.rx_warps > 2) --options_.rx_warps;
            else break;
            smem_ = dispatch_shared_bytes(lay_, options_.tx_warps, options_.rx_warps, true, options_.send_stages, options_.send_ctas);
        }
        if (use_tma_ && smem_ > static_cast<std::size_t>(max_optin)) {
            use_tma_ = false;
            smem_ = dispatch_shared_bytes(lay_, options_.tx_warps, options_.rx_warps, false, options_.send_stages, options_.send_ctas);
        }
        threads_ = 32 * dispatch_cta_warps(options_.tx_warps, options_.rx_warps, options_.send_ctas);
        grid_ctas_ = options_.channels + options_.send_ctas;
        if (smem_ > static_cast<std::size_t>(max_optin)) throw std::runtime_error("dispatch kernel needs more shared memory than the device offers");
        cuda_check(configure_kernels(smem_), "configure kernels");

        const auto i32 = at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device);
        const auto i64 = at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device);
        const auto u8 = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device);
        const int P = num_ranks, C = options_.channels, E = num_experts, K = num_topk;
        epochs_ = at::zeros({4}, i64);
        grid_bar_ = at::zeros({2}, i64);
        done_ctas_ = at::zeros({2}, i64);
        block_hist_ = at::zeros({static_cast<std::int64_t>(hist_scratch_ints(C, E + P))}, i32);
        sticky_ = at::zeros({8}, i32);
        chan_stats_ = at::zeros({2, C + options_.send_ctas, 10}, i64);
        plan_flags_ = at::zeros({C}, i64);
        rank_const_ = at::zeros({static_cast<std::int64_t>(sizeof(RankConst))}, u8);

        rc_ = RankConst{};
        rc_.lay = lay_;
        for (int r = 0; r < P; ++r) rc_.seg[r] = reinterpret_cast<std::uint8_t*>(segment_pointers[r]);
        rc_.rank = rank;
        rc_.ring_mode = lay_.slots < lay_.slots_full ? 1 : 0;
        rc_.wire_fp8 = options_.wire_fp8 ? 1 : 0;
        rc_.recv_fp8 = options_.recv_fp8 ? 1 : 0;
        rc_.use_tma = use_tma_ ? 1 : 0;
        rc_.vec_ok = vec_ok ? 1 : 0;
        rc_.tx_warps = options_.tx_warps;
        rc_.rx_warps = options_.rx_warps;
        rc_.send_stages = options_.send_stages;
        rc_.send_ctas = options_.send_ctas;
        // one system-scope fence per row: always on host segments; on peer segments only on request (the conservative
        // way to publish a row, PCIE_EP_B200_FENCE_EVERY_ROW=1 -- by default the flags of several rows share a fence)
        const char* every_row = std::getenv("PCIE_EP_B200_FENCE_EVERY_ROW");
        rc_.fence_flags = (every_row != nullptr && every_row[0] == '1') ? 2 : (options_.host_segments ? 1 : 0);
        rc_.plan_flags = reinterpret_cast<std::uint64_t*>(plan_flags_.data_ptr<std::int64_t>());
        rc_.unique_cap = P * num_max_tokens;
        rc_.expanded_cap = P * num_max_tokens * std::min(K, lay_.num_local_experts) + lay_.num_local_experts * 255;
        rc_.timeout_ns = static_cast<std::uint64_t>(options_.timeout_ms) * 1000000ull;
        rc_.epochs = reinterpret_cast<std::uint64_t*>(epochs_.data_ptr<std::int64_t>());
        rc_.grid_bar = reinterpret_cast<unsigned long long*>(grid_bar_.data_ptr<std::int64_t>());
        rc_.done_ctas = reinterpret_cast<unsigned long long*>(done_ctas_.data_ptr<std::int64_t>());
        rc_.block_hist = block_hist_.data_ptr<int>();
        rc_.sticky = sticky_.data_ptr<int>();
        rc_.chan_stats = chan_stats_.data_ptr<std::int64_t>();
        rc_.delay_meta_ns = options_.delay_meta_ns;
        rc_.delay_tx_ns = options_.delay_tx_ns;
        rc_.delay_rx_ns = options_.delay_rx_ns;
        rc_.delay_scatter_ns = options_.delay_scatter_ns;
        rc_.test_skip_done_to = -1;
        upload_constants();

        const int sets = options_.output_pool_size + (options_.enable_graph ? 1 : 0);
        for (int i = 0; i < sets; ++i) {
            pools_.push_back(std::make_shared<OutputSet>(make_output_set()));
            plans_.push_back(make_layout());
        }
        // finished CTAs of the launch in flight: [0] scatter GEMM, [1] fused reduction, [2] combine owner-side sum,
        // [3] combine push; [4..8] statistics accumulators of the combine push
        fused_counters_ = at::zeros({16 + kMaxSmTable}, i64);
        fused_counters_[6] = -1;  // "first start" accumulator of the combine push: all ones = unset
        fused_status_ = at::zeros({4}, i32);
        fused_gemm_ctas_ = grouped_gemm_ctas();
        // Forwarder CTAs of the combine push.  What keeps NVLink full is the number of bytes in flight: six row buffers per
        // forwarder CTA (more would cost the reducer CTAs their second CTA per SM), so thirty-two CTAs where the push is
        // bound by the link (four ranks and more) and sixteen where it is bound by the reducers' HBM traffic.
        combine_forward_ctas_ = std::min(num_ranks > 2 ? 32 : 16, std::max(1, fused_gemm_ctas_ / 4));
        if (options_.enable_combine && num_ranks > 1 && !combine_is_inline()) ensure_outbox();
        if (options_.enable_combine) {
            const auto bf16 = at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, device);
            for (int i = 0; i < options_.output_pool_size; ++i)
                combine_pool_.push_back(at::empty({num_max_tokens, hidden}, bf16));
        }
    }

    // ---- geometry -----------------------------------------------------------------------------
    int rank() const { return rank_; }
    int channels() const { return options_.channels; }
    int send_ctas() const { return options_.send_ctas; }
    int grid_ctas() const { return grid_ctas_; }
    int threads() const { return threads_; }
    std::size_t shared_bytes() const { return smem_; }
    bool uses_tma() const { return use_tma_; }
    int send_stages() const { return options_.send_stages; }
    const SegmentLayout& layout() const { return lay_; }
    int unique_capacity() const { return rc_.unique_cap; }
    int expanded_capacity() const { return rc_.expanded_cap; }

    // ---- dispatch -------------------------------------------------------------------------------
    PreparedDispatch prepare_dispatch(const at::Tensor& x, const at::Tensor& topk_idx,
                                      const std::optional<at::Tensor>& topk_weights, int alignment, bool expand,
                                      bool zero_padding, const std::shared_ptr<Layout>& cached, bool graph_pool) {
        check_open();
        validate_inputs(x, topk_idx, topk_weights, alignment, expand, zero_padding);
        const int T = static_cast<int>(x.size(0));
        std::shared_ptr<OutputSet> out_set = select_output(graph_pool);
        OutputSet& out = *out_set;
        std::shared_ptr<Layout> plan;
        if (cached) {
            if (!cached->valid || cached->num_tokens != T || cached->alignment != alignment || cached->expand != expand)
                throw std::invalid_argument("cached layout does not match this dispatch");
            plan = cached;
        } else {
            plan = select_plan(graph_pool);
            plan->num_tokens = T;
            plan->alignment = alignment;
            plan->expand = expand;
            plan->valid = true;
        }
        PreparedDispatch p;
        DispatchArgs& a = p.args;
        a = DispatchArgs{};
        a.rc = reinterpret_cast<const RankConst*>(rank_const_.data_ptr<std::uint8_t>());
        a.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
        a.topk_idx = topk_idx.data_ptr<std::int64_t>();
        a.topk_w = topk_weights.has_value() ? topk_weights->data_ptr<float>() : nullptr;
        a.num_tokens = T;
        a.do_expand = expand ? 1 : 0;
        a.alignment = alignment;
        a.zero_padding = zero_padding ? 1 : 0;
        a.cached = cached ? 1 : 0;
        a.plan_mask = reinterpret_cast<std::uint32_t*>(plan->mask.data_ptr<int>());
        a.plan_slot = plan->slot.data_ptr<int>();
        a.plan_expert_ord = plan->expert_ord.data_ptr<int>();
        a.plan_counts = plan->counts.data_ptr<int>();
        a.recv_x = reinterpret_cast<__nv_bfloat16*>(out.recv_x.data_ptr());
        a.recv_idx = out.recv_idx.data_ptr<std::int64_t>();
        a.recv_w = out.recv_w.data_ptr<float>();
        a.recv_scale = out.recv_scale.data_ptr<float>();
        a.source_meta = out.source_meta.data_ptr<std::int64_t>();
        a.comb_map = out.comb_map.data_ptr<int>();
        a.recv_chan_counts = out.recv_chan_counts.data_ptr<int>();
        a.unique_count = out.unique_count.data_ptr<std::int64_t>();
        a.expanded_count = out.expanded_count.data_ptr<std::int64_t>();
        a.expert_counts = out.expert_counts.data_ptr<int>();
        a.expert_offsets = out.expert_offsets.data_ptr<int>();
        a.expert_prefix = out.expert_prefix.data_ptr<int>();
        a.source_offsets = out.source_offsets.data_ptr<int>();
        a.source_expert_prefix = out.source_expert_prefix.data_ptr<int>();
        a.error = out.error.data_ptr<int>();
        a.stats = out.stats.data_ptr<std::int64_t>();
        a.timestamps = out.timestamps.data_ptr<std::int64_t>();
        a.prefix_tx_ts = out.prefix_tx_ts.data_ptr<std::int64_t>();
        a.profile = out.profile.data_ptr<std::int64_t>();
        a.role_profile = out.role_profile.numel() > 0 ? out.role_profile.data_ptr<std::int64_t>() : nullptr;
        p.result = std::make_shared<DispatchResult>(out_set, plan, expand, T, rc_.unique_cap, rc_.expanded_cap, lay_.num_topk,
                                                    options_.recv_fp8);
        return p;
    }

    // `stream` = raw cudaStream_t to launch on; 0 means the current PyTorch stream of the device.
    std::shared_ptr<DispatchResult> dispatch(const at::Tensor& x, const at::Tensor& topk_idx,
                                             const std::optional<at::Tensor>& topk_weights, int alignment, bool expand,
                                             bool zero_padding, const std::shared_ptr<Layout>& cached, bool graph_pool,
                                             std::int64_t stream) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
        PreparedDispatch p = prepare_dispatch(x, topk_idx, topk_weights, alignment, expand, zero_padding, cached, graph_pool);
        DispatchLaunch launch{};
        launch.num_virtual = 1;
        launch.r[0] = p.args;
        cudaStream_t launch_stream = stream != 0 ? reinterpret_cast<cudaStream_t>(stream)
                                                 : at::cuda::getCurrentCUDAStream(device_).stream();
        cuda_check(launch_dispatch(launch, grid_ctas_, threads_, smem_, launch_stream), "dispatch launch");
        return p.result;
    }

    // ---- combine --------------------------------------------------------------------------------
    PreparedCombine prepare_combine(const at::Tensor& y, const DispatchResult& dispatch_result, bool weighted,
                                    const std::optional<at::Tensor>& out_opt) {
        check_open();
        if (!options_.enable_combine) throw std::runtime_error("this buffer was built with enable_combine=False");
        const std::shared_ptr<Layout>& layout = dispatch_result.layout();
        if (!layout || !layout->valid) throw std::invalid_argument("dispatch result carries no routing plan");
        const bool expand = dispatch_result.expand();
        const int cap = expand ? rc_.expanded_cap : rc_.unique_cap;
        if (!y.is_cuda() || y.get_device() != device_ || y.scalar_type() != at::kBFloat16 || !y.is_contiguous() ||
            y.dim() != 2 || y.size(1) != lay_.hidden || y.size(0) < 1 || y.size(0) > cap)
            throw std::invalid_argument("expert outputs must be contiguous CUDA BF16 [rows <= capacity, hidden]");
        if (rc_.vec_ok && reinterpret_cast<std::uintptr_t>(y.data_ptr()) % 16 != 0)
            throw std::invalid_argument("expert outputs must start on a 16-byte boundary");
        const int T = layout->num_tokens;
        // No allocation on the hot path: without `out`, the result comes from a small ring of
        // preallocated [Tmax, hidden] tensors with the same "busy while referenced" rule as dispatch.
        at::Tensor out = out_opt.has_value() ? *out_opt : select_combine_output(T);
        if (!out.is_cuda() || out.scalar_type() != at::kBFloat16 || !out.is_contiguous() || out.dim() != 2 ||
            out.size(0) != T || out.size(1) != lay_.hidden)
            throw std::invalid_argument("combine output must be contiguous CUDA BF16 [T, hidden]");
        PreparedCombine p;
        p.out = out;
        CombineArgs& a = p.args;
        a = CombineArgs{};
        a.rc = reinterpret_cast<const RankConst*>(rank_const_.data_ptr<std::uint8_t>());
        a.y = reinterpret_cast<const __nv_bfloat16*>(y.data_ptr());
        const OutputSet& set = dispatch_result.set_ref();
        a.comb_map = set.comb_map.data_ptr<int>();
        a.recv_chan_counts = set.recv_chan_counts.data_ptr<int>();
        a.plan_mask = reinterpret_cast<const std::uint32_t*>(layout->mask.data_ptr<int>());
        a.num_tokens = T;
        a.weighted = weighted ? 1 : 0;
        a.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
        a.error = set.combine_error.data_ptr<int>();
        a.stats = set.combine_stats.data_ptr<std::int64_t>();
        a.profile = set.combine_profile.data_ptr<std::int64_t>();
        p.inline_kernel = combine_is_inline();
        if (p.inline_kernel) return p;
        unsigned long long* counters = reinterpret_cast<unsigned long long*>(fused_counters_.data_ptr<std::int64_t>());
        CombinePushArgs& push = p.push;
        push.rc = a.rc;
        push.y = a.y;
        push.comb_map = a.comb_map;
        push.recv_chan_counts = a.recv_chan_counts;
        push.plan_mask = a.plan_mask;
        push.num_tokens = T;
        push.weighted = a.weighted;
        push.out = a.out;
        push.error = a.error;
        push.stats = a.stats;
        push.cta_done = counters + 3;
        push.stat_scratch = counters + 4;
        push.next_unit = counters + 9;
        push.forwarder_sms = counters + 16;
        push.forward_ctas = lay_.num_ranks > 1 ? combine_forward_ctas_ : 0;
        if (push.forward_ctas > 0) {
            ensure_outbox();
            push.outbox = outbox_.data_ptr<std::uint8_t>();
            push.outbox_units = reinterpret_cast<unsigned long long*>(outbox_units_.data_ptr<std::int64_t>());
        }
        p.reduce_needed = lay_.num_ranks > 1;
        if (p.reduce_needed) {
            FusedReduceArgs& r = p.reduce;
            r.rc = a.rc;
            r.expert_ord = nullptr;
            r.rank_mask = a.plan_mask;
            r.gemm_status = nullptr;
            r.num_tokens = T;
            r.epoch = 0;  // the combine epoch the push launch has just advanced on the device
            r.cta_done = counters + 2;
            r.stage_off = lay_.cstage_off;
            r.sig_off = lay_.csig_off;
            r.done_off = lay_.cdone_off;
            r.slot_stride = static_cast<std::size_t>(lay_.num_max_tokens) * lay_.crow_stride;
            r.token_stride = static_cast<std::size_t>(lay_.crow_stride);
            r.slots = lay_.num_ranks;
            r.out = a.out;
            r.error = a.error;
        }
        return p;
    }

    // combine_reduce="inline" (and every hidden size whose rows are not 16-byte multiples) runs the one cooperative
    // kernel; otherwise combine is two ordinary launches (one with a single rank: its reduced rows are the result).
    bool combine_is_inline() const { return rc_.vec_ok == 0 || options_.combine_reduce == "inline"; }
    bool combine_is_split() const { return !combine_is_inline() && lay_.num_ranks > 1; }
    bool combine_is_local() const { return !combine_is_inline() && lay_.num_ranks == 1; }

    // CTAs of the ordinary combine launches: `num_sms` > 0 limits them to that many SMs' worth
    int combine_ctas(int per_sm, int num_sms) const {
        const int sms = num_sms > 0 ? std::min(num_sms, fused_gemm_ctas_) : fused_gemm_ctas_;
        return per_sm * std::max(1, sms);
    }

    void launch_combine_push(PreparedCombine& prepared, cudaStream_t stream, int num_sms = 0) {
        const int forward = prepared.push.forward_ctas;
        // two reducer CTAs per SM; with `num_sms` the whole launch (forwarders included) stays inside that many SMs
        // forwarders + reducers together never exceed what is resident at once (a reducer CTA that had to wait for a
        // slot would hold back the forwarders, which take rows in order)
        const int reducers = std::max(2, combine_ctas(2, num_sms) - forward);
        cuda_check(bep::launch_combine_push(prepared.push, reducers, combine_push_smem_bytes(lay_, forward), stream), "combine push launch");
    }
    // second launch of the default combine; `prepared` comes from prepare_combine of this runtime
    void launch_combine_reduce(PreparedCombine& prepared, cudaStream_t stream, int num_sms = 0) {
        if (!prepared.reduce_needed) return;
        // as many CTAs as are resident at once (the wider steps of the few-rank builds take more registers)
        cuda_check(launch_fused_reduce(prepared.reduce, combine_ctas(fused_reduce_groups(prepared.reduce.slots) == 1 ? 4 : 3, num_sms), stream),
                   "combine reduce launch");
    }

    at::Tensor combine(const at::Tensor& y, const DispatchResult& dispatch_result, bool weighted,
                       const std::optional<at::Tensor>& out_opt, std::int64_t stream, int num_sms = 0) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
        PreparedCombine p = prepare_combine(y, dispatch_result, weighted, out_opt);
        cudaStream_t launch_stream = stream != 0 ? reinterpret_cast<cudaStream_t>(stream)
                                                 : at::cuda::getCurrentCUDAStream(device_).stream();
        if (p.inline_kernel) {
            CombineLaunch launch{};
            launch.num_virtual = 1;
            launch.r[0] = p.args;
            cuda_check(launch_combine(launch, options_.channels, static_cast<std::size_t>(lay_.crow_stride), launch_stream), "combine launch");
            return p.out;
        }
        launch_combine_push(p, launch_stream, num_sms);
        launch_combine_reduce(p, launch_stream, num_sms);
        return p.out;
    }

    // ---- fused down-projection + combine ------------------------------------------------------------
    // Step 1 (expert side): out rows = hidden_rows x w_down[e]^T, multiplied by the routing weight and written by
    // the GEMM epilogue into the token owners' landing slots.  Step 2 (owner side): sum the K slots per token.
    // The two steps are separate calls so that several virtual ranks of one process can run all their GEMMs
    // before any reduction (a reduction waits for every rank's GEMM).
    void fused_scatter_gemm(const at::Tensor& hidden_rows, const at::Tensor& w_down, const DispatchResult& dispatch_result,
                            std::int64_t stream) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
        check_open();
        if (!options_.enable_fused) throw std::runtime_error("this buffer was built with fused_expert_combine=False");
        if (!dispatch_result.expand()) throw std::invalid_argument("the fused expert combine needs an expanded dispatch (do_expand=True)");
        if (lay_.hidden % 256 != 0) throw std::invalid_argument("the fused expert combine needs hidden to be a multiple of 256");
        const int cap = rc_.expanded_cap;
        if (!hidden_rows.is_cuda() || hidden_rows.get_device() != device_ || hidden_rows.scalar_type() != at::kBFloat16 ||
            !hidden_rows.is_contiguous() || hidden_rows.dim() != 2 || hidden_rows.size(0) < 1 || hidden_rows.size(0) > cap)
            throw std::invalid_argument("expert activations must be contiguous CUDA BF16 [rows <= capacity, intermediate]");
        const std::int64_t inter = hidden_rows.size(1);
        if (!w_down.is_cuda() || w_down.get_device() != device_ || w_down.scalar_type() != at::kBFloat16 || !w_down.is_contiguous() ||
            w_down.dim() != 3 || w_down.size(0) != lay_.num_local_experts || w_down.size(1) != lay_.hidden || w_down.size(2) != inter)
            throw std::invalid_argument("w_down must be contiguous CUDA BF16 [local experts, hidden, intermediate]");
        if (fused_gemm_epoch_ != fused_reduce_epoch_) throw std::runtime_error("fused_scatter_gemm called twice without fused_reduce");
        if (grouped_gemm_ctas() != fused_gemm_ctas_) throw std::runtime_error("device changed under the fused expert combine");
        const OutputSet& set = dispatch_result.set_ref();
        gemm::ScatterTarget target{};
        for (int r = 0; r < lay_.num_ranks; ++r) target.seg[r] = rc_.seg[r];
        target.source_meta = reinterpret_cast<const long long*>(set.source_meta.data_ptr<std::int64_t>());
        target.row_weights = set.recv_w.data_ptr<float>();
        target.stage_off = lay_.fstage_off;
        target.sig_off = lay_.fsig_off;
        target.done_off = lay_.fdone_off;
        target.epoch = fused_gemm_epoch_ + 1;
        target.cta_done = reinterpret_cast<unsigned long long*>(fused_counters_.data_ptr<std::int64_t>());
        target.timeout_ns = rc_.timeout_ns;
        target.row_stride = lay_.crow_stride;
        target.num_topk = lay_.num_topk;
        target.num_ranks = lay_.num_ranks;
        target.rank = rank_;
        target.flag_stride = kFlagStride;
        cudaStream_t launch_stream = stream != 0 ? reinterpret_cast<cudaStream_t>(stream)
                                                 : at::cuda::getCurrentCUDAStream(device_).stream();
        const char* message = grouped_gemm_scatter(hidden_rows.data_ptr(), w_down.data_ptr(), set.expert_offsets.data_ptr<int>(),
                                                   set.expert_counts.data_ptr<int>(), fused_status_.data_ptr<int>(),
                                                   static_cast<int>(hidden_rows.size(0)), lay_.num_local_experts, lay_.hidden,
                                                   static_cast<int>(inter), target, launch_stream);
        if (message != nullptr) throw std::runtime_error(std::string("fused scatter GEMM: ") + message);
        ++fused_gemm_epoch_;
    }

    at::Tensor fused_reduce(const DispatchResult& dispatch_result, const std::optional<at::Tensor>& out_opt, std::int64_t stream) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
        check_open();
        if (fused_reduce_epoch_ + 1 != fused_gemm_epoch_) throw std::runtime_error("fused_reduce needs one preceding fused_scatter_gemm");
        const std::shared_ptr<Layout>& layout = dispatch_result.layout();
        if (!layout || !layout->valid) throw std::invalid_argument("dispatch result carries no routing plan");
        const int T = layout->num_tokens;
        at::Tensor out = out_opt.has_value() ? *out_opt : select_combine_output(T);
        if (!out.is_cuda() || out.scalar_type() != at::kBFloat16 || !out.is_contiguous() || out.dim() != 2 ||
            out.size(0) != T || out.size(1) != lay_.hidden)
            throw std::invalid_argument("combine output must be contiguous CUDA BF16 [T, hidden]");
        FusedReduceArgs a{};
        a.rc = reinterpret_cast<const RankConst*>(rank_const_.data_ptr<std::uint8_t>());
        a.expert_ord = layout->expert_ord.data_ptr<int>();
        a.rank_mask = nullptr;
        a.gemm_status = fused_status_.data_ptr<int>();
        a.num_tokens = T;
        a.epoch = fused_reduce_epoch_ + 1;
        a.cta_done = reinterpret_cast<unsigned long long*>(fused_counters_.data_ptr<std::int64_t>()) + 1;
        a.stage_off = lay_.fstage_off;
        a.sig_off = lay_.fsig_off;
        a.done_off = lay_.fdone_off;
        a.slot_stride = static_cast<std::size_t>(lay_.crow_stride);
        a.token_stride = static_cast<std::size_t>(lay_.num_topk) * lay_.crow_stride;
        a.slots = lay_.num_topk;
        a.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
        a.error = dispatch_result.set_ref().combine_error.data_ptr<int>();
        cudaStream_t launch_stream = stream != 0 ? reinterpret_cast<cudaStream_t>(stream)
                                                 : at::cuda::getCurrentCUDAStream(device_).stream();
        cuda_check(launch_fused_reduce(a, 4 * fused_gemm_ctas_, launch_stream), "fused reduce launch");
        ++fused_reduce_epoch_;
        return out;
    }
    at::Tensor fused_status() const { return fused_status_; }

    // ---- diagnostics / test hooks --------------------------------------------------------------
    py::dict pool_debug() const {
        py::dict d;
        py::list busy;
        for (const auto& set : pools_) busy.append(!(set.use_count() == 1 && set->free()));
        d["output_busy"] = busy;
        py::list plan_busy;
        for (const auto& plan : plans_) plan_busy.append(plan.use_count() != 1);
        d["plan_busy"] = plan_busy;
        d["output_sets"] = static_cast<int>(pools_.size());
        d["graph_set"] = options_.enable_graph;
        return d;
    }
    void set_test_delays(std::uint64_t meta, std::uint64_t tx, std::uint64_t rx, std::uint64_t scatter) {
        rc_.delay_meta_ns = meta;
        rc_.delay_tx_ns = tx;
        rc_.delay_rx_ns = rx;
        rc_.delay_scatter_ns = scatter;
        upload_constants();
    }
    void set_test_prefix_delay_ns(std::uint64_t ns) {
        rc_.delay_prefix_ns = ns;
        upload_constants();
    }
    void set_test_skip_counts_ack_source(int peer) {
        rc_.test_skip_done_to = peer;
        upload_constants();
    }
    void set_test_withhold_counts(bool on) {
        rc_.test_withhold_counts = on ? 1 : 0;
        upload_constants();
    }
    void set_test_corrupt_sequence(bool on) {
        rc_.test_corrupt_sequence = on ? 1 : 0;
        upload_constants();
    }
    void set_test_control_abort_after_ns(std::uint64_t ns) {
        rc_.test_abort_after_ns = ns;
        upload_constants();
    }
    void set_timeout_ms(int ms) {
        rc_.timeout_ns = static_cast<std::uint64_t>(ms) * 1000000ull;
        upload_constants();
    }
    at::Tensor sticky_error() const { return sticky_; }
    at::Tensor epochs() const { return epochs_; }

    void close() {
        outbox_ = at::Tensor();
        outbox_units_ = at::Tensor();
        pools_.clear();
        plans_.clear();
        combine_pool_.clear();
        closed_ = true;
    }
    bool closed() const { return closed_; }

   private:
    void check_open() const {
        if (closed_) throw std::runtime_error("runtime is closed");
    }

    void upload_constants() {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
        // stream-ordered after everything already queued on the current stream
        cuda_check(cudaMemcpyAsync(rank_const_.data_ptr<std::uint8_t>(), &rc_, sizeof(RankConst), cudaMemcpyHostToDevice,
                                   at::cuda::getCurrentCUDAStream(device_)),
                   "upload rank constants");
        cuda_check(cudaStreamSynchronize(at::cuda::getCurrentCUDAStream(device_)), "upload rank constants");
    }

    void validate_inputs(const at::Tensor& x, const at::Tensor& idx, const std::optional<at::Tensor>& w, int alignment,
                         bool expand, bool zero_padding) const {
        auto on_device = [this](const at::Tensor& t) { return t.is_cuda() && t.get_device() == device_; };
        if (!on_device(x) || x.scalar_type() != at::kBFloat16 || !x.is_contiguous() || x.dim() != 2 || x.size(1) != lay_.hidden)
            throw std::invalid_argument("x must be contiguous CUDA BF16 [T, hidden] on the buffer's device");
        if (x.size(0) > lay_.num_max_tokens) throw std::invalid_argument("token count exceeds num_max_tokens_per_rank");
        if (rc_.vec_ok && reinterpret_cast<std::uintptr_t>(x.data_ptr()) % 16 != 0)
            throw std::invalid_argument("x must start on a 16-byte boundary");
        if (!on_device(idx) || idx.scalar_type() != at::kLong || !idx.is_contiguous() || idx.dim() != 2 ||
            idx.size(0) != x.size(0) || idx.size(1) != lay_.num_topk)
            throw std::invalid_argument("topk_idx must be contiguous CUDA int64 [T, num_topk]");
        if (w.has_value()) {
            if (!on_device(*w) || w->scalar_type() != at::kFloat || !w->is_contiguous() || w->sizes() != idx.sizes())
                throw std::invalid_argument("topk_weights must be contiguous CUDA float32 [T, num_topk]");
        }
        if (alignment < 1 || alignment > kMaxAlignment) throw std::invalid_argument("expert_alignment must be in [1,256]");
        if (zero_padding && !expand) throw std::invalid_argument("do_zero_padding requires do_expand");
    }

    OutputSet make_output_set() const {
        const auto bf16 = at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, device_);
        const auto i32 = at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device_);
        const auto i64 = at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device_);
        const auto f32 = at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device_);
        const std::int64_t P = lay_.num_ranks, C = lay_.num_channels, K = lay_.num_topk, El = lay_.num_local_experts;
        const std::int64_t ecap = rc_.expanded_cap, ucap = rc_.unique_cap;
        const std::int64_t rows = std::max(ecap, ucap);
        const std::int64_t scalars = std::max(ecap, ucap * K);
        OutputSet s;
        s.recv_x = at::empty({rows, lay_.hidden}, bf16);
        s.recv_idx = at::empty({scalars}, i64);
        s.recv_w = at::empty({scalars}, f32);
        s.recv_scale = at::zeros({options_.recv_fp8 ? rows : 1}, f32);
        s.source_meta = at::empty({rows, 3}, i64);
        s.comb_map = at::zeros({P * C * lay_.slots_full, 2 + 2 * K}, i32);
        s.recv_chan_counts = at::zeros({P, C}, i32);
        s.unique_count = at::zeros({1}, i64);
        s.expanded_count = at::zeros({1}, i64);
        s.expert_counts = at::zeros({El}, i32);
        s.expert_offsets = at::zeros({El + 1}, i32);
        s.expert_prefix = at::zeros({El}, i32);
        s.source_offsets = at::zeros({P + 1}, i32);
        s.source_expert_prefix = at::zeros({P, El}, i32);
        s.error = at::zeros({8}, i32);
        s.stats = at::zeros({8}, i64);
        s.timestamps = at::zeros({2}, i64);
        const std::int64_t ctas = grid_ctas_;  // channel CTAs, then the dedicated senders
        s.prefix_tx_ts = at::zeros({ctas + 1, 2}, i64);
        s.combine_error = at::zeros({8}, i32);
        s.combine_stats = at::zeros({8}, i64);
        s.profile = at::zeros({ctas, 16}, i64);
        s.combine_profile = at::zeros({C, 8}, i64);
        // per-warp role counters exist only in a library built with the role instrumentation
        s.role_profile = role_profiling_enabled() ? at::zeros({ctas, kMaxWarps, kRoleFieldCount}, i64) : at::zeros({0, kMaxWarps, kRoleFieldCount}, i64);
        return s;
    }

    std::shared_ptr<Layout> make_layout() const {
        const auto i32 = at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device_);
        const std::int64_t P = lay_.num_ranks, C = lay_.num_channels, K = lay_.num_topk, E = lay_.num_experts;
        const std::int64_t T = lay_.num_max_tokens;
        auto plan = std::make_shared<Layout>();
        plan->mask = at::zeros({T}, i32);
        plan->slot = at::zeros({T, P}, i32);
        plan->expert_ord = at::zeros({T, K}, i32);
        plan->counts = at::zeros({P + E + C * P}, i32);
        return plan;
    }

    void ensure_outbox() {
        if (outbox_.defined()) return;
        const std::int64_t rows = static_cast<std::int64_t>(lay_.num_ranks) * lay_.num_channels * lay_.slots_full;
        outbox_ = at::empty({rows * lay_.crow_stride}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device_));
        outbox_units_ = at::zeros({rows}, at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device_));
    }

    std::shared_ptr<OutputSet> select_output(bool graph_pool) {
        if (graph_pool) {
            if (!options_.enable_graph) throw std::runtime_error("graph pool requires enable_graph=True");
            return pools_.back();
        }
        for (int i = 0; i < options_.output_pool_size; ++i) {
            const int index = (next_pool_ + i) % options_.output_pool_size;
            if (pools_[index].use_count() == 1 && pools_[index]->free()) {
                next_pool_ = (index + 1) % options_.output_pool_size;
                return pools_[index];
            }
        }
        throw std::runtime_error("output pool exhausted: every preallocated result set is still referenced");
    }

    at::Tensor select_combine_output(int num_tokens) {
        if (combine_pool_.empty()) {
            const auto bf16 = at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, device_);
            for (int i = 0; i < options_.output_pool_size; ++i)
                combine_pool_.push_back(at::empty({lay_.num_max_tokens, lay_.hidden}, bf16));
        }
        const int n = static_cast<int>(combine_pool_.size());
        for (int i = 0; i < n; ++i) {
            const int index = (next_combine_ + i) % n;
            if (tensor_unowned(combine_pool_[index])) {
                next_combine_ = (index + 1) % n;
                return combine_pool_[index].narrow(0, 0, num_tokens);
            }
        }
        throw std::runtime_error("combine output pool exhausted: every preallocated output is still referenced");
    }

    std::shared_ptr<Layout> select_plan(bool graph_pool) {
        if (graph_pool) return plans_.back();
        for (int i = 0; i < options_.output_pool_size; ++i) {
            if (plans_[i].use_count() == 1) return plans_[i];
        }
        throw std::runtime_error("routing plan pool exhausted: every plan is still referenced by a handle or cached layout");
    }

    int rank_, device_;
    RuntimeOptions options_;
    SegmentLayout lay_{};
    RankConst rc_{};
    bool use_tma_ = false;
    int threads_ = 0;
    std::size_t smem_ = 0;
    at::Tensor epochs_, grid_bar_, done_ctas_, block_hist_, sticky_, chan_stats_, plan_flags_, rank_const_;
    int grid_ctas_ = 0;
    std::vector<std::shared_ptr<OutputSet>> pools_;
    std::vector<std::shared_ptr<Layout>> plans_;
    std::vector<at::Tensor> combine_pool_;
    at::Tensor fused_counters_, fused_status_;
    at::Tensor outbox_, outbox_units_;  // combine: local staging of rows owned by other ranks + per-row unit counters
    int combine_forward_ctas_ = 16;
    std::uint64_t fused_gemm_epoch_ = 0, fused_reduce_epoch_ = 0;
    int fused_gemm_ctas_ = 0;
    int next_pool_ = 0;
    int next_combine_ = 0;
    bool closed_ = false;
};

// Several virtual ranks of one process in one cooperative launch (tests, single-GPU development).
inline void launch_dispatch_group(const std::vector<std::shared_ptr<Runtime>>& runtimes,
                                  const std::vector<PreparedDispatch>& prepared, int device) {
    if (runtimes.empty() || runtimes.size() != prepared.size() || runtimes.size() > kMaxVirtualRanks)
        throw std::invalid_argument("between 1 and 8 virtual ranks per launch");
    DispatchLaunch launch{};
    launch.num_virtual = static_cast<int>(runtimes.size());
    for (std::size_t i = 0; i < runtimes.size(); ++i) {
        if (runtimes[i]->grid_ctas() != runtimes[0]->grid_ctas() || runtimes[i]->threads() != runtimes[0]->threads() ||
            runtimes[i]->shared_bytes() != runtimes[0]->shared_bytes())
            throw std::invalid_argument("virtual ranks must share one configuration");
        launch.r[i] = prepared[i].args;
    }
    const int resident = dispatch_resident_ctas(runtimes[0]->threads(), runtimes[0]->shared_bytes());
    if (runtimes[0]->grid_ctas() * launch.num_virtual > resident)
        throw std::runtime_error("(channels + send_ctas) * virtual_ranks exceeds the number of co-resident CTAs on this GPU");
    cuda_check(launch_dispatch(launch, runtimes[0]->grid_ctas(), runtimes[0]->threads(), runtimes[0]->shared_bytes(),
                               at::cuda::getCurrentCUDAStream(device)),
               "dispatch launch");
}

inline void launch_combine_group(const std::vector<std::shared_ptr<Runtime>>& runtimes,
                                 std::vector<PreparedCombine>& prepared, int device) {
    if (runtimes.empty() || runtimes.size() != prepared.size() || runtimes.size() > kMaxVirtualRanks)
        throw std::invalid_argument("between 1 and 8 virtual ranks per launch");
    cudaStream_t stream = at::cuda::getCurrentCUDAStream(device);
    if (prepared[0].inline_kernel) {
        CombineLaunch launch{};
        launch.num_virtual = static_cast<int>(runtimes.size());
        for (std::size_t i = 0; i < runtimes.size(); ++i) launch.r[i] = prepared[i].args;
        cuda_check(launch_combine(launch, runtimes[0]->channels(), static_cast<std::size_t>(runtimes[0]->layout().crow_stride), stream),
                   "combine launch");
        return;
    }
    // Ordinary launches in stream order: every rank's rows are pushed before any rank's sum starts, so no launch
    // ever waits for one that comes after it on the same GPU.
    for (std::size_t i = 0; i < runtimes.size(); ++i) runtimes[i]->launch_combine_push(prepared[i], stream);
    for (std::size_t i = 0; i < runtimes.size(); ++i) runtimes[i]->launch_combine_reduce(prepared[i], stream);
}

}  // namespace bep
