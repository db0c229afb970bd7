// Python bindings of the native runtime (parity: the reference's csrc/runtime.cu:8-29).
#include <torch/extension.h>

#include "buffers/runtime.hpp"
#include "comm/numa_relay.hpp"
#include "kernels/expert_gemm.hpp"
#include "kernels/litmus.hpp"

namespace py = pybind11;
using namespace bep;

namespace {

py::dict layout_to_dict(const SegmentLayout& l) {
    py::dict d;
    d["size_bytes"] = l.size_bytes;
    d["done_off"] = l.done_off;
    d["abort_off"] = l.abort_off;
    d["counts_flag_off"] = l.counts_flag_off;
    d["counts_off"] = l.counts_off;
    d["ready_off"] = l.ready_off;
    d["ack_off"] = l.ack_off;
    d["stage_off"] = l.stage_off;
    d["cdone_off"] = l.cdone_off;
    d["cready_off"] = l.cready_off;
    d["cstage_off"] = l.cstage_off;
    d["slots"] = l.slots;
    d["slots_full"] = l.slots_full;
    d["counts_stride"] = l.counts_stride;
    d["row_stride"] = l.row_stride;
    d["meta_off"] = l.meta_off;
    d["meta_off_fp8"] = l.meta_off_fp8;
    d["meta_bytes"] = l.meta_bytes;
    d["crow_stride"] = l.crow_stride;
    d["fsig_off"] = l.fsig_off;
    d["fdone_off"] = l.fdone_off;
    d["fstage_off"] = l.fstage_off;
    d["relay_off"] = l.relay_off;
    return d;
}

std::vector<std::shared_ptr<DispatchResult>> dispatch_group(const std::vector<std::shared_ptr<Runtime>>& runtimes,
                                     const std::vector<at::Tensor>& xs, const std::vector<at::Tensor>& idxs,
                                     const std::vector<std::optional<at::Tensor>>& weights, int alignment, bool expand,
                                     bool zero_padding, const std::vector<std::shared_ptr<Layout>>& cached,
                                     bool graph_pool, int device) {
    if (xs.size() != runtimes.size() || idxs.size() != runtimes.size() || weights.size() != runtimes.size() ||
        cached.size() != runtimes.size())
        throw std::invalid_argument("one input set per virtual rank");
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    std::vector<PreparedDispatch> prepared;
    prepared.reserve(runtimes.size());
    for (std::size_t i = 0; i < runtimes.size(); ++i)
        prepared.push_back(runtimes[i]->prepare_dispatch(xs[i], idxs[i], weights[i], alignment, expand, zero_padding,
                                                         cached[i], graph_pool));
    launch_dispatch_group(runtimes, prepared, device);
    std::vector<std::shared_ptr<DispatchResult>> results;
    for (auto& p : prepared) results.push_back(p.result);
    return results;
}

std::vector<at::Tensor> combine_group(const std::vector<std::shared_ptr<Runtime>>& runtimes,
                                      const std::vector<at::Tensor>& ys,
                                      const std::vector<std::shared_ptr<DispatchResult>>& results,
                                      bool weighted, int device) {
    if (ys.size() != runtimes.size() || results.size() != runtimes.size())
        throw std::invalid_argument("one input set per virtual rank");
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    std::vector<PreparedCombine> prepared;
    for (std::size_t i = 0; i < runtimes.size(); ++i)
        prepared.push_back(runtimes[i]->prepare_combine(ys[i], *results[i], weighted, std::nullopt));
    launch_combine_group(runtimes, prepared, device);
    std::vector<at::Tensor> outs;
    for (auto& p : prepared) outs.push_back(p.out);
    return outs;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "Blackwell expert-parallel dispatch/combine runtime";

    m.def("segment_layout", [](int P, int C, int E, int K, int H, int Tmax, int payload_slots, bool combine, bool fused) {
        return layout_to_dict(make_segment_layout(P, C, E, K, H, Tmax, payload_slots, combine, fused));
    }, py::arg("P"), py::arg("C"), py::arg("E"), py::arg("K"), py::arg("H"), py::arg("Tmax"), py::arg("payload_slots"),
       py::arg("combine"), py::arg("fused") = false);
    // dynamic shared memory one dispatch CTA needs with the given roles (no GPU needed: configuration checks and tests)
    m.def("dispatch_shared_bytes", [](int P, int C, int E, int K, int H, int Tmax, int payload_slots, int tx_warps, int rx_warps,
                                      bool bulk_engine, int stages, int send_ctas) {
        return dispatch_shared_bytes(make_segment_layout(P, C, E, K, H, Tmax, payload_slots, true, false), tx_warps, rx_warps, bulk_engine,
                                     stages, send_ctas);
    }, py::arg("P"), py::arg("C"), py::arg("E"), py::arg("K"), py::arg("H"), py::arg("Tmax"), py::arg("payload_slots"),
       py::arg("tx_warps"), py::arg("rx_warps"), py::arg("bulk_engine"), py::arg("stages"), py::arg("send_ctas"));
    m.def("allocate_device_segment", [](std::size_t bytes, int device) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        return reinterpret_cast<std::int64_t>(allocate_device_segment(bytes).ptr);
    });
    m.def("export_device_segment", [](std::int64_t ptr) { return py::bytes(export_device_segment(reinterpret_cast<void*>(ptr))); });
    m.def("import_device_segment", [](const std::string& handle, int device) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        return reinterpret_cast<std::int64_t>(import_device_segment(handle));
    });
    m.def("release_imported_segment", [](std::int64_t ptr) { release_imported_segment(reinterpret_cast<void*>(ptr)); });
    m.def("free_device_segment", [](std::int64_t ptr) { free_device_segment(reinterpret_cast<void*>(ptr)); });
    m.def("get_device_numa_node", &device_numa_node);
    m.def("query_numa_pages", [](std::int64_t address, std::size_t bytes) {
        py::dict out;
        for (const auto& [node, pages] : query_numa_pages(static_cast<std::uintptr_t>(address), bytes)) out[py::int_(node)] = pages;
        return out;
    }, py::arg("address"), py::arg("bytes"));
    m.def("create_host_segment", &create_host_segment);
    m.def("first_touch_host_segment", &first_touch_host_segment);
    m.def("tensor_refs", [](const at::Tensor& t) {
        const TensorRefs r = tensor_refs(t);
        return py::make_tuple(r.tensor_use_count, r.storage_use_count);
    });

    py::class_<HostSegment, std::shared_ptr<HostSegment>>(m, "HostSegment")
        .def(py::init<const std::string&, std::size_t, int>())
        .def("host_pointer", &HostSegment::host_pointer)
        .def("device_pointer", &HostSegment::device_pointer)
        .def("close", &HostSegment::close);

    py::class_<NumaRelay, std::shared_ptr<NumaRelay>>(m, "NumaRelay")
        // options: num_ranks, channels, num_experts, num_topk, hidden, num_max_tokens, payload_slots, enable_combine, and
        // optionally workers, cpu_affinity (list of allowed CPUs), target_numa_nodes (one per rank)
        .def(py::init([](const py::dict& options, const std::vector<std::int64_t>& outboxes, const std::vector<std::int64_t>& targets, int rank) {
            RelayOptions o;
            o.num_ranks = options["num_ranks"].cast<int>();
            o.channels = options["channels"].cast<int>();
            o.num_experts = options["num_experts"].cast<int>();
            o.num_topk = options["num_topk"].cast<int>();
            o.hidden = options["hidden"].cast<int>();
            o.num_max_tokens = options["num_max_tokens"].cast<int>();
            o.payload_slots = options["payload_slots"].cast<int>();
            o.enable_combine = options["enable_combine"].cast<bool>();
            if (options.contains("workers")) o.workers = options["workers"].cast<int>();
            if (options.contains("cpu_affinity")) o.cpu_affinity = options["cpu_affinity"].cast<std::vector<int>>();
            if (options.contains("target_numa_nodes")) o.target_numa_nodes = options["target_numa_nodes"].cast<std::vector<int>>();
            return std::make_shared<NumaRelay>(o, outboxes, targets, rank);
        }))
        .def("start", &NumaRelay::start)
        .def("stop", &NumaRelay::stop, py::call_guard<py::gil_scoped_release>())
        .def("diagnostics", [](const NumaRelay& relay) {
            py::dict d;
            py::list flows;
            for (const RelayFlowState& flow : relay.flow_states()) {
                py::dict f;
                f["dest"] = flow.dest;
                f["rows_copied"] = flow.rows_copied;
                f["bytes_copied"] = flow.bytes_copied;
                f["counts_epoch"] = flow.counts_epoch;
                f["combine_rows_copied"] = flow.combine_rows_copied;
                f["failure"] = flow.failure;
                f["worker_cpu"] = flow.worker_cpu;
                f["numa_node"] = flow.numa_node;
                f["acks_forwarded"] = flow.acks_forwarded;
                f["credit_waits"] = flow.credit_waits;
                f["drained_epoch"] = flow.drained_epoch;
                flows.append(f);
            }
            d["flows"] = flows;
            d["workers"] = relay.worker_count();
            d["running"] = relay.running();
            d["ring_mode"] = relay.ring_mode();
            return d;
        })
        .def("set_delay_ns", &NumaRelay::set_delay_ns);

    py::class_<Layout, std::shared_ptr<Layout>>(m, "_Layout")
        .def_readonly("num_tokens", &Layout::num_tokens)
        .def_readonly("alignment", &Layout::alignment)
        .def_readonly("expand", &Layout::expand)
        .def_readonly("valid", &Layout::valid)
        .def_readonly("mask", &Layout::mask)
        .def_readonly("slot", &Layout::slot)
        .def_readonly("expert_ord", &Layout::expert_ord)
        .def_readonly("counts", &Layout::counts);

    py::class_<DispatchResult, std::shared_ptr<DispatchResult>>(m, "DispatchResult")
        .def("__getitem__", &DispatchResult::get)
        .def("__setitem__", &DispatchResult::set)
        .def("__contains__", &DispatchResult::contains)
        .def("keys", &DispatchResult::keys)
        .def("get", [](DispatchResult& r, const std::string& key, py::object fallback) {
            return r.contains(key) ? r.get(key) : fallback;
        }, py::arg("key"), py::arg("default") = py::none());

    py::class_<Runtime, std::shared_ptr<Runtime>>(m, "Runtime")
        .def(py::init<int, int, int, int, int, int, const py::dict&, const std::vector<std::int64_t>&, int>())
        .def("dispatch", &Runtime::dispatch, py::arg("x"), py::arg("topk_idx"), py::arg("topk_weights"),
             py::arg("alignment"), py::arg("expand"), py::arg("zero_padding"), py::arg("cached"), py::arg("graph_pool"),
             py::arg("stream") = 0)
        .def("combine", &Runtime::combine, py::arg("y"), py::arg("dispatch_result"), py::arg("weighted"), py::arg("out"),
             py::arg("stream") = 0, py::arg("num_sms") = 0)
        .def("fused_scatter_gemm", &Runtime::fused_scatter_gemm, py::arg("hidden_rows"), py::arg("w_down"),
             py::arg("dispatch_result"), py::arg("stream") = 0)
        .def("fused_reduce", &Runtime::fused_reduce, py::arg("dispatch_result"), py::arg("out"), py::arg("stream") = 0)
        .def("fused_status", &Runtime::fused_status)
        .def("combine_is_split", &Runtime::combine_is_split)
        .def("combine_is_local", &Runtime::combine_is_local)
        .def("combine_is_inline", &Runtime::combine_is_inline)
        .def("send_stages", &Runtime::send_stages)
        .def("send_ctas", &Runtime::send_ctas)
        .def("grid_ctas", &Runtime::grid_ctas)
        .def("set_test_corrupt_sequence", &Runtime::set_test_corrupt_sequence)
        .def("set_test_control_abort_after_ns", &Runtime::set_test_control_abort_after_ns)
        .def("pool_debug", &Runtime::pool_debug)
        .def("set_test_delays", &Runtime::set_test_delays)
        .def("set_test_prefix_delay_ns", &Runtime::set_test_prefix_delay_ns)
        .def("set_test_skip_counts_ack_source", &Runtime::set_test_skip_counts_ack_source)
        .def("set_test_withhold_counts", &Runtime::set_test_withhold_counts)
        .def("set_timeout_ms", &Runtime::set_timeout_ms)
        .def("sticky_error", &Runtime::sticky_error)
        .def("epochs", &Runtime::epochs)
        .def("channels", &Runtime::channels)
        .def("threads", &Runtime::threads)
        .def("shared_bytes", &Runtime::shared_bytes)
        .def("uses_tma", &Runtime::uses_tma)
        .def("unique_capacity", &Runtime::unique_capacity)
        .def("expanded_capacity", &Runtime::expanded_capacity)
        .def("segment_layout", [](const Runtime& r) { return layout_to_dict(r.layout()); })
        .def("close", &Runtime::close);

    // out[rows of expert e] = a[rows of expert e] @ w[e].T (+ SwiGLU epilogue): tcgen05 grouped GEMM.
    // a and w are both bfloat16, or both float8_e4m3fn with a_scales [rows] and w_scales [experts, (2)n].
    m.def("grouped_gemm", [](const at::Tensor& a, const at::Tensor& w, at::Tensor& out, const at::Tensor& expert_offsets,
                             const at::Tensor& expert_counts, at::Tensor& status, bool swiglu,
                             const std::optional<at::Tensor>& a_scales, const std::optional<at::Tensor>& w_scales,
                             std::int64_t stream) {
        auto check = [](bool ok, const char* what) {
            if (!ok) throw std::invalid_argument(what);
        };
        check(a.is_cuda() && w.is_cuda() && out.is_cuda() && expert_offsets.is_cuda() && expert_counts.is_cuda() && status.is_cuda(),
              "all tensors must be CUDA tensors");
        const bool fp8 = a.scalar_type() == at::kFloat8_e4m3fn;
        check((fp8 || a.scalar_type() == at::kBFloat16) && w.scalar_type() == a.scalar_type() && out.scalar_type() == at::kBFloat16,
              "a and w must both be bfloat16 or both float8_e4m3fn; out must be bfloat16");
        check(a.dim() == 2 && w.dim() == 3 && out.dim() == 2 && a.is_contiguous() && w.is_contiguous() && out.is_contiguous(),
              "a [rows,k], w [experts,n(,x2),k], out [rows,n] must be contiguous");
        const int experts = static_cast<int>(w.size(0));
        const int k = static_cast<int>(a.size(1));
        const int n = static_cast<int>(out.size(1));
        check(w.size(2) == k && w.size(1) == (swiglu ? 2 : 1) * n && out.size(0) == a.size(0), "shape mismatch between a, w and out");
        check(expert_offsets.scalar_type() == at::kInt && expert_counts.scalar_type() == at::kInt &&
                  expert_offsets.numel() >= experts + 1 && expert_counts.numel() >= experts &&
                  expert_offsets.is_contiguous() && expert_counts.is_contiguous(),
              "expert_offsets [experts+1] and expert_counts [experts] must be contiguous int32");
        check(status.scalar_type() == at::kInt && status.numel() >= 4, "status must be int32 [4]");
        const float* a_scale_ptr = nullptr;
        const float* w_scale_ptr = nullptr;
        if (fp8) {
            check(a_scales.has_value() && w_scales.has_value(), "fp8 operands need a_scales and w_scales");
            check(a_scales->is_cuda() && a_scales->scalar_type() == at::kFloat && a_scales->is_contiguous() &&
                      a_scales->numel() >= a.size(0),
                  "a_scales must be contiguous CUDA float32 [rows]");
            check(w_scales->is_cuda() && w_scales->scalar_type() == at::kFloat && w_scales->is_contiguous() &&
                      w_scales->numel() == w.size(0) * w.size(1),
                  "w_scales must be contiguous CUDA float32 [experts, n(,x2)]");
            a_scale_ptr = a_scales->data_ptr<float>();
            w_scale_ptr = w_scales->data_ptr<float>();
        }
        c10::cuda::CUDAGuard guard(a.device());
        cudaStream_t launch_stream = stream != 0 ? reinterpret_cast<cudaStream_t>(stream)
                                                 : at::cuda::getCurrentCUDAStream(a.get_device()).stream();
        const char* error = grouped_gemm(a.data_ptr(), w.data_ptr(), out.data_ptr(), a_scale_ptr, w_scale_ptr,
                                         expert_offsets.data_ptr<int>(), expert_counts.data_ptr<int>(), status.data_ptr<int>(),
                                         static_cast<int>(a.size(0)), experts, n, k, swiglu, fp8, launch_stream);
        if (error != nullptr) throw std::runtime_error(std::string("grouped_gemm: ") + error);
    }, py::arg("a"), py::arg("w"), py::arg("out"), py::arg("expert_offsets"), py::arg("expert_counts"), py::arg("status"),
       py::arg("swiglu"), py::arg("a_scales") = py::none(), py::arg("w_scales") = py::none(), py::arg("stream") = 0);

    m.def("litmus", [](std::int64_t mine, std::int64_t theirs, int role, int rounds, int words, at::Tensor& status,
                       int timeout_ms, int device, int method) {
        if (!status.is_cuda() || status.scalar_type() != at::kLong || status.numel() < (role < 0 ? 8 : 4))
            throw std::invalid_argument("status must be a CUDA int64 tensor with 4 (8 for both roles) elements");
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        const char* error = litmus_pingpong(reinterpret_cast<void*>(mine), reinterpret_cast<void*>(theirs), role, rounds, words,
                                            reinterpret_cast<long long*>(status.data_ptr<std::int64_t>()),
                                            static_cast<unsigned long long>(timeout_ms) * 1000000ull,
                                            at::cuda::getCurrentCUDAStream(device).stream(), method);
        if (error != nullptr) throw std::runtime_error(std::string("litmus: ") + error);
    }, py::arg("mine"), py::arg("theirs"), py::arg("role"), py::arg("rounds"), py::arg("words"), py::arg("status"),
       py::arg("timeout_ms"), py::arg("device"), py::arg("method") = 0);

    m.def("role_profiling_enabled", &role_profiling_enabled);
    m.def("dispatch_group", &dispatch_group);
    m.def("combine_group", &combine_group);
}
