// pybind11 module `deep_ep._C`: registers the host runtime (buffers, contexts, events, barrier,
// runtime knobs, sizing helpers). Counterpart of the reference's `csrc/python_api.cpp:18-74`.
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "buffers/bucket.hpp"
#include "buffers/engram.hpp"
#include "buffers/ep.hpp"
#include "buffers/pp.hpp"
#include "comm/barrier.hpp"
#include "comm/stream.hpp"
#include "runtime/device.hpp"
#include "runtime/jit.hpp"
#include "runtime/specialize.hpp"
#include "utils/event.hpp"

namespace py = pybind11;
using namespace deep_ep;

namespace {

// The reference compares a device-side call against a host wait that runs out; this is the hook
// the failure-detection test uses: a bounded wait on a flag nobody sets, then the status check.
void run_bounded_wait_probe(comm::Context& context, double timeout_secs) {
    EP_HOST_ASSERT(context.common_signals != nullptr and context.host_status_device != nullptr);
    const cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
    launch::bounded_wait_probe(context.common_signals, context.host_status_device,
                               static_cast<long long>(timeout_secs * 1e9), stream);
    CUDA_CHECK(cudaStreamSynchronize(stream));
}

void clear_status(comm::Context& context) {
    CUDA_CHECK(cudaDeviceSynchronize());
    if (context.host_status != nullptr) context.host_status->code = 0;
    if (context.common_signals != nullptr) CUDA_CHECK(cudaMemset(&context.common_signals->status, 0, sizeof(int)));
}

// Routing layout of a set of tokens without communication: (dst_buffer_slot_idx [T, k], num_tokens_per_rank [R],
// num_tokens_per_expert [E]). Scratch memory is a zero-filled torch allocation per call.
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> get_dispatch_layout(const torch::Tensor& topk_idx, int num_experts,
                                                                            int num_ranks, int num_sms) {
    EP_HOST_ASSERT(topk_idx.is_cuda() and topk_idx.dim() == 2 and topk_idx.is_contiguous() and topk_idx.scalar_type() == torch::kInt64);
    const auto int_options = torch::TensorOptions().dtype(torch::kInt32).device(topk_idx.device());
    auto slots = torch::empty({topk_idx.size(0), topk_idx.size(1)}, int_options);
    auto per_rank = torch::empty({num_ranks}, int_options);
    auto per_expert = torch::empty({num_experts}, int_options);
    auto scratch = torch::zeros({static_cast<int64_t>(sizeof(kernels::LayoutScratch))},
                                torch::TensorOptions().dtype(torch::kUInt8).device(topk_idx.device()));
    kernels::LayoutArgs args = {};
    args.topk_idx = topk_idx.data_ptr<int64_t>();
    args.num_tokens = static_cast<int>(topk_idx.size(0)), args.num_topk = static_cast<int>(topk_idx.size(1));
    args.num_experts = num_experts, args.num_ranks = num_ranks;
    args.dst_slot_idx = slots.data_ptr<int>(), args.num_tokens_per_rank = per_rank.data_ptr<int>();
    args.num_tokens_per_expert = per_expert.data_ptr<int>();
    args.scratch = reinterpret_cast<kernels::LayoutScratch*>(scratch.data_ptr());
    args.timeout_ns = 10ll * 1000000000ll, args.status = nullptr;
    launch::dispatch_layout(args, num_sms, c10::cuda::getCurrentCUDAStream());
    return {slots, per_rank, per_expert};
}

// Grouped GEMM over the expanded layout. mode 0: d[rows, n_out] = a[rows, k] * b[g, n, k]^T (optionally SwiGLU);
// mode 1: d[rows, n] = a[rows, k] * b[g, k, n]; mode 2: d[g, m, n] += a[rows, m]^T * b[rows, n] (fp32).
void grouped_gemm(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const torch::Tensor& psum,
                  const torch::Tensor& count, int mode, int epilogue, int num_sms, int alignment,
                  const std::optional<torch::Tensor>& row_scale, const std::optional<torch::Tensor>& keep, bool use_pairs,
                  const std::optional<torch::Tensor>& route) {
    using namespace kernels;
    EP_HOST_ASSERT(a.is_cuda() and b.is_cuda() and d.is_cuda() and a.is_contiguous() and b.is_contiguous() and d.is_contiguous());
    EP_HOST_ASSERT(a.scalar_type() == torch::kBFloat16 and b.scalar_type() == torch::kBFloat16 and a.dim() == 2 and b.dim() == 3);
    EP_HOST_ASSERT(psum.scalar_type() == torch::kInt32 and count.scalar_type() == torch::kInt32 and psum.numel() == count.numel());
    EP_HOST_ASSERT(psum.is_cuda() and count.is_cuda() and psum.is_contiguous() and count.is_contiguous());
    GroupedGemmArgs args = {};
    args.mode = mode, args.epilogue = epilogue, args.num_groups = static_cast<int>(psum.numel());
    args.psum = psum.data_ptr<int>(), args.count = count.data_ptr<int>();
    args.d = d.data_ptr(), args.status = nullptr, args.alignment = alignment;
    const int64_t rows = a.size(0), g = args.num_groups;
    if (route.has_value()) {
        // destination table of `EPBuffer.build_combine_route`: rows with an entry are stored there instead of `d`
        EP_HOST_ASSERT(epilogue == kEpilogueStore and route->is_cuda() and route->is_contiguous() and
                       route->scalar_type() == torch::kInt64 and route->numel() >= rows);
        args.route = reinterpret_cast<const unsigned long long*>(route->data_ptr<int64_t>());
    }
    if (row_scale.has_value()) {
        EP_HOST_ASSERT(epilogue != kEpilogueStore and row_scale->is_cuda() and row_scale->is_contiguous() and
                       row_scale->scalar_type() == torch::kFloat32 and row_scale->numel() == rows);
        args.row_scale = row_scale->data_ptr<float>();
    }
    if (epilogue == kEpilogueSwiGLUKeep) {
        EP_HOST_ASSERT(keep.has_value() and keep->is_cuda() and keep->is_contiguous() and keep->scalar_type() == torch::kBFloat16 and
                       keep->dim() == 2 and keep->size(0) == rows and keep->size(1) == b.size(1));
        args.d2 = keep->data_ptr();
    }
    int64_t b_rows, b_cols;
    if (mode == kModeForward) {
        EP_HOST_ASSERT(b.size(0) == g and b.size(2) == a.size(1));
        args.n = static_cast<int>(b.size(1)), args.k = static_cast<int>(a.size(1));
        b_rows = g * b.size(1), b_cols = b.size(2);
        const int64_t n_out = epilogue != kEpilogueStore ? args.n / 2 : args.n;
        EP_HOST_ASSERT(d.dim() == 2 and d.size(0) == rows and d.size(1) == n_out);
        // fp32 output (the accumulator as it is) only from the plain-store epilogue without a destination table
        EP_HOST_ASSERT(d.scalar_type() == torch::kBFloat16 or
                       (d.scalar_type() == torch::kFloat32 and epilogue == kEpilogueStore and not route.has_value()));
        args.out_fp32 = d.scalar_type() == torch::kFloat32;
        EP_HOST_ASSERT(args.k % 8 == 0);
    } else if (mode == kModeDgrad) {
        EP_HOST_ASSERT(b.size(0) == g and b.size(1) == a.size(1) and epilogue == kEpilogueStore);
        args.n = static_cast<int>(b.size(2)), args.k = static_cast<int>(a.size(1));
        b_rows = g * b.size(1), b_cols = b.size(2);
        EP_HOST_ASSERT(d.scalar_type() == torch::kBFloat16 and d.dim() == 2 and d.size(0) == rows and d.size(1) == args.n);
        EP_HOST_ASSERT(args.k % kGemmBlockK == 0);     // a K block must not run into the next expert's weight rows
    } else {
        EP_HOST_UNREACHABLE("use grouped_gemm_wgrad for mode 2");
    }
    launch::grouped_gemm(args, a.data_ptr(), rows, a.size(1), b.data_ptr(), b_rows, b_cols, num_sms, c10::cuda::getCurrentCUDAStream(),
                         use_pairs);
}

// d = (a * a_sf) x (b * b_sf)^T per expert with e4m3 operands: a [rows, k] + a_sf [rows, k / 128], b [g, n, k] + b_sf [g, n / 128, k / 128].
// epilogue 0: d bf16 [rows, n]. epilogue 1 (SwiGLU over [gate | up] = n columns): d bf16 [rows, n / 2], or, when `d_sf` is
// given, d e4m3 [rows, n / 2] with d_sf [rows, n / 256] (re-quantised for the next GEMM).
// Scales are either all fp32 or all uint8 (UE8M0 bytes, value 2^(byte - 127)); the latter run on the hardware-scaled kernel.
void grouped_gemm_fp8(const torch::Tensor& a, const torch::Tensor& a_sf, const torch::Tensor& b, const torch::Tensor& b_sf,
                      const torch::Tensor& d, const torch::Tensor& psum, const torch::Tensor& count, int epilogue, int num_sms,
                      int alignment, const std::optional<torch::Tensor>& row_scale, const std::optional<torch::Tensor>& d_sf,
                      bool reg_split, const std::optional<torch::Tensor>& route) {
    using namespace kernels;
    for (const auto* t : {&a, &a_sf, &b, &b_sf, &d, &psum, &count}) EP_HOST_ASSERT(t->is_cuda() and t->is_contiguous());
    EP_HOST_ASSERT(a.scalar_type() == torch::kFloat8_e4m3fn and b.scalar_type() == torch::kFloat8_e4m3fn and a.dim() == 2 and b.dim() == 3);
    // fp32 weight scales -> promotion in registers; uint8 weight scales -> UE8M0 bytes applied by the tensor core, with the
    // activation scales as UE8M0 bytes too or as fp32 powers of two (what a power-of-two FP8 dispatch delivers)
    const bool hw_scales = b_sf.scalar_type() == torch::kUInt8;
    EP_HOST_ASSERT(hw_scales or (b_sf.scalar_type() == torch::kFloat32 and a_sf.scalar_type() == torch::kFloat32));
    EP_HOST_ASSERT(a_sf.scalar_type() == torch::kUInt8 ? hw_scales : a_sf.scalar_type() == torch::kFloat32);
    EP_HOST_ASSERT(psum.scalar_type() == torch::kInt32 and count.scalar_type() == torch::kInt32 and psum.numel() == count.numel());
    EP_HOST_ASSERT(epilogue == kEpilogueStore or epilogue == kEpilogueSwiGLU);
    const int64_t rows = a.size(0), k = a.size(1), g = psum.numel(), n = b.size(1);
    EP_HOST_ASSERT(b.size(0) == g and b.size(2) == k and k % kFp8BlockK == 0 and n % 128 == 0);
    EP_HOST_ASSERT(a_sf.dim() == 2 and a_sf.size(0) == rows and a_sf.size(1) == k / 128);
    EP_HOST_ASSERT(b_sf.dim() == 3 and b_sf.size(0) == g and b_sf.size(1) == n / 128 and b_sf.size(2) == k / 128);
    if (rows == 0) return;
    GroupedGemmFp8Args args = {};
    args.epilogue = epilogue, args.num_groups = static_cast<int>(g);
    args.psum = psum.data_ptr<int>(), args.count = count.data_ptr<int>();
    args.n = static_cast<int>(n), args.k = static_cast<int>(k), args.alignment = alignment;
    if (a_sf.scalar_type() == torch::kUInt8) args.sf_a_e8 = a_sf.data_ptr<uint8_t>();
    else args.sf_a = a_sf.data_ptr<float>();
    if (hw_scales) args.sf_b_e8 = b_sf.data_ptr<uint8_t>();
    else args.sf_b = b_sf.data_ptr<float>();
    args.d = d.data_ptr(), args.status = nullptr, args.reg_split = reg_split;
    const int64_t n_out = epilogue == kEpilogueStore ? n : n / 2;
    EP_HOST_ASSERT(d.dim() == 2 and d.size(0) == rows and d.size(1) == n_out);
    if (d_sf.has_value()) {
        EP_HOST_ASSERT(epilogue == kEpilogueSwiGLU and d.scalar_type() == torch::kFloat8_e4m3fn);
        EP_HOST_ASSERT(d_sf->is_cuda() and d_sf->is_contiguous() and d_sf->dim() == 2 and d_sf->size(0) == rows and
                       d_sf->size(1) == n_out / 128 and d_sf->scalar_type() == b_sf.scalar_type());
        args.out_fp8 = 1;
        if (hw_scales) args.d_sf_e8 = d_sf->data_ptr<uint8_t>();
        else args.d_sf = d_sf->data_ptr<float>();
    } else {
        EP_HOST_ASSERT(d.scalar_type() == torch::kBFloat16);
    }
    if (row_scale.has_value()) {
        EP_HOST_ASSERT(epilogue == kEpilogueSwiGLU and row_scale->is_cuda() and row_scale->is_contiguous() and
                       row_scale->scalar_type() == torch::kFloat32 and row_scale->numel() == rows);
        args.row_scale = row_scale->data_ptr<float>();
    }
    if (route.has_value()) {
        // destination table of `EPBuffer.build_combine_route` (hardware-scaled kernel, plain-store epilogue only)
        EP_HOST_ASSERT(hw_scales and epilogue == kEpilogueStore and route->is_cuda() and route->is_contiguous() and
                       route->scalar_type() == torch::kInt64 and route->numel() >= rows);
        args.route = reinterpret_cast<const unsigned long long*>(route->data_ptr<int64_t>());
    }
    launch::grouped_gemm_fp8(args, a.data_ptr(), rows, b.data_ptr(), g * n, num_sms, c10::cuda::getCurrentCUDAStream());
}

torch::Tensor swiglu_backward(const torch::Tensor& h, const torch::Tensor& dact, const std::optional<torch::Tensor>& row_scale) {
    EP_HOST_ASSERT(h.is_cuda() and h.is_contiguous() and h.scalar_type() == torch::kBFloat16 and h.dim() == 2);
    EP_HOST_ASSERT(dact.is_cuda() and dact.is_contiguous() and dact.scalar_type() == torch::kBFloat16 and dact.dim() == 2);
    EP_HOST_ASSERT(h.size(0) == dact.size(0) and h.size(1) == 2 * dact.size(1));
    if (row_scale.has_value())
        EP_HOST_ASSERT(row_scale->is_cuda() and row_scale->is_contiguous() and row_scale->scalar_type() == torch::kFloat32 and
                       row_scale->numel() == h.size(0));
    auto dh = torch::empty_like(h);
    launch::swiglu_backward(h.data_ptr(), dact.data_ptr(), row_scale.has_value() ? row_scale->data_ptr<float>() : nullptr,
                            dh.data_ptr(), h.size(0), static_cast<int>(dact.size(1)), c10::cuda::getCurrentCUDAStream());
    return dh;
}

// bf16 [rows, cols] -> (e4m3 [rows, cols], UE8M0 bytes [rows, cols / 128]): power-of-two scales, the operand format of
// the hardware-scaled FP8 GEMM
std::tuple<torch::Tensor, torch::Tensor> row_quant_ue8m0(const torch::Tensor& x) {
    EP_HOST_ASSERT(x.is_cuda() and x.is_contiguous() and x.scalar_type() == torch::kBFloat16 and x.dim() == 2 and x.size(1) % 128 == 0);
    auto q = torch::empty(x.sizes(), x.options().dtype(torch::kFloat8_e4m3fn));
    auto sf = torch::empty({x.size(0), x.size(1) / 128}, x.options().dtype(torch::kUInt8));
    launch::row_quant_ue8m0(x.data_ptr(), q.data_ptr(), sf.data_ptr(), x.size(0), static_cast<int>(x.size(1)),
                            c10::cuda::getCurrentCUDAStream());
    return {q, sf};
}

// h = [gate | up] bf16 [rows, 2 * inter] -> silu(gate) * up * row_scale as (bf16 or None, e4m3, UE8M0 bytes [rows, inter / 128])
std::tuple<std::optional<torch::Tensor>, torch::Tensor, torch::Tensor> swiglu_quant_ue8m0(
        const torch::Tensor& h, const std::optional<torch::Tensor>& row_scale, bool keep_bf16) {
    EP_HOST_ASSERT(h.is_cuda() and h.is_contiguous() and h.scalar_type() == torch::kBFloat16 and h.dim() == 2 and h.size(1) % 256 == 0);
    if (row_scale.has_value())
        EP_HOST_ASSERT(row_scale->is_cuda() and row_scale->is_contiguous() and row_scale->scalar_type() == torch::kFloat32 and
                       row_scale->numel() == h.size(0));
    const int64_t rows = h.size(0), inter = h.size(1) / 2;
    std::optional<torch::Tensor> act;
    if (keep_bf16) act = torch::empty({rows, inter}, h.options());
    auto q = torch::empty({rows, inter}, h.options().dtype(torch::kFloat8_e4m3fn));
    auto sf = torch::empty({rows, inter / 128}, h.options().dtype(torch::kUInt8));
    launch::swiglu_quant_ue8m0(h.data_ptr(), row_scale.has_value() ? row_scale->data_ptr<float>() : nullptr,
                               act.has_value() ? act->data_ptr() : nullptr, q.data_ptr(), sf.data_ptr(), rows,
                               static_cast<int>(inter), c10::cuda::getCurrentCUDAStream());
    return {act, q, sf};
}

// w bf16 [g, n, k] -> (e4m3 [g, n, k], UE8M0 [g, n / 128, k / 128]) and, with `transposed`, also
// (e4m3 [g, k, n], UE8M0 [g, k / 128, n / 128]): the same quantised values, every matrix transposed
std::vector<torch::Tensor> block_quant_ue8m0(const torch::Tensor& w, bool transposed) {
    EP_HOST_ASSERT(w.is_cuda() and w.is_contiguous() and w.scalar_type() == torch::kBFloat16 and w.dim() == 3);
    const int64_t g = w.size(0), n = w.size(1), k = w.size(2);
    EP_HOST_ASSERT(n % 128 == 0 and k % 128 == 0);
    const auto fp8 = w.options().dtype(torch::kFloat8_e4m3fn), u8 = w.options().dtype(torch::kUInt8);
    auto q = torch::empty({g, n, k}, fp8);
    auto sf = torch::empty({g, n / 128, k / 128}, u8);
    torch::Tensor qt, sft;
    if (transposed) qt = torch::empty({g, k, n}, fp8), sft = torch::empty({g, k / 128, n / 128}, u8);
    launch::block_quant_ue8m0(w.data_ptr(), q.data_ptr(), sf.data_ptr(), transposed ? qt.data_ptr() : nullptr,
                              transposed ? sft.data_ptr() : nullptr, g * n, static_cast<int>(k), static_cast<int>(n),
                              c10::cuda::getCurrentCUDAStream());
    if (transposed) return {q, sf, qt, sft};
    return {q, sf};
}

// d[g, m, n] (fp32) (+)= a[rows_e, m]^T * b[rows_e, n] for every expert e; padding rows of `a` or `b` must be zero.
void grouped_gemm_wgrad(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& d, const torch::Tensor& psum,
                        const torch::Tensor& count, int num_sms, bool accumulate, bool use_pairs) {
    using namespace kernels;
    EP_HOST_ASSERT(a.is_cuda() and b.is_cuda() and d.is_cuda() and a.is_contiguous() and b.is_contiguous() and d.is_contiguous());
    EP_HOST_ASSERT(a.scalar_type() == torch::kBFloat16 and b.scalar_type() == torch::kBFloat16 and a.dim() == 2 and b.dim() == 2);
    EP_HOST_ASSERT(a.size(0) == b.size(0) and d.dim() == 3);
    EP_HOST_ASSERT(d.scalar_type() == torch::kFloat32 or (d.scalar_type() == torch::kBFloat16 and not accumulate));
    EP_HOST_ASSERT(psum.scalar_type() == torch::kInt32 and count.scalar_type() == torch::kInt32 and psum.numel() == count.numel());
    GroupedGemmArgs args = {};
    args.mode = kModeWgrad, args.epilogue = kEpilogueStore, args.num_groups = static_cast<int>(psum.numel());
    args.accumulate = accumulate, args.out_bf16 = d.scalar_type() == torch::kBFloat16;
    args.psum = psum.data_ptr<int>(), args.count = count.data_ptr<int>();
    args.m = static_cast<int>(a.size(1)), args.n = static_cast<int>(b.size(1)), args.k = 0;
    EP_HOST_ASSERT(d.size(0) == args.num_groups and d.size(1) == args.m and d.size(2) == args.n);
    args.d = d.data_ptr(), args.status = nullptr;
    launch::grouped_gemm(args, a.data_ptr(), a.size(0), a.size(1), b.data_ptr(), b.size(0), b.size(1), num_sms,
                         c10::cuda::getCurrentCUDAStream(), use_pairs);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "deep_ep native runtime for NVIDIA B200 (sm_100a)";
    py::register_exception<EPException>(m, "EPException", PyExc_RuntimeError);

    m.attr("topk_idx_t") = py::reinterpret_borrow<py::object>(
        reinterpret_cast<PyObject*>(torch::getTHPDtype(c10::ScalarType::Long)));
    m.def("get_num_allocation_alignment", [] { return kNumAllocationAlignmentBytes; });
    m.def("get_num_rdma_alignment", [] { return kNumRDMAAlignmentBytes; });
    m.def("get_num_tma_alignment", [] { return kNumTMAAlignmentBytes; });
    m.attr("MAX_RANKS") = kMaxRanks;
    m.attr("MAX_BUCKETS") = kMaxBuckets;
    m.attr("MAX_CONTEXTS") = kMaxContexts;

    // runtime knobs
    m.def("get_num_sms", [] { return Runtime::get().get_num_sms(); });
    m.def("set_num_sms", [](int n) { Runtime::get().set_num_sms(n); });
    m.def("get_num_device_sms", [] { return Runtime::get().get_num_device_sms(); });
    m.def("get_arch", [] { return Runtime::get().get_arch(); });
    m.def("set_arch", [](const std::string& a) { Runtime::get().set_arch(a); });
    m.def("set_barrier_in_prologue", [](bool v) { return Runtime::get().set_barrier_in_prologue(v); });
    m.def("get_barrier_in_prologue", [] { return Runtime::get().get_barrier_in_prologue(); });
    m.def("set_warp_cooperation", [](bool v) { return Runtime::get().set_warp_cooperation(v); });
    m.def("get_warp_cooperation", [] { return Runtime::get().get_warp_cooperation(); });
    // names under which the reference exposes the same knobs (`csrc/runtime/jit.hpp:86-116` there): a "vector core"
    // corresponds to an SM here, there is no separate cube-core pool, and the architecture string is "sm_100a"
    m.def("get_num_vec_cores", [] { return Runtime::get().get_num_sms(); });
    m.def("set_num_vec_cores", [](int n) { Runtime::get().set_num_sms(n); });
    m.def("set_num_cube_cores", [](int) {});
    m.def("get_num_ai_cores", [] { return Runtime::get().get_num_device_sms(); });
    m.def("get_npu_arch", [] { return Runtime::get().get_arch(); });
    m.def("set_npu_arch", [](const std::string& a) { Runtime::get().set_arch(a); });
    jit::register_python_api(m);
    m.def("landing_range_ok", &layout::landing_range_ok, py::arg("offset"), py::arg("bytes"), py::arg("area_bytes"),
          "the predicate the bounds-checked kernels (EP_DEBUG) apply to every remote message store");
    jit::register_specialization_api(m);
    // Host-only self-test of the descriptor exchange used by the virtual-memory-management route: a pipe's two ends travel
    // through `FdServer` / `receive_fds` inside this process and must still be connected to each other afterwards.
    m.def("fd_exchange_selftest", [] {
        int ends[2];
        EP_HOST_ASSERT(::pipe(ends) == 0);
        bool ok = false;
        {
            comm::FdServer server({ends[0], ends[1]}, 1, 10);
            const auto received = comm::receive_fds(server.name, 2, 10);
            const char out = 'x';
            char in = 0;
            ok = ::write(received[1], &out, 1) == 1 and ::read(ends[0], &in, 1) == 1 and in == out and
                 received[0] != ends[0] and received[1] != ends[1];
            ::close(received[0]), ::close(received[1]);
        }
        ::close(ends[0]), ::close(ends[1]);
        return ok;
    });

    py::class_<EventHandle>(m, "EventHandle")
        .def(py::init<>())
        .def("current_stream_wait", &EventHandle::current_stream_wait);

    py::class_<comm::Context, std::shared_ptr<comm::Context>>(m, "Context")
        .def_readonly("rank_idx", &comm::Context::rank_idx)
        .def_readonly("num_ranks", &comm::Context::num_ranks)
        .def_readonly("context_idx", &comm::Context::context_idx)
        .def_readonly("num_workspace_bytes", &comm::Context::num_workspace_bytes)
        .def_readonly("num_gpu_buffer_bytes", &comm::Context::num_gpu_buffer_bytes)
        .def_readonly("num_rdma_storage_bytes", &comm::Context::num_rdma_storage_bytes)
        .def_readonly("peers_ready", &comm::Context::peers_ready)
        .def("get_local_handle", [](comm::Context& c) { return py::bytes(c.get_local_handle()); })
        .def("multicast_pending", &comm::Context::multicast_pending)
        .def("bind_multicast", &comm::Context::bind_multicast)
        .def("has_multicast", [](const comm::Context& c) { return c.peers.mc_base != nullptr; })
        .def("set_peer_handles", [](comm::Context& c, const std::vector<py::bytes>& handles) {
            std::vector<std::string> raw;
            for (const auto& h : handles) raw.emplace_back(static_cast<std::string>(h));
            c.set_peer_handles(raw);
        })
        .def("get_physical_domain_size", &comm::Context::get_physical_domain_size)
        .def("get_logical_domain_size", &comm::Context::get_logical_domain_size)
        .def("check_status", &comm::Context::check_status)
        .def("status_code", [](const comm::Context& c) { return c.host_status ? static_cast<int>(c.host_status->code) : 0; })
        .def("clear_status", &clear_status)
        .def("bounded_wait_probe", &run_bounded_wait_probe);

    m.def("barrier", [](comm::Context& context, bool with_cpu_sync, bool sequential, bool wait_comm_stream, int repeats) {
        comm::barrier(context, with_cpu_sync, sequential, wait_comm_stream, repeats);
    }, py::arg("context"), py::arg("with_cpu_sync") = false, py::arg("sequential") = true, py::arg("wait_comm_stream") = true,
       py::arg("repeats") = 1);
    m.def("get_comm_stream", [] {
        const auto s = comm::get_comm_stream();
        return py::make_tuple(s.id(), static_cast<int>(s.device_index()), static_cast<int>(s.device_type()));
    });
    m.def("check_peer_access", [](int device, int peer) {
        int ok = 0;
        CUDA_CHECK(cudaDeviceCanAccessPeer(&ok, device, peer));
        return ok != 0;
    });

    m.def("get_dispatch_layout", &get_dispatch_layout, py::arg("topk_idx"), py::arg("num_experts"), py::arg("num_ranks"),
          py::arg("num_sms") = 0);
    m.def("grouped_gemm", &grouped_gemm, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("psum"), py::arg("count"),
          py::arg("mode"), py::arg("epilogue") = 0, py::arg("num_sms") = 0, py::arg("alignment") = 1,
          py::arg("row_scale") = py::none(), py::arg("keep") = py::none(), py::arg("use_pairs") = false,
          py::arg("route") = py::none());
    m.def("grouped_gemm_fp8", &grouped_gemm_fp8, py::arg("a"), py::arg("a_sf"), py::arg("b"), py::arg("b_sf"), py::arg("d"),
          py::arg("psum"), py::arg("count"), py::arg("epilogue") = 0, py::arg("num_sms") = 0, py::arg("alignment") = 1,
          py::arg("row_scale") = py::none(), py::arg("d_sf") = py::none(), py::arg("reg_split") = true,
          py::arg("route") = py::none());
    m.def("swiglu_backward", &swiglu_backward, py::arg("h"), py::arg("dact"), py::arg("row_scale") = py::none());
    m.def("row_quant_ue8m0", &row_quant_ue8m0, py::arg("x"));
    m.def("swiglu_quant_ue8m0", &swiglu_quant_ue8m0, py::arg("h"), py::arg("row_scale") = py::none(), py::arg("keep_bf16") = true);
    m.def("block_quant_ue8m0", &block_quant_ue8m0, py::arg("w"), py::arg("transposed") = false);
    m.def("grouped_gemm_wgrad", &grouped_gemm_wgrad, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("psum"), py::arg("count"),
          py::arg("num_sms") = 0, py::arg("accumulate") = true, py::arg("use_pairs") = false);

    py::class_<BufferBase, std::shared_ptr<BufferBase>>(m, "BufferBase")
        .def_readonly("main_context", &BufferBase::main_context)
        .def("print_memory_usage", &BufferBase::print_memory_usage)
        .def("close_peer_mappings", &BufferBase::close_peer_mappings)
        .def("abort", &BufferBase::abort)
        .def("destroy", &BufferBase::destroy);

    py::class_<EPBuffer, BufferBase, std::shared_ptr<EPBuffer>>(m, "EPBuffer")
        .def(py::init<int, int, const std::string&, int64_t, int64_t, bool, int, int, bool>())
        .def_readonly("context", &EPBuffer::context)
        .def_readonly("lb_storage", &EPBuffer::lb_storage)
        .def("dispatch", &EPBuffer::dispatch)
        .def("combine", &EPBuffer::combine)
        .def("build_combine_route", &EPBuffer::build_combine_route)
        .def("enable_phase_trace", &EPBuffer::enable_phase_trace)
        .def("disable_phase_trace", &EPBuffer::disable_phase_trace)
        .def("lb_prefetch_weights", &EPBuffer::lb_prefetch_weights)
        .def("lb_reduce_grads", &EPBuffer::lb_reduce_grads)
        .def("check_status", &EPBuffer::check_status);
    m.def("calculate_ep_buffer_size", &EPBuffer::calculate_buffer_size);

    py::class_<PPBuffer, BufferBase, std::shared_ptr<PPBuffer>>(m, "PPBuffer")
        .def(py::init<int, int, const std::string&, int64_t, int, bool, int, bool>())
        .def_readonly("context", &PPBuffer::context)
        .def_readonly("storage", &PPBuffer::storage)
        .def("send", &PPBuffer::send)
        .def("recv", &PPBuffer::recv);

    py::class_<EngramBuffer, BufferBase, std::shared_ptr<EngramBuffer>>(m, "EngramBuffer")
        .def(py::init<int, int, const std::string&, int64_t, int64_t, bool, int, bool>())
        .def_readonly("context", &EngramBuffer::context)
        .def("set_config", &EngramBuffer::set_config)
        .def("write", &EngramBuffer::write)
        .def("fetch", &EngramBuffer::fetch);

    py::class_<BucketBuffer, BufferBase, std::shared_ptr<BucketBuffer>>(m, "BucketBuffer")
        .def(py::init<const std::vector<int>&, const std::vector<int>&, const std::vector<std::string>&, int64_t, bool, int, bool>())
        .def_readonly("contexts", &BucketBuffer::contexts)
        .def_readonly("storage", &BucketBuffer::storage)
        .def("all_gather", &BucketBuffer::all_gather)
        .def("reduce", &BucketBuffer::reduce, py::arg("srcs"), py::arg("context_idx"), py::arg("num_sms"), py::arg("scale"),
             py::arg("all_reduce"));
}
