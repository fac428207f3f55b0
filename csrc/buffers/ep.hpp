// Host side of the expert-parallel buffer: argument validation, tensor allocation, kernel launches,
// the host count handshake and the deferred epilogue closures. Counterpart of the reference's
// `csrc/buffers/ep.hpp:27-606`; the tuple shapes returned to Python follow it so that the Python
// `EPBuffer`/`EPHandle` layer sees the same contract.
#pragma once

#include <c10/cuda/CUDAStream.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <atomic>
#include <chrono>
#include <functional>
#include <optional>
#include <thread>
#include <vector>

#include <deep_ep/layout/ep.hpp>

#include "../comm/barrier.hpp"
#include "../kernels/api.hpp"
#include "../runtime/device.hpp"
#include "../utils/event.hpp"
#include "base.hpp"

namespace deep_ep {

class EPBuffer : public BufferBase, public std::enable_shared_from_this<EPBuffer> {
    // A deferred epilogue that has been handed out and neither run nor dropped yet. The epilogue kernels read the
    // buffer's CURRENT epoch, the landing area and (with the host count handshake) the one shared block of host counts,
    // so a second operation of the same kind must not be issued before the first one's epilogue has been enqueued.
    struct EpilogueTicket {
        int* pending;
        bool released = false;
        explicit EpilogueTicket(int* pending) : pending(pending) { ++*pending; }
        void release() { if (not released) released = true, --*pending; }
        ~EpilogueTicket() { release(); }
    };
    int pending_dispatch_epilogues = 0, pending_combine_epilogues = 0;

    layout::EPHostCounts* host_counts = nullptr;          // host view of the mapped pinned block
    layout::EPHostCounts* host_counts_device = nullptr;   // device view

    layout::EPSignals* signals() const { return static_cast<layout::EPSignals*>(context->workspace); }

    // optional phase trace: 4 kernels x kTraceSlots `%globaltimer` stamps (dispatch, expand, combine, reduce)
    torch::Tensor phase_trace;
    unsigned long long* trace_of(int kernel) const {
        return phase_trace.defined() ? reinterpret_cast<unsigned long long*>(phase_trace.data_ptr<int64_t>()) + kernel * kernels::kTraceSlots
                                     : nullptr;
    }

    void release_without_barrier() override {
        if (host_counts != nullptr) cudaFreeHost(host_counts), host_counts = nullptr;
        if (context != nullptr) context->finalize(), context = nullptr;
        destroyed = true;
    }

    // Spin on a tagged word in mapped host memory until its epoch half is non-zero.
    uint32_t host_wait_tagged(const volatile unsigned long long* word,
                              const std::chrono::steady_clock::time_point& deadline) const {
        int spins = 0;
        while (true) {
            const unsigned long long w = *word;
            if (layout::tagged_epoch(w) != 0) {
                std::atomic_thread_fence(std::memory_order_acquire);
                return layout::tagged_value(w);
            }
            if ((++spins & 1023) == 0) {
                if (host_counts->status.code != 0) throw_device_status();
                if (std::chrono::steady_clock::now() > deadline)
                    throw EPException("Host wait", __FILE__, __LINE__, "reduction timeout: dispatch counts did not arrive");
                std::this_thread::yield();
            }
        }
    }

    void throw_device_status() const {
        const auto& s = host_counts->status;
        throw EPException("Device status", __FILE__, __LINE__,
                          "kernel reported code " + std::to_string(s.code) + " on rank " + std::to_string(s.rank) +
                          " waiting for rank " + std::to_string(s.peer) + " at site " + std::to_string(s.where) +
                          " (expected " + std::to_string(s.expected) + ", observed " + std::to_string(s.observed) + ")");
    }

public:
    std::shared_ptr<comm::Context> context;
    int64_t num_bytes, num_lb_bytes;
    torch::Tensor lb_storage;
    torch::Tensor gsge_constant;      // all -1, shape of the last dispatch's `dst_gsge_idx`

    EPBuffer(int rank_idx, int num_ranks, const std::string& comm_name, int64_t num_bytes, int64_t num_lb_bytes,
             bool use_huge1g_page, int num_cpu_timeout_secs, int num_gpu_timeout_secs, bool explicitly_destroy)
        : BufferBase(explicitly_destroy), num_bytes(num_bytes), num_lb_bytes(num_lb_bytes) {
        (void) use_huge1g_page;
        EP_HOST_ASSERT(num_bytes >= 0 and num_lb_bytes >= 0);
        context = std::make_shared<comm::Context>(comm_name, rank_idx, num_ranks, layout::kEPWorkspaceBytes,
                                                  num_bytes + num_lb_bytes, 0, num_cpu_timeout_secs, num_gpu_timeout_secs);
        main_context = context;
        context->set_common_signals(&signals()->common);

        void* host = nullptr;
        CUDA_CHECK(cudaHostAlloc(&host, sizeof(layout::EPHostCounts), cudaHostAllocMapped));
        std::memset(host, 0, sizeof(layout::EPHostCounts));
        host_counts = static_cast<layout::EPHostCounts*>(host);
        void* device_view = nullptr;
        CUDA_CHECK(cudaHostGetDevicePointer(&device_view, host, 0));
        host_counts_device = static_cast<layout::EPHostCounts*>(device_view);

        auto options = torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, c10::cuda::current_device());
        lb_storage = num_lb_bytes > 0
            ? torch::from_blob(static_cast<uint8_t*>(context->buffer) + num_bytes, {num_lb_bytes}, [ctx = context](void*) {}, options)
            : torch::empty({0}, options);
    }

    ~EPBuffer() override { destroy_on_destruction("EP"); }

    void destroy() override {
        EP_HOST_ASSERT(not destroyed);
        comm::barrier(*context, /*with_cpu_sync=*/true);
        release_without_barrier();
    }

    // ------------------------------------------------------------------------------ sizing
    static int num_sf_bytes_hint(int hidden, bool use_fp8) { return use_fp8 ? math::ceil_div(hidden, 32) * 2 : 0; }

    static int64_t get_dispatch_buffer_size(int num_max_tokens_per_rank, int hidden_bytes, int sf_bytes, int num_topk, int num_ranks) {
        return layout::BufferLayout(layout::DispatchTokenLayout(hidden_bytes, sf_bytes, num_topk).num_bytes(),
                                    num_ranks, num_max_tokens_per_rank).num_bytes();
    }
    static int64_t get_combine_buffer_size(int num_ranks, int num_max_tokens_per_rank, int hidden, int num_topk) {
        return layout::BufferLayout(layout::CombineTokenLayout(hidden * 2, num_topk).num_bytes(),
                                    std::min(num_topk, num_ranks), num_max_tokens_per_rank).num_bytes();
    }
    // max(dispatch, combine) landing area, 2 MiB aligned; `num_topk == 0` reserves the maximum top-k.
    static int64_t calculate_buffer_size(int num_ranks, int num_max_tokens_per_rank, int hidden, int num_topk, bool use_fp8_dispatch) {
        EP_HOST_ASSERT(num_ranks > 0 and num_max_tokens_per_rank > 0 and hidden > 0 and num_topk >= 0);
        num_topk = num_topk == 0 ? kMaxTopk : num_topk;
        const auto dispatch_bytes = get_dispatch_buffer_size(num_max_tokens_per_rank, hidden * (use_fp8_dispatch ? 1 : 2),
                                                             num_sf_bytes_hint(hidden, use_fp8_dispatch), num_topk, num_ranks);
        const auto combine_bytes = get_combine_buffer_size(num_ranks, num_max_tokens_per_rank, hidden, num_topk);
        return math::align(std::max(dispatch_bytes, combine_bytes), kNumAllocationAlignmentBytes);
    }

    // ------------------------------------------------------------------------------ dispatch
    pybind11::tuple dispatch(const torch::Tensor& x, const std::optional<torch::Tensor>& sf,
                             const torch::Tensor& topk_idx, const std::optional<torch::Tensor>& topk_weights,
                             const std::optional<torch::Tensor>& cumulative_local_expert_recv_stats,
                             const std::optional<int>& cached_num_recv_tokens,
                             const std::optional<int>& cached_num_expanded_tokens,
                             const std::optional<std::vector<int>>& cached_num_recv_tokens_per_expert_list,
                             const std::optional<torch::Tensor>& cached_psum_num_recv_tokens_per_rank,
                             const std::optional<torch::Tensor>& cached_psum_num_recv_tokens_per_expert,
                             const std::optional<torch::Tensor>& cached_num_unaligned_recv_tokens_per_expert,
                             const std::optional<torch::Tensor>& cached_dst_buffer_slot_idx,
                             const std::optional<torch::Tensor>& cached_dst_gsge_idx,
                             const std::optional<torch::Tensor>& cached_recv_src_metadata,
                             int num_max_tokens_per_rank, int num_experts, int expert_alignment, int num_sms,
                             const std::optional<EventHandle>& previous_event,
                             bool async_with_compute_stream, bool allocate_on_comm_stream,
                             bool do_handle_copy, bool do_cpu_sync, bool do_expand, bool do_zero_padding,
                             bool use_col_major_sf, bool defer_epilogue, int fused_fp8_quant) {
        EP_HOST_ASSERT(not destroyed and context->peers_ready);
        EP_HOST_ASSERT(do_expand and not do_handle_copy);
        EP_HOST_ASSERT_MSG(pending_dispatch_epilogues == 0,
                           "the deferred epilogue of the previous dispatch on this buffer has not been run yet: call its hook "
                           "(`current_stream_wait()`) before the next dispatch");
        (void) allocate_on_comm_stream;
        const bool cached_mode = cached_recv_src_metadata.has_value();
        const int num_ranks = context->num_ranks;
        const auto device = x.device();

        // ---- validation
        EP_HOST_ASSERT(x.dim() == 2 and x.is_contiguous() and x.is_cuda());
        const int num_tokens = static_cast<int>(x.size(0)), hidden = static_cast<int>(x.size(1));
        EP_HOST_ASSERT(num_experts > 0 and num_experts % num_ranks == 0 and num_experts <= kMaxExperts);
        const int num_local_experts = num_experts / num_ranks;
        EP_HOST_ASSERT(num_local_experts <= kMaxLocalExperts);
        EP_HOST_ASSERT(math::is_pow2(expert_alignment));
        EP_HOST_ASSERT(num_tokens <= num_max_tokens_per_rank and num_max_tokens_per_rank > 0);
        EP_HOST_ASSERT(topk_idx.dim() == 2 and topk_idx.is_contiguous() and topk_idx.scalar_type() == torch::kInt64);
        EP_HOST_ASSERT(topk_idx.size(0) == num_tokens and topk_idx.device() == device);
        const int num_topk = static_cast<int>(topk_idx.size(1));
        EP_HOST_ASSERT(1 <= num_topk and num_topk <= kMaxTopk);
        if (topk_weights.has_value()) {
            EP_HOST_ASSERT(topk_weights->dim() == 2 and topk_weights->is_contiguous() and topk_weights->scalar_type() == torch::kFloat32);
            EP_HOST_ASSERT(topk_weights->size(0) == num_tokens and topk_weights->size(1) == num_topk);
        }
        if (cached_mode) {
            EP_HOST_ASSERT(not do_cpu_sync and not cumulative_local_expert_recv_stats.has_value());
            EP_HOST_ASSERT(cached_num_recv_tokens.has_value() and cached_num_expanded_tokens.has_value() and
                           cached_psum_num_recv_tokens_per_rank.has_value() and cached_psum_num_recv_tokens_per_expert.has_value() and
                           cached_num_unaligned_recv_tokens_per_expert.has_value() and cached_dst_buffer_slot_idx.has_value());
        }
        if (cumulative_local_expert_recv_stats.has_value()) {
            EP_HOST_ASSERT(cumulative_local_expert_recv_stats->scalar_type() == torch::kInt32 and
                           cumulative_local_expert_recv_stats->numel() == num_local_experts and
                           cumulative_local_expert_recv_stats->is_contiguous());
        }

        // wire element type and scale factors
        int hidden_bytes, sf_bytes = 0;
        int64_t sf_token_stride = 0, sf_pack_stride = 0;
        int num_sf_packs = 0;
        auto wire_dtype = x.scalar_type();
        // 0: `x` is sent as given; 1: bf16 `x` is quantised in the kernel (fp32 scales amax / 448); 2: the same with the
        // scales rounded up to powers of two
        EP_HOST_ASSERT(fused_fp8_quant >= 0 and fused_fp8_quant <= 2);
        if (fused_fp8_quant) {
            EP_HOST_ASSERT(x.scalar_type() == torch::kBFloat16 and not sf.has_value() and hidden % 128 == 0);
            hidden_bytes = hidden, num_sf_packs = hidden / 128 * 2, sf_bytes = num_sf_packs * 2;
            wire_dtype = torch::kFloat8_e4m3fn;
        } else if (sf.has_value()) {
            EP_HOST_ASSERT(x.element_size() == 1);
            EP_HOST_ASSERT(sf->dim() == 2 and sf->size(0) == num_tokens and sf->element_size() == 2 and sf->device() == device);
            num_sf_packs = static_cast<int>(sf->size(1));
            sf_token_stride = sf->stride(0), sf_pack_stride = sf->stride(1);
            EP_HOST_ASSERT((sf_pack_stride == 1 and sf_token_stride == num_sf_packs) or
                           (sf_token_stride == 1 and sf_pack_stride == num_tokens) or num_tokens <= 1 or num_sf_packs <= 1);
            hidden_bytes = hidden, sf_bytes = num_sf_packs * 2;
        } else {
            EP_HOST_ASSERT(x.scalar_type() == torch::kBFloat16);
            hidden_bytes = hidden * 2;
        }
        EP_HOST_ASSERT_MSG(hidden_bytes % 16 == 0, "rows must be a multiple of 16 bytes for bulk copies");
        const layout::DispatchTokenLayout token_layout(hidden_bytes, sf_bytes, num_topk);
        EP_HOST_ASSERT_MSG(get_dispatch_buffer_size(num_max_tokens_per_rank, hidden_bytes, sf_bytes, num_topk, num_ranks) <= num_bytes,
                           "EP buffer too small for this dispatch");
        EP_HOST_ASSERT(static_cast<int64_t>(num_max_tokens_per_rank) * num_ranks < (1ll << 31));

        // ---- handle tensors
        const auto int_options = torch::TensorOptions().dtype(torch::kInt32).device(device);
        auto psum_rank = cached_mode ? *cached_psum_num_recv_tokens_per_rank : torch::empty({num_ranks}, int_options);
        auto psum_expert = cached_mode ? *cached_psum_num_recv_tokens_per_expert : torch::empty({num_local_experts}, int_options);
        auto num_unaligned = cached_mode ? *cached_num_unaligned_recv_tokens_per_expert : torch::empty({num_local_experts}, int_options);
        auto dst_buffer_slot_idx = cached_mode ? *cached_dst_buffer_slot_idx : torch::empty({num_tokens, num_topk}, int_options);
        // no scatter-gather bookkeeping exists on NVLink; the tensor is kept (all -1) for API shape
        // (the tensor is never written, so one instance per shape is shared by all handles)
        if (not cached_mode and (not gsge_constant.defined() or gsge_constant.size(0) != num_tokens or
                                 gsge_constant.size(1) != num_topk or gsge_constant.device() != device))
            gsge_constant = torch::full({num_tokens, num_topk}, -1, int_options);
        auto dst_gsge_idx = cached_mode and cached_dst_gsge_idx.has_value() ? *cached_dst_gsge_idx : gsge_constant;
        if (cached_mode) {
            EP_HOST_ASSERT(dst_buffer_slot_idx.size(0) == num_tokens and dst_buffer_slot_idx.size(1) == num_topk and
                           dst_buffer_slot_idx.is_contiguous() and dst_buffer_slot_idx.scalar_type() == torch::kInt32);
            EP_HOST_ASSERT(psum_rank.numel() == num_ranks and psum_expert.numel() == num_local_experts);
        }

        const auto stream = c10::cuda::getCurrentCUDAStream();
        if (previous_event.has_value()) previous_event->current_stream_wait();
        const bool barrier_in_prologue = Runtime::get().get_barrier_in_prologue();
        if (num_sms <= 0) num_sms = Runtime::get().get_num_sms();

        if (do_cpu_sync) {
            host_counts->num_recv_tokens = 0;
            host_counts->num_expanded_tokens = 0;
            std::atomic_thread_fence(std::memory_order_seq_cst);
        }

        kernels::DispatchArgs args = {};
        args.x = static_cast<const uint8_t*>(x.data_ptr());
        args.sf = sf.has_value() ? static_cast<const sf_pack_t*>(sf->data_ptr()) : nullptr;
        args.sf_token_stride = sf_token_stride, args.sf_pack_stride = sf_pack_stride;
        args.topk_idx = topk_idx.data_ptr<int64_t>();
        args.topk_weights = topk_weights.has_value() ? topk_weights->data_ptr<float>() : nullptr;
        args.num_tokens = num_tokens, args.hidden_bytes = hidden_bytes, args.sf_bytes = sf_bytes, args.num_topk = num_topk;
        args.num_experts = num_experts, args.num_max_tokens = num_max_tokens_per_rank, args.expert_alignment = expert_alignment;
        args.cached = cached_mode, args.fused_quant = fused_fp8_quant, args.do_cpu_sync = do_cpu_sync;
        args.wait_arrival = barrier_in_prologue;
        args.dst_slot_idx = dst_buffer_slot_idx.data_ptr<int>();
        args.psum_rank = psum_rank.data_ptr<int>(), args.psum_expert = psum_expert.data_ptr<int>();
        args.num_unaligned = num_unaligned.data_ptr<int>();
        args.cumulative_stats = cumulative_local_expert_recv_stats.has_value() ? cumulative_local_expert_recv_stats->data_ptr<int>() : nullptr;
        args.ws = signals(), args.buffer_offset = context->num_workspace_bytes, args.buffer_bytes = num_bytes, args.peers = context->peers;
        args.host = host_counts_device, args.timeout_ns = context->num_gpu_timeout_ns;
        args.trace = trace_of(0);
        launch::dispatch(args, num_sms, stream);

        // ---- epilogue (possibly deferred): sizes, outputs, expand kernel. The closure keeps the
        // inputs and the context alive until the expand kernel has been enqueued.
        // the closure keeps the buffer itself alive (a hook may outlive the Python object that created it)
        auto epilogue = [=, this, self = shared_from_this(), ticket = std::make_shared<EpilogueTicket>(&pending_dispatch_epilogues),
                         x = x, sf = sf, topk_idx = topk_idx, topk_weights = topk_weights, context = context]() -> pybind11::object {
            EP_HOST_ASSERT_MSG(not ticket->released, "this dispatch epilogue has already been run");
            int num_recv_tokens = num_ranks * num_max_tokens_per_rank;
            int num_expanded_tokens = 0;
            std::vector<int> per_expert_list;
            if (cached_mode) {
                num_recv_tokens = *cached_num_recv_tokens, num_expanded_tokens = *cached_num_expanded_tokens;
                if (cached_num_recv_tokens_per_expert_list.has_value()) per_expert_list = *cached_num_recv_tokens_per_expert_list;
            } else if (do_cpu_sync) {
                pybind11::gil_scoped_release release;
                const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(context->num_cpu_timeout_secs);
                num_recv_tokens = static_cast<int>(host_wait_tagged(&host_counts->num_recv_tokens, deadline));
                num_expanded_tokens = static_cast<int>(host_wait_tagged(&host_counts->num_expanded_tokens, deadline));
                per_expert_list.assign(host_counts->aligned_recv_per_expert, host_counts->aligned_recv_per_expert + num_local_experts);
            } else {
                int64_t worst = static_cast<int64_t>(num_ranks) * num_max_tokens_per_rank * std::min(num_topk, num_local_experts);
                worst += static_cast<int64_t>(expert_alignment - 1) * num_local_experts;
                num_expanded_tokens = static_cast<int>(math::align<int64_t>(worst, expert_alignment));
            }

            const auto out_stream = c10::cuda::getCurrentCUDAStream();
            auto recv_x = torch::empty({num_expanded_tokens, hidden}, torch::TensorOptions().dtype(wire_dtype).device(device));
            std::optional<torch::Tensor> recv_sf, recv_topk_weights;
            int64_t recv_sf_token_stride = 0, recv_sf_pack_stride = 0;
            if (sf_bytes > 0) {
                recv_sf_token_stride = use_col_major_sf ? 1 : num_sf_packs;
                recv_sf_pack_stride = use_col_major_sf ? num_expanded_tokens : 1;
                recv_sf = torch::empty_strided({num_expanded_tokens, num_sf_packs}, {recv_sf_token_stride, recv_sf_pack_stride},
                                               torch::TensorOptions().dtype(torch::kInt16).device(device));
            }
            if (topk_weights.has_value())
                recv_topk_weights = torch::empty({num_expanded_tokens}, torch::TensorOptions().dtype(torch::kFloat32).device(device));
            auto recv_src_metadata = cached_mode ? *cached_recv_src_metadata : torch::empty({num_recv_tokens, num_topk + 2}, int_options);
            if (cached_mode)
                EP_HOST_ASSERT(recv_src_metadata.dim() == 2 and recv_src_metadata.size(0) == num_recv_tokens and
                               recv_src_metadata.size(1) == num_topk + 2 and recv_src_metadata.is_contiguous() and
                               recv_src_metadata.scalar_type() == torch::kInt32);

            kernels::ExpandArgs e = {};
            e.ws = signals(), e.buffer = static_cast<const uint8_t*>(context->buffer), e.host = host_counts_device;
            e.trace = trace_of(1);
            e.psum_rank = psum_rank.data_ptr<int>(), e.psum_expert = psum_expert.data_ptr<int>();
            e.num_unaligned = num_unaligned.data_ptr<int>();
            e.recv_x = static_cast<uint8_t*>(recv_x.data_ptr());
            e.recv_sf = recv_sf.has_value() ? static_cast<sf_pack_t*>(recv_sf->data_ptr()) : nullptr;
            e.recv_sf_token_stride = recv_sf_token_stride, e.recv_sf_pack_stride = recv_sf_pack_stride;
            e.recv_topk_weights = recv_topk_weights.has_value() ? recv_topk_weights->data_ptr<float>() : nullptr;
            e.recv_src_metadata = recv_src_metadata.data_ptr<int>();
            e.num_metadata_rows = num_recv_tokens, e.num_expanded_rows = num_expanded_tokens;
            e.rank = context->rank_idx, e.num_ranks = num_ranks, e.num_max_tokens = num_max_tokens_per_rank;
            e.num_experts = num_experts, e.num_topk = num_topk, e.expert_alignment = expert_alignment;
            e.hidden_bytes = hidden_bytes, e.sf_bytes = sf_bytes;
            e.cached = cached_mode, e.do_zero_padding = do_zero_padding, e.wait_arrival = not barrier_in_prologue;
            e.timeout_ns = context->num_gpu_timeout_ns;
            launch::dispatch_expand(e, num_sms, out_stream);
            ticket->release();

            return pybind11::make_tuple(recv_x, recv_sf, recv_topk_weights, num_recv_tokens, num_expanded_tokens, per_expert_list,
                                        psum_rank, psum_expert, num_unaligned, recv_src_metadata, dst_buffer_slot_idx, dst_gsge_idx);
        };

        if (defer_epilogue) {
            EP_HOST_ASSERT(async_with_compute_stream);
            std::function<pybind11::object()> hook = std::move(epilogue);
            return pybind11::make_tuple(pybind11::none(), std::optional<EventHandle>(EventHandle()), hook);
        }
        const auto result = epilogue();
        const auto event = async_with_compute_stream ? std::optional<EventHandle>(EventHandle()) : std::nullopt;
        return pybind11::make_tuple(result, event, pybind11::none());
    }

    // ------------------------------------------------------------------------------ combine
    pybind11::tuple combine(const torch::Tensor& x, const std::optional<torch::Tensor>& topk_weights,
                            const std::optional<torch::Tensor>& bias_0, const std::optional<torch::Tensor>& bias_1,
                            const torch::Tensor& recv_src_metadata, const torch::Tensor& topk_idx,
                            const torch::Tensor& psum_num_recv_tokens_per_rank,
                            int num_experts, int num_max_tokens_per_rank, int num_sms,
                            const std::optional<EventHandle>& previous_event,
                            bool async_with_compute_stream, bool allocate_on_comm_stream, bool defer_epilogue,
                            bool skip_single_rows, bool apply_weights) {
        EP_HOST_ASSERT(not destroyed and context->peers_ready);
        EP_HOST_ASSERT_MSG(pending_combine_epilogues == 0,
                           "the deferred epilogue of the previous combine on this buffer has not been run yet: call its hook "
                           "(`current_stream_wait()`) before the next combine");
        (void) allocate_on_comm_stream;
        const int num_ranks = context->num_ranks;
        const auto device = x.device();
        EP_HOST_ASSERT(x.dim() == 2 and x.is_contiguous() and x.is_cuda() and x.scalar_type() == torch::kBFloat16);
        const int hidden = static_cast<int>(x.size(1));
        EP_HOST_ASSERT_MSG(hidden % 8 == 0, "combine needs rows that are a multiple of 16 bytes");
        EP_HOST_ASSERT(topk_idx.dim() == 2 and topk_idx.is_contiguous() and topk_idx.scalar_type() == torch::kInt64);
        const int num_tokens = static_cast<int>(topk_idx.size(0)), num_topk = static_cast<int>(topk_idx.size(1));
        EP_HOST_ASSERT(recv_src_metadata.dim() == 2 and recv_src_metadata.size(1) == num_topk + 2 and
                       recv_src_metadata.is_contiguous() and recv_src_metadata.scalar_type() == torch::kInt32);
        EP_HOST_ASSERT(psum_num_recv_tokens_per_rank.numel() == num_ranks and psum_num_recv_tokens_per_rank.scalar_type() == torch::kInt32);
        EP_HOST_ASSERT(num_experts % num_ranks == 0 and num_tokens <= num_max_tokens_per_rank);
        if (topk_weights.has_value())
            EP_HOST_ASSERT(topk_weights->dim() == 1 and topk_weights->size(0) == x.size(0) and topk_weights->is_contiguous() and
                           topk_weights->scalar_type() == torch::kFloat32);
        for (const auto& bias : {bias_0, bias_1})
            if (bias.has_value())
                EP_HOST_ASSERT(bias->dim() == 2 and bias->size(0) == num_tokens and bias->size(1) == hidden and
                               bias->is_contiguous() and bias->scalar_type() == torch::kBFloat16);
        EP_HOST_ASSERT_MSG(get_combine_buffer_size(num_ranks, num_max_tokens_per_rank, hidden, num_topk) <= num_bytes,
                           "EP buffer too small for this combine");

        const auto stream = c10::cuda::getCurrentCUDAStream();
        if (previous_event.has_value()) previous_event->current_stream_wait();
        const bool barrier_in_prologue = Runtime::get().get_barrier_in_prologue();
        if (num_sms <= 0) num_sms = Runtime::get().get_num_sms();

        kernels::CombineArgs args = {};
        args.x = static_cast<const uint8_t*>(x.data_ptr());
        args.topk_weights = topk_weights.has_value() ? topk_weights->data_ptr<float>() : nullptr;
        args.recv_src_metadata = recv_src_metadata.data_ptr<int>();
        args.psum_rank = psum_num_recv_tokens_per_rank.data_ptr<int>();
        args.num_metadata_rows = static_cast<int>(recv_src_metadata.size(0));
        args.num_topk = num_topk, args.num_max_tokens = num_max_tokens_per_rank, args.hidden_bytes = hidden * 2;
        args.wait_arrival = barrier_in_prologue;
        args.ws = signals(), args.buffer_offset = context->num_workspace_bytes, args.buffer_bytes = num_bytes, args.peers = context->peers;
        args.host = host_counts_device, args.timeout_ns = context->num_gpu_timeout_ns;
        args.trace = trace_of(2);
        const bool coop = Runtime::get().get_warp_cooperation();
        EP_HOST_ASSERT_MSG(not apply_weights or (topk_weights.has_value() and not skip_single_rows),
                           "a weighted combine needs `topk_weights` and cannot be mixed with GEMM-delivered rows");
        args.coop = coop, args.skip_single = skip_single_rows, args.weighted = apply_weights;
        launch::combine(args, num_sms, stream);

        const bool with_weights = topk_weights.has_value();
        auto epilogue = [=, this, self = shared_from_this(), ticket = std::make_shared<EpilogueTicket>(&pending_combine_epilogues),
                         x = x, topk_weights = topk_weights, bias_0 = bias_0, bias_1 = bias_1, topk_idx = topk_idx,
                         context = context]() -> pybind11::object {
            EP_HOST_ASSERT_MSG(not ticket->released, "this combine epilogue has already been run");
            auto combined_x = torch::empty({num_tokens, hidden}, x.options());
            std::optional<torch::Tensor> combined_topk_weights;
            if (with_weights)
                combined_topk_weights = torch::empty({num_tokens, num_topk}, torch::TensorOptions().dtype(torch::kFloat32).device(device));
            kernels::CombineReduceArgs r = {};
            r.ws = signals(), r.buffer = static_cast<const uint8_t*>(context->buffer), r.host = host_counts_device;
            r.trace = trace_of(3), r.coop = coop;
            r.topk_idx = topk_idx.data_ptr<int64_t>();
            r.bias_0 = bias_0.has_value() ? static_cast<const uint8_t*>(bias_0->data_ptr()) : nullptr;
            r.bias_1 = bias_1.has_value() ? static_cast<const uint8_t*>(bias_1->data_ptr()) : nullptr;
            r.combined_x = static_cast<uint8_t*>(combined_x.data_ptr());
            r.combined_topk_weights = with_weights ? combined_topk_weights->data_ptr<float>() : nullptr;
            r.num_tokens = num_tokens, r.num_topk = num_topk, r.num_experts = num_experts;
            r.num_max_tokens = num_max_tokens_per_rank, r.hidden_bytes = hidden * 2;
            r.rank = context->rank_idx, r.num_ranks = num_ranks;
            r.wait_arrival = not barrier_in_prologue, r.timeout_ns = context->num_gpu_timeout_ns;
            launch::combine_reduce(r, Runtime::get().get_num_device_sms(), c10::cuda::getCurrentCUDAStream());
            ticket->release();
            return pybind11::make_tuple(combined_x, combined_topk_weights);
        };

        if (defer_epilogue) {
            EP_HOST_ASSERT(async_with_compute_stream);
            std::function<pybind11::object()> hook = std::move(epilogue);
            return pybind11::make_tuple(pybind11::none(), std::optional<EventHandle>(EventHandle()), hook);
        }
        const auto result = epilogue();
        const auto event = async_with_compute_stream ? std::optional<EventHandle>(EventHandle()) : std::nullopt;
        return pybind11::make_tuple(result, event, pybind11::none());
    }

    // ------------------------------------------------------------------------------ load balancing
    int64_t lb_offset_of(const torch::Tensor& t) const {
        const auto base = reinterpret_cast<int64_t>(context->buffer) + num_bytes;
        const auto ptr = reinterpret_cast<int64_t>(t.data_ptr());
        EP_HOST_ASSERT_MSG(ptr >= base and ptr + static_cast<int64_t>(t.nbytes()) <= base + num_lb_bytes,
                           "redundant expert tensors must live in this buffer's LB region");
        return context->num_workspace_bytes + num_bytes + (ptr - base);
    }

    kernels::LBArgs lb_common(const torch::Tensor& mapping, int num_local_experts) const {
        EP_HOST_ASSERT(not destroyed and context->peers_ready);
        EP_HOST_ASSERT(mapping.is_cuda() and mapping.dim() == 2 and mapping.scalar_type() == torch::kInt32 and mapping.is_contiguous());
        EP_HOST_ASSERT(mapping.size(0) == context->num_ranks and num_local_experts > 0);
        kernels::LBArgs args = {};
        args.peers = context->peers, args.cs = context->common_signals, args.host_status = context->host_status_device;
        args.timeout_ns = context->num_gpu_timeout_ns;
        args.mapping = mapping.data_ptr<int>(), args.num_redundant = static_cast<int>(mapping.size(1));
        args.num_local_experts = num_local_experts;
        return args;
    }

    // Landing addresses for GEMM epilogues that take over the combine push of single-row tokens: `route[r]` is where
    // expanded row r (bf16, `hidden` values) has to be stored instead of the GEMM's output tensor, 0 for all other rows.
    // The caller passes the table to the producing GEMM and then calls `combine(..., skip_single_rows=true)` with the
    // same handle. Between the dispatch epilogues of ALL ranks and the first store through the table there must be a
    // barrier over the group (the landing area is the one dispatch has just been read from).
    torch::Tensor build_combine_route(const torch::Tensor& recv_src_metadata, const torch::Tensor& psum_num_recv_tokens_per_rank,
                                      int num_expanded_rows, int num_max_tokens_per_rank, int hidden) const {
        EP_HOST_ASSERT(not destroyed and context->peers_ready);
        EP_HOST_ASSERT(recv_src_metadata.is_cuda() and recv_src_metadata.is_contiguous() and recv_src_metadata.dim() == 2 and
                       recv_src_metadata.scalar_type() == torch::kInt32);
        EP_HOST_ASSERT(psum_num_recv_tokens_per_rank.is_cuda() and psum_num_recv_tokens_per_rank.scalar_type() == torch::kInt32 and
                       psum_num_recv_tokens_per_rank.numel() == context->num_ranks);
        const int num_topk = static_cast<int>(recv_src_metadata.size(1)) - 2;
        EP_HOST_ASSERT(num_topk >= 1 and num_expanded_rows >= 0 and hidden > 0 and (hidden * 2) % 16 == 0);
        const layout::CombineTokenLayout tl(hidden * 2, num_topk);
        EP_HOST_ASSERT_MSG(get_combine_buffer_size(context->num_ranks, num_max_tokens_per_rank, hidden, num_topk) <= num_bytes,
                           "EP buffer too small for this combine");
        (void) tl;
        auto route = torch::zeros({num_expanded_rows}, torch::TensorOptions().dtype(torch::kInt64).device(recv_src_metadata.device()));
        if (recv_src_metadata.size(0) == 0 or num_expanded_rows == 0) return route;
        kernels::CombineRouteArgs args = {};
        args.recv_src_metadata = recv_src_metadata.data_ptr<int>();
        args.psum_rank = psum_num_recv_tokens_per_rank.data_ptr<int>();
        args.num_metadata_rows = static_cast<int>(recv_src_metadata.size(0)), args.num_expanded_rows = num_expanded_rows;
        args.num_topk = num_topk, args.num_max_tokens = num_max_tokens_per_rank, args.hidden_bytes = hidden * 2;
        args.buffer_offset = context->num_workspace_bytes, args.peers = context->peers;
        args.route = reinterpret_cast<unsigned long long*>(route.data_ptr<int64_t>());
        launch::combine_route(args, c10::cuda::getCurrentCUDAStream());
        return route;
    }

    // Phase trace (diagnostics): from now on the four EP kernels stamp `%globaltimer` at their phase boundaries into the
    // returned int64 tensor `[4, kTraceSlots]` (rows: dispatch, expand, combine, reduce; slot meaning: the `*Trace`
    // enums of `kernels/ep_args.hpp`). Each call overwrites the stamps of its kernels.
    torch::Tensor enable_phase_trace() {
        phase_trace = torch::zeros({4, kernels::kTraceSlots}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, c10::cuda::current_device()));
        return phase_trace;
    }
    void disable_phase_trace() { phase_trace = torch::Tensor(); }

    EventHandle lb_prefetch_weights(const std::vector<torch::Tensor>& redundant_expert_weights,
                                    const std::vector<torch::Tensor>& expert_weights, const torch::Tensor& redundancy_mapping,
                                    int num_sms, const std::optional<EventHandle>& previous_event) const {
        EP_HOST_ASSERT(not expert_weights.empty() and expert_weights.size() == redundant_expert_weights.size());
        EP_HOST_ASSERT(static_cast<int>(expert_weights.size()) <= kernels::kMaxLBTensors);
        auto args = lb_common(redundancy_mapping, static_cast<int>(expert_weights[0].size(0)));
        args.mode = 0, args.num_tensors = static_cast<int>(expert_weights.size());
        for (int i = 0; i < args.num_tensors; ++i) {
            const auto &src = expert_weights[i], &dst = redundant_expert_weights[i];
            EP_HOST_ASSERT(src.is_cuda() and src.is_contiguous() and src.dim() >= 2 and src.size(0) == args.num_local_experts);
            EP_HOST_ASSERT(dst.is_cuda() and dst.is_contiguous() and dst.dim() >= 2 and dst.size(0) == args.num_redundant);
            const int64_t bytes = static_cast<int64_t>(src.nbytes()) / src.size(0);
            EP_HOST_ASSERT(bytes == static_cast<int64_t>(dst.nbytes()) / dst.size(0) and bytes % 16 == 0);
            args.src[i] = static_cast<const uint8_t*>(src.data_ptr());
            args.dst_offset[i] = lb_offset_of(dst), args.bytes_per_expert[i] = bytes;
        }
        if (previous_event.has_value()) previous_event->current_stream_wait();
        launch::lb_exchange(args, num_sms > 0 ? num_sms : Runtime::get().get_num_sms(), c10::cuda::getCurrentCUDAStream());
        return EventHandle();
    }

    EventHandle lb_reduce_grads(const torch::Tensor& redundant_expert_grads, const torch::Tensor& expert_grads,
                                const torch::Tensor& redundancy_mapping, int num_sms,
                                const std::optional<EventHandle>& previous_event) const {
        EP_HOST_ASSERT(expert_grads.is_cuda() and expert_grads.is_contiguous() and expert_grads.dim() == 2 and
                       expert_grads.scalar_type() == torch::kFloat32);
        EP_HOST_ASSERT(redundant_expert_grads.is_cuda() and redundant_expert_grads.is_contiguous() and
                       redundant_expert_grads.dim() == 2 and redundant_expert_grads.scalar_type() == torch::kFloat32 and
                       redundant_expert_grads.size(1) == expert_grads.size(1));
        auto args = lb_common(redundancy_mapping, static_cast<int>(expert_grads.size(0)));
        EP_HOST_ASSERT(redundant_expert_grads.size(0) == args.num_redundant);
        args.mode = 1, args.num_tensors = 1;
        args.dst_offset[0] = lb_offset_of(redundant_expert_grads);
        args.expert_grads = expert_grads.data_ptr<float>(), args.hidden = expert_grads.size(1);
        if (previous_event.has_value()) previous_event->current_stream_wait();
        launch::lb_exchange(args, num_sms > 0 ? num_sms : Runtime::get().get_num_sms(), c10::cuda::getCurrentCUDAStream());
        return EventHandle();
    }

    void check_status() const {
        if (host_counts != nullptr and host_counts->status.code != 0) throw_device_status();
        if (context != nullptr) context->check_status();
    }
};

}  // namespace deep_ep
