// Pipeline-parallel buffer: buffered send/recv between ring neighbours over a credit-controlled
// ring of landing slots in symmetric memory (reference: `csrc/buffers/pp.hpp:14-92`).
#pragma once

#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <deep_ep/layout/pp.hpp>

#include "../comm/barrier.hpp"
#include "../kernels/api.hpp"
#include "../runtime/device.hpp"
#include "base.hpp"

namespace deep_ep {

class PPBuffer : public BufferBase {
    int64_t num_max_tensor_bytes, slot_bytes;
    int num_max_inflight_tensors;

    void release_without_barrier() override {
        storage = torch::Tensor();
        if (context != nullptr) context->finalize(), context = nullptr;
        destroyed = true;
    }

    kernels::PPArgs make_args(const torch::Tensor& x, int peer, int direction) const {
        EP_HOST_ASSERT(not destroyed and context->peers_ready);
        EP_HOST_ASSERT(x.is_cuda() and x.is_contiguous() and x.numel() > 0);
        EP_HOST_ASSERT(static_cast<int64_t>(x.nbytes()) <= num_max_tensor_bytes);
        kernels::PPArgs args = {};
        args.peers = context->peers;
        args.ws = static_cast<layout::PPSignals*>(context->workspace);
        args.host_status = context->host_status_device;
        args.x = static_cast<uint8_t*>(x.data_ptr());
        args.num_bytes = static_cast<int64_t>(x.nbytes());
        args.slot_bytes = slot_bytes;
        args.storage_offset = context->num_workspace_bytes;
        args.num_inflight = num_max_inflight_tensors;
        args.peer = peer, args.direction = direction;
        args.timeout_ns = context->num_gpu_timeout_ns;
        return args;
    }

    static int default_sms(int num_sms) { return num_sms > 0 ? num_sms : std::min(Runtime::get().get_num_sms(), 32); }

public:
    std::shared_ptr<comm::Context> context;
    torch::Tensor storage;

    // Two landing regions (from next rank, from previous rank) of `num_max_inflight_tensors` slots.
    static int64_t get_storage_bytes(int64_t num_max_tensor_bytes, int num_max_inflight_tensors) {
        return math::align<int64_t>(2 * math::align<int64_t>(num_max_tensor_bytes, 128) * num_max_inflight_tensors,
                                    kNumAllocationAlignmentBytes);
    }

    PPBuffer(int rank_idx, int num_ranks, const std::string& comm_name, int64_t num_max_tensor_bytes,
             int num_max_inflight_tensors, bool use_huge1g_page, int num_gpu_timeout_secs, bool explicitly_destroy)
        : BufferBase(explicitly_destroy), num_max_tensor_bytes(num_max_tensor_bytes),
          slot_bytes(math::align<int64_t>(num_max_tensor_bytes, 128)), num_max_inflight_tensors(num_max_inflight_tensors) {
        (void) use_huge1g_page;
        EP_HOST_ASSERT(num_max_tensor_bytes > 0 and num_max_tensor_bytes < (4ll << 30) and num_max_inflight_tensors > 0);
        const auto num_storage_bytes = get_storage_bytes(num_max_tensor_bytes, num_max_inflight_tensors);
        context = std::make_shared<comm::Context>(comm_name, rank_idx, num_ranks, layout::kPPWorkspaceBytes,
                                                  num_storage_bytes, 0, 300, num_gpu_timeout_secs);
        main_context = context;
        context->set_common_signals(&static_cast<layout::PPSignals*>(context->workspace)->common);
        storage = torch::from_blob(context->buffer, {num_storage_bytes}, [ctx = context](void*) {},
                                   torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, c10::cuda::current_device()));
    }

    ~PPBuffer() override { destroy_on_destruction("PP"); }

    void destroy() override {
        EP_HOST_ASSERT(not destroyed);
        comm::barrier(*context, true);
        release_without_barrier();
    }

    void send(const torch::Tensor& x, int dst_rank_idx, int num_sms) const {
        const int n = context->num_ranks, r = context->rank_idx;
        const bool to_next = dst_rank_idx == (r + 1) % n, to_prev = dst_rank_idx == (r + n - 1) % n;
        EP_HOST_ASSERT_MSG(to_next or to_prev, "PP send only reaches the previous or next rank of the ring");
        launch::pp_send(make_args(x, dst_rank_idx, to_next ? 0 : 1), default_sms(num_sms), c10::cuda::getCurrentCUDAStream());
    }

    void recv(const torch::Tensor& x, int src_rank_idx, int num_sms) const {
        const int n = context->num_ranks, r = context->rank_idx;
        const bool from_prev = src_rank_idx == (r + n - 1) % n, from_next = src_rank_idx == (r + 1) % n;
        EP_HOST_ASSERT_MSG(from_prev or from_next, "PP recv only listens to the previous or next rank of the ring");
        launch::pp_recv(make_args(x, src_rank_idx, from_prev ? 1 : 0), default_sms(num_sms), c10::cuda::getCurrentCUDAStream());
    }
};

}  // namespace deep_ep
