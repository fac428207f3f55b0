// Bucket buffer: one symmetric storage registered with up to eight process groups, and a batched
// all-gather of up to 64 tensors per call (reference: `csrc/buffers/bucket.hpp:23-153`).
// The gather runs on the communication stream; its epilogue (a barrier that proves every peer's
// writes have landed) runs on the caller's stream.
#pragma once

#include <c10/cuda/CUDAStream.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <deep_ep/layout/bucket.hpp>

#include "../comm/barrier.hpp"
#include "../kernels/api.hpp"
#include "../runtime/device.hpp"
#include "../utils/event.hpp"
#include "base.hpp"

namespace deep_ep {

struct BucketWorkspace {
    layout::BucketSignals signals[kMaxContexts];
};

class BucketBuffer : public BufferBase {
    int64_t num_storage_bytes;

    void release_without_barrier() override {
        storage = torch::Tensor();
        for (const auto& c : contexts) c->finalize();
        contexts.clear();
        destroyed = true;
    }

public:
    std::vector<std::shared_ptr<comm::Context>> contexts;
    torch::Tensor storage;

    BucketBuffer(const std::vector<int>& rank_indices, const std::vector<int>& num_ranks,
                 const std::vector<std::string>& comm_names, int64_t num_storage_bytes, bool use_huge1g_page,
                 int num_gpu_timeout_secs, bool explicitly_destroy)
        : BufferBase(explicitly_destroy), num_storage_bytes(num_storage_bytes) {
        (void) use_huge1g_page;
        const int num_groups = static_cast<int>(comm_names.size());
        EP_HOST_ASSERT(num_groups > 0 and num_groups <= kMaxContexts);
        EP_HOST_ASSERT(static_cast<int>(rank_indices.size()) == num_groups and static_cast<int>(num_ranks.size()) == num_groups);
        EP_HOST_ASSERT(num_storage_bytes > 0 and num_storage_bytes % kNumAllocationAlignmentBytes == 0);
        const auto workspace_bytes = math::align<int64_t>(sizeof(BucketWorkspace), kNumAllocationAlignmentBytes);
        for (int i = 0; i < num_groups; ++i) {
            contexts.emplace_back(std::make_shared<comm::Context>(comm_names[i], rank_indices[i], num_ranks[i], workspace_bytes,
                                                                  num_storage_bytes, 0, 300, num_gpu_timeout_secs,
                                                                  contexts.empty() ? nullptr : contexts.front(), i));
            auto* workspace = static_cast<BucketWorkspace*>(contexts.back()->workspace);
            contexts.back()->set_common_signals(&workspace->signals[i].common);
        }
        main_context = contexts.front();
        storage = torch::from_blob(main_context->buffer, {num_storage_bytes}, [ctx = main_context](void*) {},
                                   torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, c10::cuda::current_device()));
    }

    ~BucketBuffer() override { destroy_on_destruction("bucket"); }

    void destroy() override {
        EP_HOST_ASSERT(not destroyed);
        for (const auto& c : contexts) comm::barrier(*c, true);
        release_without_barrier();
    }

    pybind11::tuple all_gather(const std::vector<torch::Tensor>& srcs, const std::vector<torch::Tensor>& dsts,
                               int context_idx, int num_sms) const {
        EP_HOST_ASSERT(not destroyed);
        EP_HOST_ASSERT(context_idx >= 0 and context_idx < static_cast<int>(contexts.size()));
        EP_HOST_ASSERT(not srcs.empty() and static_cast<int>(srcs.size()) <= kMaxBuckets);
        EP_HOST_ASSERT(dsts.empty() or dsts.size() == srcs.size());
        const auto& context = contexts[context_idx];
        EP_HOST_ASSERT(context->peers_ready);
        const int rank = context->rank_idx, num_ranks = context->num_ranks;

        kernels::AllGatherArgs args = {};
        args.peers = context->peers, args.cs = context->common_signals, args.host_status = context->host_status_device;
        args.timeout_ns = context->num_gpu_timeout_ns;
        args.use_multicast = context->peers.mc_base != nullptr, args.skip_local = 0;
        args.list.num_buckets = static_cast<int>(srcs.size());
        std::vector<torch::Tensor> gathered;
        const auto storage_ptr = reinterpret_cast<int64_t>(storage.data_ptr());
        for (size_t i = 0; i < srcs.size(); ++i) {
            const auto& src = srcs[i];
            EP_HOST_ASSERT(src.is_cuda() and src.is_contiguous() and src.numel() > 0);
            const auto shard_bytes = static_cast<int64_t>(src.nbytes());
            const auto src_offset = reinterpret_cast<int64_t>(src.data_ptr()) - storage_ptr;
            int64_t bucket_offset = src_offset - rank * shard_bytes;      // in-place: src is my shard of the gathered tensor
            if (not dsts.empty()) {
                const auto& dst = dsts[i];
                EP_HOST_ASSERT(dst.device() == src.device() and dst.is_contiguous() and dst.scalar_type() == src.scalar_type());
                EP_HOST_ASSERT(static_cast<int64_t>(dst.nbytes()) == num_ranks * shard_bytes);
                bucket_offset = reinterpret_cast<int64_t>(dst.data_ptr()) - storage_ptr;
            }
            EP_HOST_ASSERT_MSG(bucket_offset >= 0 and bucket_offset <= num_storage_bytes and
                               shard_bytes <= (num_storage_bytes - bucket_offset) / num_ranks,
                               "all-gather outputs must belong to this BucketBuffer");
            // the source is either exactly my shard of the output or does not overlap the output at all
            EP_HOST_ASSERT(src_offset == bucket_offset + rank * shard_bytes or src_offset + shard_bytes <= bucket_offset or
                           src_offset >= bucket_offset + num_ranks * shard_bytes);
            args.list.buckets[i] = {context->num_workspace_bytes + bucket_offset, shard_bytes, static_cast<const uint8_t*>(src.data_ptr())};
            gathered.push_back(storage.narrow(0, bucket_offset, num_ranks * shard_bytes).view(src.scalar_type()));
        }

        const auto compute_stream = c10::cuda::getCurrentCUDAStream();
        const auto comm_stream = comm::get_comm_stream();
        comm::stream_wait(comm_stream, compute_stream);
        if (num_sms <= 0) num_sms = std::min(Runtime::get().get_num_sms(), 32);
        launch::all_gather(args, num_sms, comm_stream);
        auto event = EventHandle(comm_stream);

        // Sources stay referenced until the epilogue has been enqueued.
        std::function<pybind11::object()> epilogue = [context, srcs, gathered = std::move(gathered)]() {
            comm::barrier(*context, false, true, true);
            return pybind11::cast(gathered);
        };
        return pybind11::make_tuple(event, epilogue, num_sms);
    }

    // In-place batched reduce-scatter (`all_reduce == false`) or all-reduce of registered tensors. Every rank passes
    // tensors at the same storage offsets; tensor i is cut into `num_ranks` equal shards and rank r reduces shard r.
    // Returns `(results, event, num_sms)`: for a reduce-scatter `results[i]` is this rank's reduced shard (a view of
    // `srcs[i]`), for an all-reduce it is `srcs[i]` itself. The kernel runs on the communication stream and contains
    // both rank barriers, so the event marks completion on every rank's data.
    // (The reference declares both without an implementation: `csrc/buffers/bucket.hpp:66-75`.)
    pybind11::tuple reduce(const std::vector<torch::Tensor>& srcs, int context_idx, int num_sms, float scale, bool all_reduce) const {
        EP_HOST_ASSERT(not destroyed);
        EP_HOST_ASSERT(context_idx >= 0 and context_idx < static_cast<int>(contexts.size()));
        EP_HOST_ASSERT(not srcs.empty() and static_cast<int>(srcs.size()) <= kMaxBuckets);
        const auto& context = contexts[context_idx];
        EP_HOST_ASSERT(context->peers_ready);
        const int rank = context->rank_idx, num_ranks = context->num_ranks;

        kernels::BucketReduceArgs args = {};
        args.peers = context->peers, args.cs = context->common_signals, args.host_status = context->host_status_device;
        args.timeout_ns = context->num_gpu_timeout_ns, args.scale = scale, args.all_reduce = all_reduce;
        args.use_multicast = context->peers.mc_base != nullptr;      // NVLS route (EP_NVLS=1): the switch adds and broadcasts
        args.list.num_buckets = static_cast<int>(srcs.size());
        std::vector<torch::Tensor> results;
        const auto storage_ptr = reinterpret_cast<int64_t>(storage.data_ptr());
        for (size_t i = 0; i < srcs.size(); ++i) {
            const auto& src = srcs[i];
            EP_HOST_ASSERT(src.is_cuda() and src.is_contiguous() and src.numel() > 0);
            const auto bytes = static_cast<int64_t>(src.nbytes());
            const auto offset = reinterpret_cast<int64_t>(src.data_ptr()) - storage_ptr;
            EP_HOST_ASSERT_MSG(offset >= 0 and offset + bytes <= num_storage_bytes, "reduced tensors must belong to this BucketBuffer");
            EP_HOST_ASSERT_MSG(offset % 16 == 0 and bytes % (int64_t(num_ranks) * 16) == 0,
                               "reduced tensors must start on a 16-byte boundary and split into 16-byte aligned shards");
            switch (src.scalar_type()) {
                case torch::kBFloat16: args.dtype[i] = kernels::kReduceBF16; break;
                case torch::kFloat32: args.dtype[i] = kernels::kReduceFP32; break;
                case torch::kFloat16: args.dtype[i] = kernels::kReduceFP16; break;
                default: EP_HOST_UNREACHABLE("reduce-scatter / all-reduce support bf16, fp16 and fp32 tensors");
            }
            args.list.buckets[i] = {context->num_workspace_bytes + offset, bytes, nullptr};
            const auto shard_numel = src.numel() / num_ranks;
            results.push_back(all_reduce ? src : src.view(-1).narrow(0, rank * shard_numel, shard_numel));
        }
        const auto compute_stream = c10::cuda::getCurrentCUDAStream();
        const auto comm_stream = comm::get_comm_stream();
        comm::stream_wait(comm_stream, compute_stream);
        if (num_sms <= 0) num_sms = Runtime::get().get_num_sms();
        launch::bucket_reduce(args, num_sms, comm_stream);
        return pybind11::make_tuple(results, EventHandle(comm_stream), num_sms);
    }
};

}  // namespace deep_ep
