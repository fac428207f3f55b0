// Engram buffer: sharded embedding tables in symmetric memory and a per-layer remote gather
// (reference: `csrc/buffers/engram.hpp:19-212`). Allocation = [workspace | receive region + SF shards | table shards].
#pragma once

#include <c10/cuda/CUDAStream.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <deep_ep/layout/engram.hpp>

#include "../comm/barrier.hpp"
#include "../kernels/api.hpp"
#include "../runtime/device.hpp"
#include "base.hpp"

namespace deep_ep {

class EngramBuffer : public BufferBase {
    std::vector<int> num_entries_per_layer;
    int hidden = 0, elem_size = 0, num_max_tokens = 0, num_entries_per_token = 0, num_sf_packs = 0;
    int64_t num_recv_bytes = 0;

    void release_without_barrier() override {
        if (context != nullptr) context->finalize(), context = nullptr;
        destroyed = true;
    }

public:
    std::shared_ptr<comm::Context> context;

    EngramBuffer(int rank_idx, int num_ranks, const std::string& comm_name, int64_t num_gpu_bytes,
                 int64_t num_rdma_storage_bytes, bool use_huge1g_page, int num_gpu_timeout_secs, bool explicitly_destroy)
        : BufferBase(explicitly_destroy) {
        (void) use_huge1g_page;
        EP_HOST_ASSERT(num_gpu_bytes > 0 and num_rdma_storage_bytes > 0);
        context = std::make_shared<comm::Context>(comm_name, rank_idx, num_ranks, layout::kEngramWorkspaceBytes,
                                                  num_gpu_bytes, num_rdma_storage_bytes, 300, num_gpu_timeout_secs);
        main_context = context;
        context->set_common_signals(&static_cast<layout::EngramSignals*>(context->workspace)->common);
    }

    ~EngramBuffer() override { destroy_on_destruction("Engram"); }

    void destroy() override {
        EP_HOST_ASSERT(not destroyed);
        comm::barrier(*context, true);
        release_without_barrier();
    }

    void set_config(const std::vector<int>& entries_per_layer, int hidden_, int elem_size_, int num_max_tokens_,
                    int num_entries_per_token_, int num_sf_packs_) {
        EP_HOST_ASSERT(not destroyed);
        comm::barrier(*context);
        EP_HOST_ASSERT(num_max_tokens_ > 0 and num_entries_per_token_ > 0 and hidden_ > 0 and num_sf_packs_ >= 0);
        EP_HOST_ASSERT(not entries_per_layer.empty() and static_cast<int>(entries_per_layer.size()) <= layout::kMaxEngramLayers);
        EP_HOST_ASSERT((elem_size_ == 1 and num_sf_packs_ > 0) or (elem_size_ == 2 and num_sf_packs_ == 0));
        EP_HOST_ASSERT_MSG((static_cast<int64_t>(hidden_) * elem_size_) % 16 == 0, "entries must be a multiple of 16 bytes");
        int64_t total_entries = 0;
        for (const auto n : entries_per_layer) {
            EP_HOST_ASSERT(n > 0);
            total_entries += n;
        }
        const int64_t recv_bytes = static_cast<int64_t>(entries_per_layer.size()) * num_max_tokens_ * num_entries_per_token_ * hidden_ * elem_size_;
        const int64_t sf_bytes = total_entries * num_sf_packs_ * static_cast<int64_t>(sizeof(sf_pack_t));
        EP_HOST_ASSERT(recv_bytes + sf_bytes <= context->num_gpu_buffer_bytes);
        EP_HOST_ASSERT(total_entries * hidden_ * elem_size_ <= context->num_rdma_storage_bytes);
        num_entries_per_layer = entries_per_layer;
        hidden = hidden_, elem_size = elem_size_, num_max_tokens = num_max_tokens_;
        num_entries_per_token = num_entries_per_token_, num_sf_packs = num_sf_packs_, num_recv_bytes = recv_bytes;
    }

    // Copy this rank's table shards (and its slice of every replicated SF table) into symmetric memory.
    void write(const std::vector<torch::Tensor>& storages, const std::optional<std::vector<torch::Tensor>>& sfs) {
        EP_HOST_ASSERT(not destroyed);
        const auto stream = c10::cuda::getCurrentCUDAStream();
        comm::barrier(*context);     // no peer is still reading the previous tables
        const int num_layers = static_cast<int>(num_entries_per_layer.size());
        EP_HOST_ASSERT(num_layers > 0 and static_cast<int>(storages.size()) == num_layers);
        EP_HOST_ASSERT(sfs.has_value() == (num_sf_packs > 0));
        auto* dst = static_cast<uint8_t*>(context->local_rdma_storage_ptr);
        for (int l = 0; l < num_layers; ++l) {
            const auto& t = storages[l];
            EP_HOST_ASSERT(t.dim() == 2 and t.size(0) == num_entries_per_layer[l] and t.size(1) == hidden and
                           t.element_size() == elem_size and t.is_cuda() and t.is_contiguous());
            EP_HOST_ASSERT(t.scalar_type() == (num_sf_packs > 0 ? torch::kFloat8_e4m3fn : torch::kBFloat16));
            CUDA_CHECK(cudaMemcpyAsync(dst, t.data_ptr(), t.nbytes(), cudaMemcpyDeviceToDevice, stream));
            dst += t.nbytes();
        }
        if (sfs.has_value()) {
            EP_HOST_ASSERT(static_cast<int>(sfs->size()) == num_layers);
            auto* sf_dst = static_cast<uint8_t*>(context->buffer) + num_recv_bytes;
            for (int l = 0; l < num_layers; ++l) {
                const auto& sf = sfs->at(l);
                EP_HOST_ASSERT(sf.dim() == 2 and sf.size(0) == static_cast<int64_t>(context->num_ranks) * num_entries_per_layer[l] and
                               sf.size(1) == num_sf_packs and sf.is_cuda() and sf.is_contiguous() and sf.element_size() == 2);
                const int64_t shard = static_cast<int64_t>(sf.nbytes()) / context->num_ranks;
                CUDA_CHECK(cudaMemcpyAsync(sf_dst, static_cast<const uint8_t*>(sf.data_ptr()) + context->rank_idx * shard, shard,
                                           cudaMemcpyDeviceToDevice, stream));
                sf_dst += shard;
            }
        }
        comm::barrier(*context);     // every rank's tables are in place before anyone fetches
    }

    std::vector<std::function<pybind11::object()>> fetch(const torch::Tensor& indices, int num_qps, bool use_col_major_sf) const {
        EP_HOST_ASSERT(not destroyed and num_qps == 0 and context->peers_ready);
        EP_HOST_ASSERT(indices.dim() == 3 and indices.scalar_type() == torch::kInt32 and indices.is_contiguous() and indices.is_cuda());
        const bool use_fp8 = num_sf_packs > 0;
        const int num_layers = static_cast<int>(indices.size(0)), num_tokens = static_cast<int>(indices.size(1));
        const int per_token = static_cast<int>(indices.size(2));
        EP_HOST_ASSERT(num_layers == static_cast<int>(num_entries_per_layer.size()));
        EP_HOST_ASSERT(num_tokens <= num_max_tokens and per_token == num_entries_per_token);
        const auto device = indices.device();

        const int64_t hidden_bytes = static_cast<int64_t>(hidden) * elem_size;
        const int64_t layer_bytes = static_cast<int64_t>(num_max_tokens) * per_token * hidden_bytes;
        std::vector<torch::Tensor> fetched, fetched_sf;
        for (int l = 0; l < num_layers; ++l)
            fetched.push_back(torch::from_blob(static_cast<uint8_t*>(context->buffer) + l * layer_bytes,
                                               {num_tokens, static_cast<int64_t>(per_token) * hidden}, [ctx = context](void*) {},
                                               torch::TensorOptions().dtype(use_fp8 ? torch::kFloat8_e4m3fn : torch::kBFloat16).device(device)));

        kernels::EngramFetchArgs args = {};
        args.peers = context->peers;
        args.table.num_layers = num_layers;
        int64_t storage_offset = context->num_workspace_bytes + context->num_gpu_buffer_bytes;
        int64_t sf_offset = context->num_workspace_bytes + num_recv_bytes;
        for (int l = 0; l < num_layers; ++l) {
            args.table.storage_offset[l] = storage_offset, args.table.sf_offset[l] = sf_offset;
            args.table.num_entries_per_rank[l] = num_entries_per_layer[l];
            storage_offset += static_cast<int64_t>(num_entries_per_layer[l]) * hidden_bytes;
            sf_offset += static_cast<int64_t>(num_entries_per_layer[l]) * num_sf_packs * static_cast<int64_t>(sizeof(sf_pack_t));
        }
        args.indices = indices.data_ptr<int>();
        args.recv = static_cast<uint8_t*>(context->buffer);
        if (use_fp8) {
            args.sf_token_stride = use_col_major_sf ? 1 : static_cast<int64_t>(per_token) * num_sf_packs;
            args.sf_pack_stride = use_col_major_sf ? num_tokens : 1;
            args.sf_layer_stride = static_cast<int64_t>(num_tokens) * per_token * num_sf_packs;
            const auto backing = torch::empty({num_layers, args.sf_layer_stride}, torch::TensorOptions().dtype(torch::kInt16).device(device));
            for (int l = 0; l < num_layers; ++l)
                fetched_sf.push_back(backing[l].as_strided({num_tokens, static_cast<int64_t>(per_token) * num_sf_packs},
                                                           {args.sf_token_stride, args.sf_pack_stride}));
            args.sf_out = static_cast<sf_pack_t*>(backing.data_ptr());
        }
        args.num_layers = num_layers, args.num_tokens = num_tokens, args.num_entries_per_token = per_token;
        args.num_max_tokens = num_max_tokens, args.hidden_bytes = static_cast<int>(hidden_bytes), args.num_sf_packs = num_sf_packs;
        launch::engram_fetch(args, Runtime::get().get_num_device_sms(), c10::cuda::getCurrentCUDAStream());

        std::vector<std::function<pybind11::object()>> hooks;
        for (int l = 0; l < num_layers; ++l)
            hooks.emplace_back([=]() -> pybind11::object {
                return use_fp8 ? pybind11::object(pybind11::make_tuple(fetched[l], fetched_sf[l])) : pybind11::cast(fetched[l]);
            });
        return hooks;
    }
};

}  // namespace deep_ep
