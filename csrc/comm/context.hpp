// `Context`: one per (buffer, process group). Owns or shares the symmetric allocation, split as
// `[workspace | buffer | storage]`, the table of peer base addresses, the time-outs and the
// host-visible status word. Counterpart of the reference's `comm::Context`
// (`csrc/kernels/comm/api.hpp:16-101`).
#pragma once

#include <chrono>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include <deep_ep/layout/signals.hpp>

#include "symmetric.hpp"

namespace deep_ep::comm {

class Context {
    std::vector<std::string> opened_handles;
    bool finalized = false;

public:
    std::string comm_name;
    int rank_idx, num_ranks;
    int context_idx = 0;                       // index of this context's signal block in the workspace
    int64_t num_workspace_bytes, num_gpu_buffer_bytes, num_rdma_storage_bytes;
    int num_cpu_timeout_secs, num_gpu_timeout_secs;
    long long num_gpu_timeout_ns;

    std::shared_ptr<SymmetricMemory> memory;   // shared with the main context when several groups use one allocation
    std::shared_ptr<Context> main_context;     // nullptr for the main context itself
    void* workspace = nullptr;                 // start of the allocation
    void* buffer = nullptr;                    // workspace + num_workspace_bytes
    void* local_rdma_storage_ptr = nullptr;    // buffer + num_gpu_buffer_bytes
    layout::CommonSignals* common_signals = nullptr;
    layout::PeerTable peers = {};
    bool peers_ready = false;

    // mapped pinned host memory the kernels write their failure record to
    layout::HostStatus* host_status = nullptr;        // host view
    layout::HostStatus* host_status_device = nullptr; // device view of the same memory

    Context(const std::string& comm_name, int rank_idx, int num_ranks,
            int64_t num_workspace_bytes, int64_t num_gpu_buffer_bytes, int64_t num_rdma_storage_bytes,
            int num_cpu_timeout_secs, int num_gpu_timeout_secs,
            const std::shared_ptr<Context>& main_context = nullptr, int context_idx = 0)
        : comm_name(comm_name), rank_idx(rank_idx), num_ranks(num_ranks), context_idx(context_idx),
          num_workspace_bytes(num_workspace_bytes), num_gpu_buffer_bytes(num_gpu_buffer_bytes),
          num_rdma_storage_bytes(num_rdma_storage_bytes),
          num_cpu_timeout_secs(num_cpu_timeout_secs), num_gpu_timeout_secs(num_gpu_timeout_secs),
          num_gpu_timeout_ns(static_cast<long long>(num_gpu_timeout_secs) * 1000000000ll),
          main_context(main_context) {
        EP_HOST_ASSERT(0 <= rank_idx and rank_idx < num_ranks and num_ranks <= kMaxRanks);
        EP_HOST_ASSERT(0 <= context_idx and context_idx < kMaxContexts);
        EP_HOST_ASSERT(num_workspace_bytes % kNumAllocationAlignmentBytes == 0);
        EP_HOST_ASSERT(num_gpu_buffer_bytes % kNumAllocationAlignmentBytes == 0);
        EP_HOST_ASSERT(num_rdma_storage_bytes % kNumAllocationAlignmentBytes == 0);
        if (main_context != nullptr) {
            EP_HOST_ASSERT(main_context->num_workspace_bytes == num_workspace_bytes and
                           main_context->num_gpu_buffer_bytes == num_gpu_buffer_bytes and
                           main_context->num_rdma_storage_bytes == num_rdma_storage_bytes);
            memory = main_context->memory;
        } else {
            memory = std::make_shared<SymmetricMemory>(num_workspace_bytes + num_gpu_buffer_bytes + num_rdma_storage_bytes);
        }
        workspace = memory->ptr;
        buffer = static_cast<uint8_t*>(workspace) + num_workspace_bytes;
        local_rdma_storage_ptr = static_cast<uint8_t*>(buffer) + num_gpu_buffer_bytes;

        void* host = nullptr;
        CUDA_CHECK(cudaHostAlloc(&host, sizeof(layout::HostStatus), cudaHostAllocMapped));
        std::memset(host, 0, sizeof(layout::HostStatus));
        host_status = static_cast<layout::HostStatus*>(host);
        void* device_view = nullptr;
        CUDA_CHECK(cudaHostGetDevicePointer(&device_view, host, 0));
        host_status_device = static_cast<layout::HostStatus*>(device_view);

        peers.rank = rank_idx, peers.num_ranks = num_ranks, peers.mc_base = nullptr;
        for (auto& p : peers.base) p = nullptr;
        peers.base[rank_idx] = static_cast<uint8_t*>(workspace);
        if (num_ranks == 1) peers_ready = true;
    }

    ~Context() {
        if (not finalized) {
            try { finalize(); } catch (...) {}
        }
    }

    // Register where this context's `CommonSignals` block lives (inside the workspace).
    void set_common_signals(void* ptr) {
        const auto offset = static_cast<uint8_t*>(ptr) - static_cast<uint8_t*>(workspace);
        EP_HOST_ASSERT(offset >= 0 and offset + static_cast<int64_t>(sizeof(layout::CommonSignals)) <= num_workspace_bytes);
        common_signals = static_cast<layout::CommonSignals*>(ptr);
    }

    std::string get_local_handle() const { return memory->export_handle(); }

    // `handles[r]` is rank r's exported allocation handle, gathered over the process group.
    void set_peer_handles(const std::vector<std::string>& handles) {
        EP_HOST_ASSERT(static_cast<int>(handles.size()) == num_ranks and not peers_ready);
        for (int r = 0; r < num_ranks; ++r) {
            if (r == rank_idx) continue;
            peers.base[r] = static_cast<uint8_t*>(IpcMappingCache::get().open(handles[r]));
            opened_handles.push_back(handles[r]);
        }
        peers_ready = true;
    }

    std::pair<int, int> get_physical_domain_size() const { return {1, num_ranks}; }
    std::pair<int, int> get_logical_domain_size() const { return {1, num_ranks}; }

    // Throws if a kernel of this context recorded a failure.
    void check_status() const {
        if (host_status == nullptr or host_status->code == 0) return;
        static const char* names[] = {"ok", "rank barrier timeout", "grid sync timeout", "count exchange timeout",
                                      "arrival timeout", "credit timeout", "bad argument", "bulk copy timeout"};
        const int code = host_status->code;
        std::ostringstream os;
        os << "device-side failure: " << (code >= 0 and code < 8 ? names[code] : "unknown") << " (code " << code
           << ") on rank " << host_status->rank << ", waiting for rank " << host_status->peer << " at site "
           << host_status->where << ", expected " << host_status->expected << ", observed " << host_status->observed;
        throw EPException("Device status", __FILE__, __LINE__, os.str());
    }

    void finalize() {
        if (finalized) return;
        finalized = true;
        for (const auto& h : opened_handles) IpcMappingCache::get().close(h);
        opened_handles.clear();
        if (host_status != nullptr) cudaFreeHost(const_cast<layout::HostStatus*>(host_status));
        host_status = nullptr, host_status_device = nullptr;
        memory = nullptr, main_context = nullptr;
        workspace = buffer = local_rdma_storage_ptr = nullptr;
    }
};

}  // namespace deep_ep::comm
