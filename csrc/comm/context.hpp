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
    // virtual-memory-management route: descriptor server for the peers, imported peer allocations, multicast object
    std::unique_ptr<FdServer> fd_server;
    std::vector<std::unique_ptr<VmmPeerMapping>> vmm_peers;
    std::unique_ptr<VmmPeerMapping> multicast;
    bool multicast_added = false, multicast_bound = false;
    int multicast_fd = -1;

    static bool env_flag(const char* name) {
        const char* value = std::getenv(name);
        return value != nullptr and std::string(value) == "1";
    }

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
            // EP_NVLS=1: allocate through the virtual-memory-management API and bind the allocation to an NVLink multicast
            // object of the group (`multimem.*` instructions); EP_SYMMETRIC_VMM=1: the same allocation route without multicast
            const bool want_multicast = env_flag("EP_NVLS") and num_ranks > 1;
            const bool use_vmm = want_multicast or env_flag("EP_SYMMETRIC_VMM");
            if (want_multicast) {
                CUDA_CHECK(cudaFree(nullptr));      // the driver query needs a current context
                EP_HOST_ASSERT_MSG(multicast_supported(), "EP_NVLS=1 but this GPU reports no multicast support");
            }
            memory = std::make_shared<SymmetricMemory>(num_workspace_bytes + num_gpu_buffer_bytes + num_rdma_storage_bytes,
                                                       use_vmm, num_ranks, want_multicast);
            wants_multicast = want_multicast;
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

    bool wants_multicast = false;     // main context only: a multicast object is created with the peer exchange

    // What the peers need to map this rank's allocation: the CUDA IPC handle, or on the virtual-memory-management route
    // the name of a socket that hands out the allocation's descriptor (rank 0: and the multicast object's).
    std::string get_local_handle() {
        if (memory->vmm == nullptr) return memory->export_handle();
        if (fd_server == nullptr) {
            std::vector<int> fds = {memory->vmm->fd};
            int mc_fd = -1;
            if (wants_multicast and rank_idx == 0) {
                const auto handle = create_multicast_object(num_ranks, memory->vmm->size, mc_fd);
                multicast = std::make_unique<VmmPeerMapping>(handle, memory->vmm->size);
                fds.push_back(mc_fd);
            }
            multicast_fd = mc_fd;      // stays open until the server has handed it to every peer (closed in finalize)
            fd_server = std::make_unique<FdServer>(fds, num_ranks - 1, num_cpu_timeout_secs);
        }
        return "vmm:" + fd_server->name + ":" + std::to_string(memory->vmm->size) + ":" + (wants_multicast ? "1" : "0");
    }

    // `handles[r]` is what rank r's `get_local_handle` returned, gathered over the process group.
    void set_peer_handles(const std::vector<std::string>& handles) {
        EP_HOST_ASSERT(static_cast<int>(handles.size()) == num_ranks and not peers_ready);
        const bool vmm_route = memory->vmm != nullptr;
        for (int r = 0; r < num_ranks; ++r) {
            EP_HOST_ASSERT_MSG((handles[r].rfind("vmm:", 0) == 0) == vmm_route,
                               "every rank must use the same allocation route (EP_SYMMETRIC_VMM / EP_NVLS)");
            if (r == rank_idx) continue;
            if (not vmm_route) {
                peers.base[r] = static_cast<uint8_t*>(IpcMappingCache::get().open(handles[r]));
                opened_handles.push_back(handles[r]);
                continue;
            }
            // "vmm:<socket name>:<mapped bytes>:<multicast wanted>"
            const auto first = handles[r].find(':', 4), second = handles[r].find(':', first + 1);
            EP_HOST_ASSERT(first != std::string::npos and second != std::string::npos);
            const std::string name = handles[r].substr(4, first - 4);
            const size_t peer_bytes = std::stoull(handles[r].substr(first + 1, second - first - 1));
            const bool peer_multicast = handles[r].substr(second + 1) == "1";
            EP_HOST_ASSERT_MSG(peer_bytes == memory->vmm->size and peer_multicast == wants_multicast,
                               "ranks disagree about the size or the multicast setting of the symmetric allocation");
            const int num_fds = (r == 0 and peer_multicast) ? 2 : 1;
            const auto fds = receive_fds(name, num_fds, num_cpu_timeout_secs);
            try {
                // each mapping closes the descriptor it is given, whether or not the import succeeds
                vmm_peers.push_back(std::make_unique<VmmPeerMapping>(fds[0], peer_bytes, memory->vmm_granularity_bytes));
            } catch (...) {
                if (num_fds == 2) ::close(fds[1]);
                throw;
            }
            peers.base[r] = reinterpret_cast<uint8_t*>(vmm_peers.back()->va);
            if (num_fds == 2)
                multicast = std::make_unique<VmmPeerMapping>(fds[1], peer_bytes, memory->vmm_granularity_bytes, /*map_now=*/false);
        }
        if (wants_multicast) {
            EP_HOST_ASSERT(multicast != nullptr);
            DRV_CHECK(driver::cuMulticastAddDevice()(multicast->handle, vmm_detail::current_device()));
            multicast_added = true;
        }
        peers_ready = true;
    }

    // True between `set_peer_handles` and `bind_multicast`: the caller has to put a barrier over the group in between
    // (every device must have been added to the multicast object before any memory is bound to it) and one after.
    bool multicast_pending() const { return multicast_added and not multicast_bound; }

    void bind_multicast() {
        EP_HOST_ASSERT(multicast_pending());
        DRV_CHECK(driver::cuMulticastBindMem()(multicast->handle, 0, memory->vmm->handle, 0, memory->vmm->size, 0));
        multicast->map(memory->vmm_granularity_bytes);
        peers.mc_base = reinterpret_cast<uint8_t*>(multicast->va);
        multicast_bound = true;
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

    // First half of a teardown without a device-side barrier (after a failure): this rank stops mapping its peers'
    // memory. Once every rank has done so (the caller meets the others on the host), each may free its own allocation.
    void close_peer_mappings() {
        for (const auto& h : opened_handles) IpcMappingCache::get().close(h);
        opened_handles.clear();
        for (int r = 0; r < num_ranks; ++r)
            if (r != rank_idx and memory != nullptr and memory->vmm == nullptr) peers.base[r] = nullptr;
        peers_ready = num_ranks == 1;
    }

    void finalize() {
        if (finalized) return;
        finalized = true;
        for (const auto& h : opened_handles) IpcMappingCache::get().close(h);
        opened_handles.clear();
        if (multicast != nullptr) {
            multicast->unmap();
            if (multicast_bound) driver::cuMulticastUnbind()(multicast->handle, vmm_detail::current_device(), 0, memory->vmm->size);
            multicast = nullptr, peers.mc_base = nullptr;
        }
        vmm_peers.clear();
        fd_server = nullptr;
        if (multicast_fd >= 0) ::close(multicast_fd), multicast_fd = -1;
        if (host_status != nullptr) cudaFreeHost(const_cast<layout::HostStatus*>(host_status));
        host_status = nullptr, host_status_device = nullptr;
        memory = nullptr, main_context = nullptr;
        workspace = buffer = local_rdma_storage_ptr = nullptr;
    }
};

}  // namespace deep_ep::comm
