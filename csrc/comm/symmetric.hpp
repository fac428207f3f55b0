// Symmetric device memory: one zero-filled allocation per process that every peer of the group
// maps into its own address space through CUDA IPC. Role of the reference's `SymmetricMemory`
// (`csrc/kernels/comm/symmetric.hpp:11-29`) plus the peer-address discovery of `HCCLContext`
// (`csrc/kernels/comm/hccl.hpp:173-194`); NVLink needs no queue pairs, so a pointer table is all
// the device code requires.
#pragma once

#include <cuda_runtime.h>

#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <deep_ep/common/exception.hpp>
#include <deep_ep/common/compiled.hpp>

#include "vmm.hpp"

namespace deep_ep::comm {

// Peer mappings are cached per process: a peer allocation shared by several groups is opened once.
class IpcMappingCache {
    struct Entry { void* ptr; int refs; };
    std::map<std::string, Entry> entries;
    std::mutex mutex;

public:
    static IpcMappingCache& get() {
        static IpcMappingCache instance;
        return instance;
    }

    void* open(const std::string& handle_bytes) {
        std::lock_guard<std::mutex> guard(mutex);
        auto it = entries.find(handle_bytes);
        if (it != entries.end()) { ++it->second.refs; return it->second.ptr; }
        EP_HOST_ASSERT(handle_bytes.size() == sizeof(cudaIpcMemHandle_t));
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, handle_bytes.data(), sizeof(handle));
        void* ptr = nullptr;
        CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess));
        entries[handle_bytes] = {ptr, 1};
        return ptr;
    }

    void close(const std::string& handle_bytes) {
        std::lock_guard<std::mutex> guard(mutex);
        auto it = entries.find(handle_bytes);
        if (it == entries.end()) return;
        if (--it->second.refs == 0) {
            cudaIpcCloseMemHandle(it->second.ptr);
            entries.erase(it);
        }
    }
};

class SymmetricMemory {
public:
    void* ptr = nullptr;
    int64_t num_bytes = 0;
    // set on the virtual-memory-management route (`EP_SYMMETRIC_VMM=1` / `EP_NVLS=1`), see vmm.hpp
    std::unique_ptr<VmmAllocation> vmm;
    size_t vmm_granularity_bytes = 0;

    SymmetricMemory(int64_t num_bytes, bool use_vmm = false, int num_ranks = 1, bool with_multicast = false) : num_bytes(num_bytes) {
        EP_HOST_ASSERT(num_bytes > 0 and num_bytes % kNumAllocationAlignmentBytes == 0);
        if (use_vmm) {
            CUDA_CHECK(cudaFree(nullptr));          // the driver calls need a current context
            vmm_granularity_bytes = vmm_granularity(num_ranks, with_multicast);
            vmm = std::make_unique<VmmAllocation>(static_cast<size_t>(num_bytes), vmm_granularity_bytes);
            ptr = reinterpret_cast<void*>(vmm->va);
            return;
        }
        CUDA_CHECK(cudaMalloc(&ptr, static_cast<size_t>(num_bytes)));
        CUDA_CHECK(cudaMemset(ptr, 0, static_cast<size_t>(num_bytes)));
        CUDA_CHECK(cudaDeviceSynchronize());
    }
    SymmetricMemory(const SymmetricMemory&) = delete;
    ~SymmetricMemory() {
        if (vmm == nullptr and ptr != nullptr) cudaFree(ptr);
    }

    std::string export_handle() const {
        EP_HOST_ASSERT(vmm == nullptr);
        cudaIpcMemHandle_t handle;
        CUDA_CHECK(cudaIpcGetMemHandle(&handle, ptr));
        return std::string(reinterpret_cast<const char*>(&handle), sizeof(handle));
    }
};

}  // namespace deep_ep::comm
