// Process-wide runtime knobs (reference: `Runtime` in `csrc/runtime/jit.hpp:17-70`): device
// properties queried once, the default SM budget of communication kernels, and the benchmark
// switch that moves the completion wait from the epilogue kernel into the issue kernel.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <memory>
#include <string>

#include <deep_ep/common/exception.hpp>
#include <deep_ep/common/compiled.hpp>

namespace deep_ep {

class Runtime {
    int device_sms = 0;          // SMs of the current device (0 until first query, or no GPU)
    int smem_per_block = 0;
    int num_sms_override = 0;    // user override of the default SM budget (0 = automatic)
    bool barrier_in_prologue = false;
    bool warp_cooperation = false;      // decode-sized EP calls: several warps share one row / token (see ep_combine.cuh)
    std::string arch = "sm_100a";

    void query() {
        if (device_sms != 0) return;
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return; }
        cudaDeviceGetAttribute(&device_sms, cudaDevAttrMultiProcessorCount, device);
        cudaDeviceGetAttribute(&smem_per_block, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    }

public:
    static Runtime& get() {
        static Runtime instance;
        return instance;
    }

    // SMs physically present (148 on B200); 0 when no GPU is visible.
    int get_num_device_sms() { query(); return device_sms; }
    int get_smem_bytes_per_block() { query(); return smem_per_block; }

    // Default SM budget of one communication kernel. NVLink saturates with a fraction of the
    // chip, so the default leaves most SMs to overlapped compute.
    int get_num_sms() {
        query();
        if (num_sms_override > 0) return num_sms_override;
        return device_sms > 0 ? std::min(device_sms, 64) : 64;
    }
    void set_num_sms(int n) {
        EP_HOST_ASSERT(n >= 0 and n <= kMaxCtas);
        num_sms_override = n;
    }

    const std::string& get_arch() const { return arch; }
    void set_arch(const std::string& a) { arch = a; }

    bool get_barrier_in_prologue() const { return barrier_in_prologue; }
    bool set_barrier_in_prologue(bool v) { std::swap(v, barrier_in_prologue); return v; }
    bool get_warp_cooperation() const { return warp_cooperation; }
    bool set_warp_cooperation(bool v) { std::swap(v, warp_cooperation); return v; }
};

}  // namespace deep_ep
