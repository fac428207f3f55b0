// CUDA driver API entry points resolved at run time through the runtime library, so that the extension
// has no link-time dependency on libcuda (it must import on machines without a GPU driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

#include <deep_ep/common/exception.hpp>

namespace deep_ep::driver {

template <typename Fn>
Fn resolve(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult result;
    const auto err = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &result);
    if (err != cudaSuccess or result != cudaDriverEntryPointSuccess or fn == nullptr) {
        cudaGetLastError();
        throw EPException("CUDA driver", __FILE__, __LINE__, std::string("cannot resolve ") + name);
    }
    return reinterpret_cast<Fn>(fn);
}

#define EP_DRIVER_FN(name)                                                   \
    inline decltype(&::name) name() {                                        \
        static auto fn = resolve<decltype(&::name)>(#name);                  \
        return fn;                                                           \
    }

EP_DRIVER_FN(cuGetErrorString)
EP_DRIVER_FN(cuTensorMapEncodeTiled)
EP_DRIVER_FN(cuModuleLoad)
EP_DRIVER_FN(cuModuleGetFunction)
EP_DRIVER_FN(cuFuncSetAttribute)
EP_DRIVER_FN(cuLaunchKernelEx)
// virtual memory management and NVLink multicast (the optional NVLS route of the symmetric allocation)
EP_DRIVER_FN(cuCtxGetDevice)
EP_DRIVER_FN(cuDeviceGetAttribute)
EP_DRIVER_FN(cuMemGetAllocationGranularity)
EP_DRIVER_FN(cuMemCreate)
EP_DRIVER_FN(cuMemRelease)
EP_DRIVER_FN(cuMemAddressReserve)
EP_DRIVER_FN(cuMemAddressFree)
EP_DRIVER_FN(cuMemMap)
EP_DRIVER_FN(cuMemUnmap)
EP_DRIVER_FN(cuMemSetAccess)
EP_DRIVER_FN(cuMemExportToShareableHandle)
EP_DRIVER_FN(cuMemImportFromShareableHandle)
EP_DRIVER_FN(cuMulticastGetGranularity)
EP_DRIVER_FN(cuMulticastCreate)
EP_DRIVER_FN(cuMulticastAddDevice)
EP_DRIVER_FN(cuMulticastBindMem)
EP_DRIVER_FN(cuMulticastUnbind)

#undef EP_DRIVER_FN

inline void check(CUresult r, const char* expr, const char* file, int line) {
    if (r == CUDA_SUCCESS) return;
    const char* text = nullptr;
    cuGetErrorString()(r, &text);
    throw EPException("CUDA driver", file, line, std::string(expr) + " -> " + (text ? text : "unknown"));
}

}  // namespace deep_ep::driver

#define DRV_CHECK(expr) deep_ep::driver::check((expr), #expr, __FILE__, __LINE__)
