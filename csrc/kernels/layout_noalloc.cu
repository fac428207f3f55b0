// Allocation-free variant of the routing-layout kernel: same device code as `ep_layout_kernel`, with its
// scratch block in a file-scope device array instead of memory obtained from an allocator. See
// `layout_noalloc.h` for who needs this and for the rules of use.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include <deep_ep/kernels/ep_layout.cuh>

#include "layout_noalloc.h"

namespace {

using deep_ep::kernels::LayoutArgs;
using deep_ep::kernels::LayoutScratch;

// One scratch block per GPU that loads this library, held until the process exits. In host code this
// name is only a handle for the runtime; the device address is obtained once per device below.
static __device__ __align__(256) unsigned char g_layout_scratch[sizeof(LayoutScratch)];

// How the most recent launch on this device ended (0, or the code of a device-side wait that ran out); same lifetime.
static __device__ int g_layout_status;

constexpr int kMaxDevices = 64;
LayoutScratch* g_scratch_address[kMaxDevices] = {};
int* g_status_address[kMaxDevices] = {};
std::mutex g_setup_mutex;
thread_local std::string g_last_error;

__global__ void __launch_bounds__(256, 1) ep_layout_noalloc_kernel(const __grid_constant__ LayoutArgs a) {
    deep_ep::kernels::ep_layout_body(a);
}

int fail(int code, const std::string& what) {
    g_last_error = what;
    return code;
}

// Device addresses of the scratch array and of the status word on the current device; looked up on the first call per device.
int scratch_for_current_device(LayoutScratch** out, int** status_out) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return fail(DEEP_EP_NOALLOC_CUDA_ERROR, std::string("cudaGetDevice: ") + cudaGetErrorString(err));
    if (device < 0 or device >= kMaxDevices) return fail(DEEP_EP_NOALLOC_BAD_ARGUMENT, "device index beyond 63");
    std::lock_guard<std::mutex> guard(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, g_layout_scratch);
        if (err != cudaSuccess or address == nullptr)
            return fail(DEEP_EP_NOALLOC_CUDA_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(err));
        void* status_address = nullptr;
        err = cudaGetSymbolAddress(&status_address, g_layout_status);
        if (err != cudaSuccess or status_address == nullptr)
            return fail(DEEP_EP_NOALLOC_CUDA_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(err));
        g_status_address[device] = static_cast<int*>(status_address);
        g_scratch_address[device] = static_cast<LayoutScratch*>(address);
    }
    *out = g_scratch_address[device];
    *status_out = g_status_address[device];
    return DEEP_EP_NOALLOC_OK;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int deep_ep_dispatch_layout_noalloc(const long long* topk_idx, int num_tokens, int num_topk, int num_experts,
                                    int num_ranks, int* dst_slot_idx, int* num_tokens_per_rank,
                                    int* num_tokens_per_expert, void* stream_handle) {
    g_last_error.clear();
    if (topk_idx == nullptr or dst_slot_idx == nullptr or num_tokens_per_rank == nullptr or num_tokens_per_expert == nullptr)
        return fail(DEEP_EP_NOALLOC_BAD_ARGUMENT, "null pointer argument");
    if (num_tokens <= 0 or num_tokens > DEEP_EP_NOALLOC_MAX_TOKENS)
        return fail(DEEP_EP_NOALLOC_BAD_ARGUMENT, "num_tokens must be in [1, " + std::to_string(DEEP_EP_NOALLOC_MAX_TOKENS) + "]");
    if (num_topk <= 0 or num_topk > deep_ep::kMaxTopk)
        return fail(DEEP_EP_NOALLOC_BAD_ARGUMENT, "num_topk must be in [1, 32]");
    if (num_ranks <= 0 or num_ranks > deep_ep::kMaxRanks)
        return fail(DEEP_EP_NOALLOC_BAD_ARGUMENT, "num_ranks must be in [1, 64]");
    if (num_experts <= 0 or num_experts > deep_ep::kMaxExperts or num_experts % num_ranks != 0)
        return fail(DEEP_EP_NOALLOC_BAD_ARGUMENT, "num_experts must be in [1, 2048] and a multiple of num_ranks");

    LayoutScratch* scratch = nullptr;
    int* device_status = nullptr;
    if (const int rc = scratch_for_current_device(&scratch, &device_status); rc != DEEP_EP_NOALLOC_OK) return rc;
    const auto stream = static_cast<cudaStream_t>(stream_handle);

    // every call starts from a clean scratch block and a clean status word, whatever the previous call left behind
    cudaError_t err = cudaMemsetAsync(scratch, 0, sizeof(LayoutScratch), stream);
    if (err == cudaSuccess) err = cudaMemsetAsync(device_status, 0, sizeof(int), stream);
    if (err != cudaSuccess) return fail(DEEP_EP_NOALLOC_CUDA_ERROR, std::string("cudaMemsetAsync: ") + cudaGetErrorString(err));

    LayoutArgs args = {};
    args.topk_idx = reinterpret_cast<const int64_t*>(topk_idx);
    args.num_tokens = num_tokens, args.num_topk = num_topk, args.num_experts = num_experts, args.num_ranks = num_ranks;
    args.dst_slot_idx = dst_slot_idx, args.num_tokens_per_rank = num_tokens_per_rank;
    args.num_tokens_per_expert = num_tokens_per_expert;
    args.scratch = scratch, args.timeout_ns = 10ll * 1000000000ll, args.status = device_status;

    int grid = (num_tokens + 255) / 256;
    grid = grid < 1 ? 1 : (grid > deep_ep::kernels::kLayoutMaxCtas ? deep_ep::kernels::kLayoutMaxCtas : grid);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid), config.blockDim = dim3(256), config.dynamicSmemBytes = 0, config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative, attr[0].val.cooperative = 1;     // the kernel synchronises its CTAs
    config.attrs = attr, config.numAttrs = 1;
    err = cudaLaunchKernelEx(&config, ep_layout_noalloc_kernel, args);
    if (err != cudaSuccess) return fail(DEEP_EP_NOALLOC_CUDA_ERROR, std::string("kernel launch: ") + cudaGetErrorString(err));
    return DEEP_EP_NOALLOC_OK;
}

extern "C" __attribute__((visibility("default")))
int deep_ep_noalloc_wait_status(void* stream_handle, int* device_status_out) {
    g_last_error.clear();
    if (device_status_out == nullptr) return fail(DEEP_EP_NOALLOC_BAD_ARGUMENT, "null pointer argument");
    LayoutScratch* scratch = nullptr;
    int* device_status = nullptr;
    if (const int rc = scratch_for_current_device(&scratch, &device_status); rc != DEEP_EP_NOALLOC_OK) return rc;
    const auto stream = static_cast<cudaStream_t>(stream_handle);
    cudaError_t err = cudaMemcpyAsync(device_status_out, device_status, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return fail(DEEP_EP_NOALLOC_CUDA_ERROR, std::string("reading the status word: ") + cudaGetErrorString(err));
    if (*device_status_out != 0)
        g_last_error = "the layout kernel gave up waiting for its own thread blocks (device status " +
                       std::to_string(*device_status_out) + "); its outputs are incomplete";
    return DEEP_EP_NOALLOC_OK;
}

extern "C" __attribute__((visibility("default")))
const char* deep_ep_noalloc_last_error(void) { return g_last_error.c_str(); }
