// Launchers for the sm_100a kernels. Persistent kernels that synchronise their CTAs are launched
// cooperatively so that every CTA is resident; the grid never exceeds the SM count.
#include <algorithm>
#include <string>

#include <deep_ep/common/exception.hpp>
#include <deep_ep/kernels/elementwise.cuh>
#include <deep_ep/kernels/ep_combine.cuh>
#include <deep_ep/kernels/ep_dispatch.cuh>
#include <deep_ep/kernels/ep_expand.cuh>
#include <deep_ep/kernels/ep_layout.cuh>
#include <deep_ep/kernels/ep_route.cuh>
#include <deep_ep/kernels/misc.cuh>

#include "../runtime/driver.hpp"
#include "api.hpp"

namespace deep_ep::launch {

namespace {

SpecializedKernelProvider& specialized_provider() {
    static SpecializedKernelProvider provider;
    return provider;
}

// Launch of a run-time compiled kernel that takes the same by-value argument block as its generic counterpart.
template <typename Args>
void launch_function(void* function, const Args& args, int grid, int block, int64_t smem, bool cooperative, cudaStream_t stream) {
    const auto fn = static_cast<CUfunction>(function);
    if (smem > 48 * 1024)
        DRV_CHECK(driver::cuFuncSetAttribute()(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, static_cast<int>(smem)));
    CUlaunchConfig config = {};
    config.gridDimX = grid, config.gridDimY = 1, config.gridDimZ = 1;
    config.blockDimX = block, config.blockDimY = 1, config.blockDimZ = 1;
    config.sharedMemBytes = static_cast<unsigned>(smem), config.hStream = stream;
    CUlaunchAttribute attr[1];
    attr[0].id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE, attr[0].value.cooperative = cooperative ? 1 : 0;
    config.attrs = attr, config.numAttrs = 1;
    void* params[1] = {const_cast<Args*>(&args)};
    DRV_CHECK(driver::cuLaunchKernelEx()(&config, fn, params, nullptr));
}

// The generic kernel, or its shape-specialised variant when a provider offers one.
template <typename Kernel, typename Args>
void launch_ep_kernel(const char* name, const EPShape& shape, Kernel kernel, const Args& args, int grid, int block, int64_t smem,
                      bool cooperative, cudaStream_t stream);

constexpr int64_t kSmemBudget = 200 * 1024;   // of the 227 KiB a CTA may opt into

template <typename Kernel, typename Args>
void launch_kernel(Kernel kernel, const Args& args, int grid, int block, int64_t smem, bool cooperative,
                   cudaStream_t stream) {
    if (smem > 48 * 1024)
        CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid), config.blockDim = dim3(block);
    config.dynamicSmemBytes = static_cast<size_t>(smem), config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative, attr[0].val.cooperative = cooperative ? 1 : 0;
    config.attrs = attr, config.numAttrs = 1;
    CUDA_CHECK(cudaLaunchKernelEx(&config, kernel, args));
}

template <typename Kernel, typename Args>
void launch_ep_kernel(const char* name, const EPShape& shape, Kernel kernel, const Args& args, int grid, int block, int64_t smem,
                      bool cooperative, cudaStream_t stream) {
    void* function = specialized_provider() ? specialized_provider()(name, shape) : nullptr;
    if (function != nullptr) launch_function(function, args, grid, block, smem, cooperative, stream);
    else launch_kernel(kernel, args, grid, block, smem, cooperative, stream);
}

int clamp_sms(int num_sms) {
    int device = 0, count = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    CUDA_CHECK(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device));
    return std::max(1, std::min({num_sms, count, kMaxCtas}));
}

}  // namespace

void set_specialized_kernel_provider(SpecializedKernelProvider provider) { specialized_provider() = std::move(provider); }

PipelineConfig choose_dispatch_config(int token_bytes, int src_row_bytes, int num_topk, int num_experts) {
    for (int stages : {3, 2}) {
        for (int warps = 8; warps >= 2; --warps) {
            const auto bytes = kernels::dispatch_detail::smem_bytes(warps, stages, num_topk, num_experts, token_bytes, src_row_bytes);
            if (bytes <= kSmemBudget and (warps >= 4 or stages == 2)) return {warps, stages, bytes};
        }
    }
    EP_HOST_UNREACHABLE("dispatch message too large for shared memory: " + std::to_string(token_bytes) + " bytes");
}

PipelineConfig choose_expand_config(int token_bytes, int num_topk, int num_local_experts) {
    for (int stages : {3, 2}) {
        for (int warps = 8; warps >= 2; --warps) {
            const auto bytes = kernels::expand_detail::smem_bytes(warps, stages, num_topk, num_local_experts, token_bytes);
            if (bytes <= kSmemBudget and (warps >= 4 or stages == 2)) return {warps, stages, bytes};
        }
    }
    EP_HOST_UNREACHABLE("dispatch message too large for shared memory: " + std::to_string(token_bytes) + " bytes");
}

PipelineConfig choose_combine_config(int token_bytes) {
    // two stages per warp are enough to overlap a row's store with the next row's loads; warps matter more
    for (int stages : {2}) {
        for (int warps = 8; warps >= 2; --warps) {
            const auto bytes = kernels::combine_detail::smem_bytes(warps, stages, token_bytes);
            if (bytes <= kSmemBudget and (warps >= 4 or stages == 2)) return {warps, stages, bytes};
        }
    }
    EP_HOST_UNREACHABLE("combine message too large for shared memory: " + std::to_string(token_bytes) + " bytes");
}

void dispatch(kernels::DispatchArgs args, int num_sms, cudaStream_t stream) {
    const layout::DispatchTokenLayout tl(args.hidden_bytes, args.sf_bytes, args.num_topk);
    const auto config = choose_dispatch_config(tl.num_bytes(), args.fused_quant ? args.hidden_bytes * 2 : 0,
                                               args.num_topk, args.num_experts);
    args.num_warps = config.num_warps, args.num_stages = config.num_stages;
    launch_ep_kernel("dispatch", {args.peers.num_ranks, args.num_topk, args.hidden_bytes, args.num_experts}, kernels::ep_dispatch_kernel,
                     args, clamp_sms(num_sms), 32 * (config.num_warps + 1), config.smem_bytes, true, stream);
}

void dispatch_expand(kernels::ExpandArgs args, int num_sms, cudaStream_t stream) {
    const layout::DispatchTokenLayout tl(args.hidden_bytes, args.sf_bytes, args.num_topk);
    const auto config = choose_expand_config(tl.num_bytes(), args.num_topk, args.num_experts / args.num_ranks);
    args.num_warps = config.num_warps, args.num_stages = config.num_stages;
    launch_ep_kernel("expand", {args.num_ranks, args.num_topk, args.hidden_bytes, args.num_experts}, kernels::ep_dispatch_expand_kernel,
                     args, clamp_sms(num_sms), 32 * config.num_warps, config.smem_bytes, true, stream);
}

void combine(kernels::CombineArgs args, int num_sms, cudaStream_t stream) {
    const layout::CombineTokenLayout tl(args.hidden_bytes, args.num_topk);
    const auto config = choose_combine_config(tl.num_bytes());
    args.num_warps = config.num_warps, args.num_stages = config.num_stages;
    launch_ep_kernel("combine", {args.peers.num_ranks, args.num_topk, args.hidden_bytes, 0}, kernels::ep_combine_kernel,
                     args, clamp_sms(num_sms), 32 * config.num_warps, config.smem_bytes, true, stream);
}

void combine_route(const kernels::CombineRouteArgs& args, cudaStream_t stream) {
    const int blocks = std::max(1, std::min((args.num_metadata_rows + 255) / 256, 592));
    launch_kernel(kernels::ep_combine_route_kernel, args, blocks, 256, 0, false, stream);
}

void combine_reduce(kernels::CombineReduceArgs args, int num_sms, cudaStream_t stream) {
    // not cooperative: oversubscribe the SMs so that enough loads are in flight
    const EPShape shape = {args.num_ranks, args.num_topk, args.hidden_bytes, args.num_experts};
    if (std::min(args.num_topk, args.num_ranks) <= 2)
        launch_ep_kernel("reduce", shape, kernels::ep_combine_reduce_few_rows_kernel, args, clamp_sms(num_sms) * 4, 256, 0, false, stream);
    else
        launch_ep_kernel("reduce", shape, kernels::ep_combine_reduce_kernel, args, clamp_sms(num_sms) * 6, 256, 0, false, stream);
}

namespace {
__global__ void __launch_bounds__(256, 1) ep_layout_kernel(const __grid_constant__ kernels::LayoutArgs a) {
    kernels::ep_layout_body(a);
}
}  // namespace

void dispatch_layout(const kernels::LayoutArgs& args, int num_sms, cudaStream_t stream) {
    EP_HOST_ASSERT(args.num_experts <= kMaxExperts and args.num_ranks <= kMaxRanks and args.num_topk <= kMaxTopk);
    EP_HOST_ASSERT(args.num_ranks > 0 and args.num_experts % args.num_ranks == 0);
    const int grid = std::max(1, std::min({num_sms > 0 ? num_sms : kernels::kLayoutMaxCtas, kernels::kLayoutMaxCtas,
                                           (args.num_tokens + 255) / 256 > 0 ? (args.num_tokens + 255) / 256 : 1}));
    launch_kernel(ep_layout_kernel, args, grid, 256, 0, true, stream);
}

void barrier(const kernels::BarrierArgs& args, cudaStream_t stream) {
    launch_kernel(kernels::rank_barrier_kernel, args, 1, 32, 0, false, stream);
}

void engram_fetch(const kernels::EngramFetchArgs& args, int num_sms, cudaStream_t stream) {
    launch_kernel(kernels::engram_fetch_kernel, args, clamp_sms(num_sms) * 4, 256, 0, false, stream);
}

void all_gather(const kernels::AllGatherArgs& args, int num_sms, cudaStream_t stream) {
    launch_kernel(kernels::bucket_all_gather_kernel, args, clamp_sms(num_sms), 256, dev::bulk_copy_smem_bytes(8), true, stream);
}

void bucket_reduce(const kernels::BucketReduceArgs& args, int num_sms, cudaStream_t stream) {
    const int sms = clamp_sms(num_sms);
    if (args.use_multicast) {
        EP_HOST_ASSERT(args.peers.mc_base != nullptr);
        launch_kernel(kernels::bucket_reduce_multicast_kernel, args, sms, 256, 0, true, stream);
        return;
    }
    switch (args.peers.num_ranks) {
        case 1: launch_kernel(kernels::bucket_reduce_kernel<1>, args, sms, 256, 0, true, stream); break;
        case 2: launch_kernel(kernels::bucket_reduce_kernel<2>, args, sms, 256, 0, true, stream); break;
        case 4: launch_kernel(kernels::bucket_reduce_kernel<4>, args, sms, 256, 0, true, stream); break;
        case 8: launch_kernel(kernels::bucket_reduce_kernel<8>, args, sms, 256, 0, true, stream); break;
        default: launch_kernel(kernels::bucket_reduce_kernel<0>, args, sms, 256, 0, true, stream); break;
    }
}

void pp_send(const kernels::PPArgs& args, int num_sms, cudaStream_t stream) {
    launch_kernel(kernels::pp_send_kernel, args, clamp_sms(num_sms), 256, dev::bulk_copy_smem_bytes(8), true, stream);
}

void pp_recv(const kernels::PPArgs& args, int num_sms, cudaStream_t stream) {
    launch_kernel(kernels::pp_recv_kernel, args, clamp_sms(num_sms), 256, dev::bulk_copy_smem_bytes(8), true, stream);
}

void swiglu_backward(const void* h, const void* dact, const float* row_scale, void* dh, int64_t rows, int inter,
                     cudaStream_t stream) {
    EP_HOST_ASSERT(inter % 8 == 0);
    if (rows == 0) return;
    const kernels::SwiGLUBackwardArgs args = {static_cast<const uint8_t*>(h), static_cast<const uint8_t*>(dact), row_scale,
                                              static_cast<uint8_t*>(dh), rows, inter};
    const int64_t blocks = std::min<int64_t>((rows * (inter / 8) + 255) / 256, 148 * 16);
    launch_kernel(kernels::swiglu_backward_kernel, args, static_cast<int>(blocks), 256, 0, false, stream);
}

void row_quant_ue8m0(const void* x, void* q, void* sf, int64_t rows, int cols, cudaStream_t stream) {
    EP_HOST_ASSERT(cols > 0 and cols % 128 == 0);
    if (rows == 0) return;
    const kernels::RowQuantArgs args = {static_cast<const uint8_t*>(x), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), rows, cols};
    const int64_t blocks = std::min<int64_t>((rows + 7) / 8, 148 * 8);
    launch_kernel(kernels::row_quant_ue8m0_kernel, args, static_cast<int>(blocks), 256, 0, false, stream);
}

void swiglu_quant_ue8m0(const void* h, const float* row_scale, void* act, void* q, void* sf, int64_t rows, int inter,
                        cudaStream_t stream) {
    EP_HOST_ASSERT(inter > 0 and inter % 128 == 0);
    if (rows == 0) return;
    const kernels::SwiGLUQuantArgs args = {static_cast<const uint8_t*>(h), row_scale, static_cast<uint8_t*>(act),
                                           static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), rows, inter};
    const int64_t blocks = std::min<int64_t>((rows + 7) / 8, 148 * 8);
    launch_kernel(kernels::swiglu_quant_ue8m0_kernel, args, static_cast<int>(blocks), 256, 0, false, stream);
}

void block_quant_ue8m0(const void* w, void* q, void* sf, void* qt, void* sft, int64_t rows, int cols, int n, cudaStream_t stream) {
    EP_HOST_ASSERT(cols > 0 and cols % 128 == 0 and n > 0 and n % 128 == 0 and rows % n == 0);
    EP_HOST_ASSERT((qt == nullptr) == (sft == nullptr) and rows / 128 <= 65535);
    if (rows == 0) return;
    const kernels::BlockQuantArgs args = {static_cast<const uint8_t*>(w), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf),
                                          static_cast<uint8_t*>(qt), static_cast<uint8_t*>(sft), rows, cols, n};
    kernels::block_quant_ue8m0_kernel<<<dim3(cols / 128, static_cast<unsigned>(rows / 128)), 256, 0, stream>>>(args);
    CUDA_CHECK(cudaGetLastError());
}

void lb_exchange(const kernels::LBArgs& args, int num_sms, cudaStream_t stream) {
    launch_kernel(kernels::lb_exchange_kernel, args, clamp_sms(num_sms), 512, 0, true, stream);
}

namespace {

struct ProbeArgs {
    layout::CommonSignals* cs;
    layout::HostStatus* hs;
    long long timeout_ns;
};

__global__ void bounded_wait_probe_kernel(const __grid_constant__ ProbeArgs a) {
    // waits for a generation change that no one produces; must give up and record a status
    const unsigned gen = ptx::ld_acquire_gpu(&a.cs->grid_gen);
    const dev::Deadline deadline(a.timeout_ns);
    const bool ok = dev::spin_until(deadline, [&]() { return ptx::ld_acquire_gpu(&a.cs->grid_gen) != gen; });
    if (not ok) dev::report_status(a.cs, a.hs, kStatusGridSyncTimeout, -1, -1, /*where=*/99, gen + 1, gen);
}

}  // namespace

void bounded_wait_probe(layout::CommonSignals* cs, layout::HostStatus* host_status, long long timeout_ns,
                        cudaStream_t stream) {
    const ProbeArgs args = {cs, host_status, timeout_ns};
    launch_kernel(bounded_wait_probe_kernel, args, 1, 32, 0, false, stream);
}

}  // namespace deep_ep::launch
