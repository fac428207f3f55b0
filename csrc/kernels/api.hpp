// Host-callable launchers of the sm_100a kernels (defined in `launch.cu`, compiled by nvcc).
// Same role as the reference's `csrc/kernels/**` launchers: choose grid, shared memory and
// pipeline depth, then launch on the given stream.
#pragma once

#include <cuda_runtime.h>

#include <functional>

#include <deep_ep/kernels/ep_args.hpp>
#include <deep_ep/kernels/ep_layout_args.hpp>
#include <deep_ep/kernels/grouped_gemm_args.hpp>
#include <deep_ep/kernels/misc_args.hpp>

namespace deep_ep::launch {

struct PipelineConfig {
    int num_warps;
    int num_stages;
    int64_t smem_bytes;
};

// Largest warp/stage combination that fits the opt-in shared memory of one CTA.
PipelineConfig choose_dispatch_config(int token_bytes, int src_row_bytes, int num_topk, int num_experts);
PipelineConfig choose_expand_config(int token_bytes, int num_topk, int num_local_experts);
PipelineConfig choose_combine_config(int token_bytes);

// Shape-specialised variants of the four EP kernels (optional): when a provider is installed and returns a driver function
// (`CUfunction`, passed as `void*`) for a kernel name ("dispatch", "expand", "combine", "reduce") and shape, the launchers
// below start that function instead of the generic kernel linked into this library; the argument block is the same.
struct EPShape {
    int num_ranks, num_topk, hidden_bytes, num_experts;
};
using SpecializedKernelProvider = std::function<void*(const char* kernel, const EPShape& shape)>;
void set_specialized_kernel_provider(SpecializedKernelProvider provider);

void dispatch(kernels::DispatchArgs args, int num_sms, cudaStream_t stream);
void dispatch_expand(kernels::ExpandArgs args, int num_sms, cudaStream_t stream);
void combine(kernels::CombineArgs args, int num_sms, cudaStream_t stream);
void combine_reduce(kernels::CombineReduceArgs args, int num_sms, cudaStream_t stream);
// Fills `args.route` (zero-initialised by the caller) with the landing address of every single-row token's row.
void combine_route(const kernels::CombineRouteArgs& args, cudaStream_t stream);

void barrier(const kernels::BarrierArgs& args, cudaStream_t stream);
void engram_fetch(const kernels::EngramFetchArgs& args, int num_sms, cudaStream_t stream);
void all_gather(const kernels::AllGatherArgs& args, int num_sms, cudaStream_t stream);
// Batched in-place reduce-scatter (`args.all_reduce == 0`) or all-reduce over symmetric tensors.
void bucket_reduce(const kernels::BucketReduceArgs& args, int num_sms, cudaStream_t stream);
void pp_send(const kernels::PPArgs& args, int num_sms, cudaStream_t stream);
void pp_recv(const kernels::PPArgs& args, int num_sms, cudaStream_t stream);
void lb_exchange(const kernels::LBArgs& args, int num_sms, cudaStream_t stream);

// Standalone routing layout (cooperative launch, at most `kLayoutMaxCtas` CTAs). `args.scratch` must point to a
// zero-initialised `LayoutScratch` in device memory.
void dispatch_layout(const kernels::LayoutArgs& args, int num_sms, cudaStream_t stream);

// Grouped BF16 GEMM on tcgen05 tensor cores over the expanded layout. `a`/`b` are row-major bf16 matrices
// ([a_rows, a_cols], [b_rows, b_cols]); their roles depend on `args.mode` (see grouped_gemm.cuh). `use_pairs` selects
// the CTA-pair kernel (`cta_group::2`, 256 x 256 tiles) when the shape allows it.
void grouped_gemm(kernels::GroupedGemmArgs args, const void* a, int64_t a_rows, int64_t a_cols,
                  const void* b, int64_t b_rows, int64_t b_cols, int num_sms, cudaStream_t stream, bool use_pairs = false);

// Grouped FP8 (e4m3) forward GEMM with fp32 block scales (1 x 128 for `a`, 128 x 128 for `b`), see grouped_gemm_fp8.cuh.
// `a` is [a_rows, args.k] bytes, `b` is [b_rows = G * args.n, args.k] bytes.
void grouped_gemm_fp8(kernels::GroupedGemmFp8Args args, const void* a, int64_t a_rows, const void* b, int64_t b_rows,
                      int num_sms, cudaStream_t stream);

// dh = d(silu(gate) * up * row_scale) / d[gate | up] for bf16 rows; `inter` must be a multiple of 8.
void swiglu_backward(const void* h, const void* dact, const float* row_scale, void* dh, int64_t rows, int inter,
                     cudaStream_t stream);

// FP8 training path. Row-wise e4m3 quantisation of bf16 `x [rows, cols]` with one power-of-two scale (UE8M0 byte) per 128
// columns; the SwiGLU of `h = [gate | up]` (times `row_scale`) as bf16 (`act`, optional) and quantised the same way; and
// weights `w [rows, cols]` (stacked matrices of `n` rows) with one scale per 128 x 128 block plus, optionally, every matrix
// transposed (`qt [rows / n, cols, n]`, `sft [rows / n, cols / 128, n / 128]`).
void row_quant_ue8m0(const void* x, void* q, void* sf, int64_t rows, int cols, cudaStream_t stream);
void swiglu_quant_ue8m0(const void* h, const float* row_scale, void* act, void* q, void* sf, int64_t rows, int inter,
                        cudaStream_t stream);
void block_quant_ue8m0(const void* w, void* q, void* sf, void* qt, void* sft, int64_t rows, int cols, int n, cudaStream_t stream);

// Test hook: a one-warp kernel that waits (bounded) for a flag nobody sets and records the status.
void bounded_wait_probe(layout::CommonSignals* cs, layout::HostStatus* host_status, long long timeout_ns,
                        cudaStream_t stream);

}  // namespace deep_ep::launch
