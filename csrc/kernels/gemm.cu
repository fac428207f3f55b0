// Launcher of the grouped tcgen05 GEMM: builds the two TMA tensor maps (128-byte swizzle) and starts one
// persistent CTA per SM.
#include <algorithm>
#include <cstdlib>

#include <deep_ep/common/exception.hpp>
#include <deep_ep/kernels/grouped_gemm.cuh>
#include <deep_ep/kernels/grouped_gemm2.cuh>
#include <deep_ep/kernels/grouped_gemm_fp8.cuh>
#include <deep_ep/kernels/grouped_gemm_fp8_hw.cuh>

#include "../runtime/driver.hpp"
#include "api.hpp"

namespace deep_ep::launch {

namespace {

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with a {box_cols, box_rows} box.
CUtensorMap make_map_2d(const void* base, int64_t rows, int64_t cols, int box_cols, int box_rows) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    EP_HOST_ASSERT(reinterpret_cast<uintptr_t>(base) % 16 == 0 and (cols * 2) % 16 == 0);
    DRV_CHECK(driver::cuTensorMapEncodeTiled()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                               box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return map;
}

// 2-D byte tensor map (e4m3 operands) over a row-major [rows, cols] matrix with a {128, box_rows} box.
CUtensorMap make_map_2d_u8(const void* base, int64_t rows, int64_t cols, int box_rows) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols)};
    const cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    EP_HOST_ASSERT(reinterpret_cast<uintptr_t>(base) % 16 == 0 and cols % 16 == 0);
    DRV_CHECK(driver::cuTensorMapEncodeTiled()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                                               box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return map;
}

// One word of mapped pinned host memory that the GEMM kernels set when one of their bounded waits ran out. It is looked
// at before every launch, so a kernel that gave up (and left its output incomplete) is reported at the next call at the
// latest instead of passing silently.
struct FailureWord {
    int* host = nullptr;
    int* device = nullptr;
    FailureWord() {
        CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
        *host = 0;
        CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&device), host, 0));
    }
};

int* failure_word_checked() {
    static FailureWord word;
    if (*static_cast<volatile int*>(word.host) != 0) {
        *word.host = 0;
        throw EPException("Grouped GEMM", __FILE__, __LINE__,
                          "an earlier grouped GEMM kernel gave up waiting on one of its barriers; its output is incomplete");
    }
    return word.device;
}

}  // namespace

namespace {

// The tensor-map encoder is a driver entry point and wants a current context on the calling thread; autograd worker
// threads may not have touched the runtime yet. Done once per thread, so that later launches (for instance inside a
// CUDA-graph capture, where memory-management calls are not allowed) make no such call.
void ensure_context_once_per_thread() {
    static thread_local bool ready = false;
    if (ready) return;
    CUDA_CHECK(cudaFree(nullptr));
    ready = true;
}

}  // namespace

void grouped_gemm_fp8(kernels::GroupedGemmFp8Args args, const void* a, int64_t a_rows, const void* b, int64_t b_rows,
                      int num_sms, cudaStream_t stream) {
    using namespace kernels;
    EP_HOST_ASSERT(args.num_groups > 0 and args.num_groups <= kMaxLocalExperts);
    EP_HOST_ASSERT_MSG(args.k > 0 and args.k % kFp8BlockK == 0, "K must be a multiple of 128");
    EP_HOST_ASSERT(a_rows > 0);
    ensure_context_once_per_thread();
    args.status = failure_word_checked();
    if (args.epilogue != kEpilogueStore) {
        EP_HOST_ASSERT_MSG(args.epilogue == kEpilogueSwiGLU and args.n % 256 == 0, "SwiGLU needs N (gate + up) to be a multiple of 256");
        args.n_out = args.n / 2;
    } else {
        EP_HOST_ASSERT_MSG(args.n % kFp8BlockN == 0, "N must be a multiple of 256");
        args.n_out = args.n;
    }
    args.total_rows = static_cast<int>(a_rows);
    int device = 0, sms = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int grid = num_sms > 0 ? std::min(num_sms, sms) : sms;
    const int64_t budget = 200 * 1024;
    args.num_stages = static_cast<int>(std::min<int64_t>(kGemmMaxStages, (budget - 1024) / ((kGemmBlockM + kFp8BlockN) * kFp8BlockK)));
    const CUtensorMap map_a = make_map_2d_u8(a, a_rows, args.k, 128);
    const CUtensorMap map_b = make_map_2d_u8(b, b_rows, args.k, 128);
    const auto smem = grouped_gemm_fp8_smem_bytes(args.num_stages);
    if (args.sf_b_e8 != nullptr) {
        // hardware-scaled variant: UE8M0 scale bytes (A may also come as fp32 powers of two), whole groups of four K blocks
        EP_HOST_ASSERT_MSG(args.k % (kFp8BlockK * kFp8SfGroup) == 0, "the hardware-scaled FP8 GEMM needs K to be a multiple of 512");
        EP_HOST_ASSERT((args.sf_a_e8 != nullptr) != (args.sf_a != nullptr));
        EP_HOST_ASSERT(reinterpret_cast<uintptr_t>(args.sf_a_e8) % 4 == 0 and reinterpret_cast<uintptr_t>(args.sf_a) % 16 == 0 and
                       reinterpret_cast<uintptr_t>(args.sf_b_e8) % 4 == 0);
        CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_fp8_hw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        grouped_gemm_fp8_hw_kernel<<<grid, kFp8ThreadsRegSplit, smem, stream>>>(map_a, map_b, args);
    } else if (args.reg_split) {
        CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        grouped_gemm_fp8_kernel<true><<<grid, kFp8ThreadsRegSplit, smem, stream>>>(map_a, map_b, args);
    } else {
        CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        grouped_gemm_fp8_kernel<false><<<grid, kFp8Threads, smem, stream>>>(map_a, map_b, args);
    }
    CUDA_CHECK(cudaGetLastError());
}

namespace {

// Tensor map over a result matrix [rows, cols] whose box is 32 rows of 128 bytes (128-byte swizzle): the unit an epilogue
// warp hands to the TMA store / reduce-add
CUtensorMap make_map_out(const void* base, int64_t rows, int64_t cols, CUtensorMapDataType type, int element_bytes) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * element_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / element_bytes), 32};
    const cuuint32_t elem_strides[2] = {1, 1};
    EP_HOST_ASSERT(reinterpret_cast<uintptr_t>(base) % 16 == 0 and (cols * element_bytes) % 16 == 0);
    DRV_CHECK(driver::cuTensorMapEncodeTiled()(&map, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return map;
}
// fp32 weight gradients: 32 x 32 box
CUtensorMap make_map_2d_f32(const void* base, int64_t rows, int64_t cols) {
    return make_map_out(base, rows, cols, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4);
}
// the same for bf16 results: 32 rows x 64 columns
CUtensorMap make_map_2d_bf16_out(const void* base, int64_t rows, int64_t cols) {
    return make_map_out(base, rows, cols, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
}

// staging chunk of one epilogue warp (32 rows x 128 bytes); four warps, one or two chunks each, behind the operand ring
constexpr int64_t kStagingChunkBytes = 4096;

}  // namespace

void grouped_gemm(kernels::GroupedGemmArgs args, const void* a, int64_t a_rows, int64_t a_cols,
                  const void* b, int64_t b_rows, int64_t b_cols, int num_sms, cudaStream_t stream, bool use_pairs) {
    using namespace kernels;
    EP_HOST_ASSERT(args.num_groups > 0 and args.num_groups <= kMaxLocalExperts);
    ensure_context_once_per_thread();
    args.status = failure_word_checked();
    if (args.epilogue != kEpilogueStore) {
        EP_HOST_ASSERT(args.mode == kModeForward and args.n % 256 == 0);
        args.block_n = 256, args.block_n_out = 128, args.n_out = args.n / 2;
    } else {
        args.block_n = args.n % 256 == 0 ? 256 : 128;
        EP_HOST_ASSERT_MSG(args.n % args.block_n == 0, "N must be a multiple of 128");
        args.block_n_out = args.block_n, args.n_out = args.n;
    }
    if (args.mode == kModeWgrad) EP_HOST_ASSERT(args.m % kGemmBlockM == 0);

    int device = 0, sms = 0;
    CUDA_CHECK(cudaGetDevice(&device));
    CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    int grid = num_sms > 0 ? std::min(num_sms, sms) : sms;
    const int64_t budget = 216 * 1024;      // dynamic shared memory: operand ring + staging; 227 KiB minus the kernel's static 4 KiB is the limit
    // Results leave through staging buffers and the TMA (tiled store; reduce-add for accumulated fp32 weight gradients)
    // except those that need a per-row decision or another element type: rows sent to a combine route, the SwiGLU
    // epilogues, fp32 forward results. Weight gradients (few K blocks per tile) take two buffers per warp, the others one,
    // which keeps the operand ring at its depth.
    const bool wgrad_fp32 = args.mode == kModeWgrad and not args.out_bf16;
    const bool tma_out = args.mode == kModeWgrad or (args.epilogue == kEpilogueStore and args.route == nullptr and not args.out_fp32);
    args.staging_buffers = not tma_out ? 0 : (args.mode == kModeWgrad ? 2 : 1);
    const int64_t staging = 4 * args.staging_buffers * kStagingChunkBytes;
    const int64_t d_rows = args.mode == kModeWgrad ? int64_t(args.num_groups) * args.m : a_rows;

    // CTA pairs (256 x 256 tiles) whenever the shape allows it; the single-CTA kernel covers the rest
    const bool pair = use_pairs and args.block_n == 256 and grid >= 2 and not args.out_fp32 and (args.mode != kModeWgrad or args.m % 256 == 0);
    if (pair) {
        grid -= grid % 2;
        args.num_stages = static_cast<int>(std::min<int64_t>(kGemmMaxStages, (budget - 1024 - staging) / (2 * 128 * kGemmBlockK * 2)));
        const CUtensorMap map_a = args.mode == kModeWgrad ? make_map_2d(a, a_rows, a_cols, 64, 64) : make_map_2d(a, a_rows, a_cols, 64, 128);
        const CUtensorMap map_b = args.mode == kModeForward ? make_map_2d(b, b_rows, b_cols, 64, 128) : make_map_2d(b, b_rows, b_cols, 64, 64);
        const CUtensorMap map_d = not tma_out ? map_a : (wgrad_fp32 ? make_map_2d_f32(args.d, d_rows, args.n) : make_map_2d_bf16_out(args.d, d_rows, args.n_out));
        const auto smem = int64_t(args.num_stages) * 2 * 128 * kGemmBlockK * 2 + 1024 + staging;
        CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        grouped_gemm_pair_kernel<<<grid, 192, smem, stream>>>(map_a, map_b, map_d, args);
        CUDA_CHECK(cudaGetLastError());
        return;
    }

    args.num_stages = static_cast<int>(std::min<int64_t>(kGemmMaxStages, (budget - 1024 - staging) / ((kGemmBlockM + args.block_n) * kGemmBlockK * 2)));
    EP_HOST_ASSERT(args.num_stages >= 2);
    // A: K-major activations (box 64 x 128) or, for wgrad, MN-major (box 64 x 64)
    const CUtensorMap map_a = args.mode == kModeWgrad ? make_map_2d(a, a_rows, a_cols, 64, 64) : make_map_2d(a, a_rows, a_cols, 64, 128);
    // B: K-major weights (box 64 x 128) for forward, MN-major (box 64 x 64) otherwise
    const CUtensorMap map_b = args.mode == kModeForward ? make_map_2d(b, b_rows, b_cols, 64, 128) : make_map_2d(b, b_rows, b_cols, 64, 64);
    const CUtensorMap map_d = not tma_out ? map_a : (wgrad_fp32 ? make_map_2d_f32(args.d, d_rows, args.n) : make_map_2d_bf16_out(args.d, d_rows, args.n_out));
    const auto smem = grouped_gemm_smem_bytes(args.block_n, args.num_stages) + staging;
    CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    grouped_gemm_kernel<<<grid, 192, smem, stream>>>(map_a, map_b, map_d, args);
    CUDA_CHECK(cudaGetLastError());
}

}  // namespace deep_ep::launch
