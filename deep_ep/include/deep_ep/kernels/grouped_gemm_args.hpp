// Plain-data arguments of the grouped GEMM kernel (usable from g++ and nvcc).
#pragma once

#include "../common/math.hpp"

namespace deep_ep::kernels {

constexpr int kGemmBlockM = 128;
constexpr int kGemmBlockK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmMaxStages = 8;

enum GroupedGemmMode : int { kModeForward = 0, kModeDgrad = 1, kModeWgrad = 2 };
// kEpilogueSwiGLU: d = silu(gate) * up (* row_scale). kEpilogueSwiGLUKeep: additionally stores the pre-activation
// [gate | up] into d2 for the backward pass.
enum GroupedGemmEpilogue : int { kEpilogueStore = 0, kEpilogueSwiGLU = 1, kEpilogueSwiGLUKeep = 2 };

struct GroupedGemmArgs {
    int mode, epilogue;
    int num_groups;
    const int* psum;          // [G] end (exclusive) of each expert's rows; start = psum - count
    const int* count;         // [G] exact rows per expert
    int m;                    // wgrad: rows of each per-expert output
    int n;                    // columns of B per expert (forward: rows of the K-major weight)
    int k;                    // forward/dgrad: contraction length
    int n_out;                // columns of D (n, or n / 2 with the SwiGLU epilogue)
    int block_n;              // accumulator columns per tile (128 or 256)
    int block_n_out;          // output columns per tile
    int num_stages;
    int out_bf16;             // wgrad: 1 = d is bf16 (overwrite only), 0 = d is fp32
    int accumulate;           // wgrad: 1 = add to the existing contents of d, 0 = overwrite (experts without rows get zeros)
    void* d;                  // bf16 [rows, n_out] (forward/dgrad) or fp32 [G, m, n] accumulated into (wgrad)
    void* d2;                 // kEpilogueSwiGLUKeep: bf16 [rows, n] pre-activation output
    const float* row_scale;   // optional fp32 [rows] factor applied by the SwiGLU epilogues
    int alignment;            // expert alignment: rows in [count, align(count)) of a tile are written as zeros
    int* status;              // set to 1 if a bounded wait ran out (may be nullptr)
};

EP_HOST_DEVICE int64_t grouped_gemm_smem_bytes(int block_n, int num_stages) {
    return int64_t(num_stages) * (kGemmBlockM + block_n) * kGemmBlockK * 2 + 1024;
}

}  // namespace deep_ep::kernels
