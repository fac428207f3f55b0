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
    int staging_buffers;      // chunk buffers per epilogue warp for results that leave through the TMA (0 = none: register stores)
    int out_fp32;             // forward / dgrad with the plain-store epilogue: 1 = d is fp32 [rows, n_out] (single-CTA kernel only)
    int accumulate;           // wgrad: 1 = add to the existing contents of d, 0 = overwrite (experts without rows get zeros)
    void* d;                  // bf16 [rows, n_out] (forward/dgrad) or fp32 [G, m, n] accumulated into (wgrad)
    void* d2;                 // kEpilogueSwiGLUKeep: bf16 [rows, n] pre-activation output
    const float* row_scale;   // optional fp32 [rows] factor applied by the SwiGLU epilogues
    int alignment;            // expert alignment: rows in [count, align(count)) of a tile are written as zeros
    int* status;              // set to 1 if a bounded wait ran out (may be nullptr)
    // Plain-store epilogue only (forward / dgrad): optional [rows] table of destination addresses. A non-zero entry
    // is where row r's n_out bf16 values go INSTEAD of d (local or a peer's memory: the combine landing slot of a
    // token that has only this one row on this rank, see `ep_route.cuh`); zero = store into d as usual.
    const unsigned long long* route;
};

EP_HOST_DEVICE int64_t grouped_gemm_smem_bytes(int block_n, int num_stages) {
    return int64_t(num_stages) * (kGemmBlockM + block_n) * kGemmBlockK * 2 + 1024;
}

// ---------------------------------------------------------------- FP8 (e4m3) block-scaled forward GEMM
// A: e4m3 [rows, k] with one fp32 scale per row and 128 columns (the format the FP8 dispatch delivers);
// B: e4m3 [G, n, k] with one fp32 scale per 128 x 128 block. K blocks of 128 are multiplied on the tensor cores
// and promoted into fp32 registers with `sf_a[row, kb] * sf_b[g, n / 128, kb]`.
constexpr int kFp8BlockK = 128;        // 128 e4m3 = one 128-byte swizzle row = one scale block
constexpr int kFp8BlockN = 256;        // accumulator columns per tile
constexpr int kFp8Threads = 320;       // producer warp, MMA warp, eight promotion/epilogue warps
constexpr int kFp8ThreadsRegSplit = 384;   // the same plus two idle warps: three warpgroups that re-split the register file

struct GroupedGemmFp8Args {
    int epilogue;             // kEpilogueStore: d = bf16 [rows, n]; kEpilogueSwiGLU: d = silu(gate) * up (* row_scale), [rows, n / 2]
    int out_fp8;              // SwiGLU only: 1 = d is e4m3 [rows, n / 2] and d_sf receives fp32 [rows, n / 256] scales
    int num_groups;
    const int* psum;          // [G] end (exclusive) of each expert's rows; start = psum - count
    const int* count;         // [G] exact rows per expert
    int total_rows;           // rows of A (scale reads are clamped to it)
    int n, k, n_out;
    int num_stages;
    const float* sf_a;        // [rows, k / 128]
    const float* sf_b;        // [G, n / 128, k / 128]
    void* d;
    float* d_sf;
    const float* row_scale;   // optional fp32 [rows] factor applied by the SwiGLU epilogue
    int alignment;            // rows in [count, align(count)) of a tile are written as zeros
    int* status;              // set to 1 if a bounded wait ran out (may be nullptr)
    int reg_split;            // 1: 384-thread kernel that moves registers to the promotion warps (`setmaxnreg`)
    // hardware-scaled variant (UE8M0 = power-of-two scales, one byte each, applied by the tensor core)
    const uint8_t* sf_a_e8;   // [rows, k / 128]
    const uint8_t* sf_b_e8;   // [G, n / 128, k / 128]
    uint8_t* d_sf_e8;         // SwiGLU with e4m3 output: [rows, n / 256]
    // plain-store epilogue of the hardware-scaled kernel: optional destination table, see GroupedGemmArgs::route
    const unsigned long long* route;
};

constexpr int kFp8SfGroup = 4;             // K blocks whose scale bytes share one 32-bit tensor-memory column
constexpr int kFp8SfStages = 4;            // shared-memory stages of re-laid-out scale factors
constexpr int kFp8SfStageBytes = 3 * 512;  // one 128-row atom for A, two for the 256 columns of B

EP_HOST_DEVICE int64_t grouped_gemm_fp8_smem_bytes(int num_stages) {
    return int64_t(num_stages) * (kGemmBlockM + kFp8BlockN) * kFp8BlockK + 1024;
}

}  // namespace deep_ep::kernels
