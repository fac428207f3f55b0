// Per-token BF16 -> e4m3 quantisation with one fp32 scale per 128 columns (the 1x128 format of the FP8
// dispatch), as a standalone kernel body with the hidden size as a compile-time constant. It is compiled at run
// time for the hidden size in use (see `deep_ep/ops/quant.py`), which is how shape-specialised kernels are
// produced in this library; the math is bit-identical to the quantiser fused into the dispatch kernel and to
// `deep_ep.utils.math.per_token_cast_to_fp8` on CUDA tensors.
#pragma once

#include "../device/ptx.cuh"

namespace deep_ep::kernels {

// One warp per row. `kHidden` must be a multiple of 128.
template <int kHidden>
EP_DEVICE void per_token_quant_body(const __nv_bfloat16* x, uint8_t* q, float* sf, int num_rows) {
    static_assert(kHidden % 128 == 0, "hidden must be a multiple of 128");
    constexpr int kIters = (kHidden + 255) / 256;
    const int lane = ptx::lane_id();
    const int warps = (gridDim.x * blockDim.x) / 32;
    for (int row = (blockIdx.x * blockDim.x + threadIdx.x) / 32; row < num_rows; row += warps) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(x + int64_t(row) * kHidden);
        int4 raw[kIters];
        #pragma unroll
        for (int it = 0; it < kIters; ++it) {
            const int col = it * 256 + lane * 8;
            raw[it] = col < kHidden ? ptx::ld_nc_v4(src + col * 2) : make_int4(0, 0, 0, 0);
        }
        #pragma unroll
        for (int it = 0; it < kIters; ++it) {
            const int col = it * 256 + lane * 8;
            float v[8];
            const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw[it]);
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = ptx::bf16x2_to_float2(w[i]);
                v[2 * i] = f.x, v[2 * i + 1] = f.y;
            }
            float amax = 0.f;
            #pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            #pragma unroll
            for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            amax = fmaxf(amax, 1e-4f);
            const float inv = __fmul_rn(__frcp_rn(amax), 448.0f);
            if (col < kHidden) {
                uint2 packed;
                packed.x = ptx::float2_to_e4m3x2(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv)) |
                           (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[2], inv), __fmul_rn(v[3], inv))) << 16);
                packed.y = ptx::float2_to_e4m3x2(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv)) |
                           (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[6], inv), __fmul_rn(v[7], inv))) << 16);
                *reinterpret_cast<uint2*>(q + int64_t(row) * kHidden + col) = packed;
                if ((lane & 15) == 0) sf[int64_t(row) * (kHidden / 128) + col / 128] = __fmul_rn(amax, 1.0f / 448.0f);
            }
        }
    }
}

}  // namespace deep_ep::kernels
