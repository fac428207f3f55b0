// Elementwise kernels of the MoE layer that are not worth a GEMM epilogue of their own.
#pragma once

#include "../device/ptx.cuh"

namespace deep_ep::kernels {

struct SwiGLUBackwardArgs {
    const uint8_t* h;          // bf16 [rows, 2 * inter]: [gate | up] pre-activation kept by the forward pass
    const uint8_t* dact;       // bf16 [rows, inter]: gradient of silu(gate) * up * row_scale
    const float* row_scale;    // fp32 [rows] or nullptr
    uint8_t* dh;               // bf16 [rows, 2 * inter]
    int64_t rows;
    int inter;
};

// dgate = dact * scale * up * silu'(gate), dup = dact * scale * silu(gate); 8 columns per thread.
__global__ void __launch_bounds__(256) swiglu_backward_kernel(const __grid_constant__ SwiGLUBackwardArgs a) {
    const int64_t vec_per_row = a.inter / 8;
    const int64_t total = a.rows * vec_per_row;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t row = i / vec_per_row, col = (i % vec_per_row) * 8;
        const float scale = a.row_scale != nullptr ? a.row_scale[row] : 1.0f;
        const int4 g4 = ptx::ld_nc_v4(a.h + (row * 2 * a.inter + col) * 2);
        const int4 u4 = ptx::ld_nc_v4(a.h + (row * 2 * a.inter + a.inter + col) * 2);
        const int4 d4 = ptx::ld_nc_v4(a.dact + (row * a.inter + col) * 2);
        int4 og, ou;
        const uint32_t *gw = reinterpret_cast<const uint32_t*>(&g4), *uw = reinterpret_cast<const uint32_t*>(&u4),
                       *dw = reinterpret_cast<const uint32_t*>(&d4);
        uint32_t *ogw = reinterpret_cast<uint32_t*>(&og), *ouw = reinterpret_cast<uint32_t*>(&ou);
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = ptx::bf16x2_to_float2(gw[j]), u = ptx::bf16x2_to_float2(uw[j]), d = ptx::bf16x2_to_float2(dw[j]);
            float dg[2], du[2];
            const float gs[2] = {g.x, g.y}, us[2] = {u.x, u.y}, ds[2] = {d.x * scale, d.y * scale};
            #pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float sig = 1.0f / (1.0f + __expf(-gs[e]));
                du[e] = ds[e] * gs[e] * sig;
                dg[e] = ds[e] * us[e] * sig * (1.0f + gs[e] * (1.0f - sig));
            }
            ogw[j] = ptx::float2_to_bf16x2(dg[0], dg[1]), ouw[j] = ptx::float2_to_bf16x2(du[0], du[1]);
        }
        ptx::st_na_v4(a.dh + (row * 2 * a.inter + col) * 2, og);
        ptx::st_na_v4(a.dh + (row * 2 * a.inter + a.inter + col) * 2, ou);
    }
}

}  // namespace deep_ep::kernels
