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

// ---- FP8 training path: row-wise e4m3 quantisation with power-of-two scales (UE8M0 bytes, one per 128 columns), the
// operand format of the hardware-scaled grouped GEMM. Same arithmetic as the quantiser fused into the dispatch kernel.

namespace quant_detail {

// Quantises the 8 values of this lane; the 16 lanes that share a 128-column group agree on the scale.
// All 32 lanes must call it (shuffles inside). Returns the packed e4m3 bytes and the group's UE8M0 byte.
EP_DEVICE uint2 quantize8_ue8m0(const float (&v)[8], uint32_t& byte) {
    float amax = 0.f;
    #pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    #pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, 1e-4f);
    float inv;
    ptx::ue8m0_ceil(__fmul_rn(amax, 1.0f / 448.0f), byte, inv);
    uint2 packed;
    packed.x = ptx::float2_to_e4m3x2(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv)) |
               (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[2], inv), __fmul_rn(v[3], inv))) << 16);
    packed.y = ptx::float2_to_e4m3x2(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv)) |
               (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[6], inv), __fmul_rn(v[7], inv))) << 16);
    return packed;
}

EP_DEVICE void unpack8(const int4& raw, float (&v)[8]) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = ptx::bf16x2_to_float2(w[i]);
        v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
}

}  // namespace quant_detail

struct RowQuantArgs {
    const uint8_t* x;          // bf16 [rows, cols]
    uint8_t* q;                // e4m3 [rows, cols]
    uint8_t* sf;               // UE8M0 bytes [rows, cols / 128]
    int64_t rows;
    int cols;                  // multiple of 128
};

// One warp per row, four 16-byte vectors per lane in flight.
__global__ void __launch_bounds__(256) row_quant_ue8m0_kernel(const __grid_constant__ RowQuantArgs a) {
    using namespace quant_detail;
    constexpr int kInFlight = 4;
    const int lane = ptx::lane_id(), warps_per_cta = blockDim.x / 32;
    const int vecs = a.cols / 8, groups = a.cols / 128;
    for (int64_t row = int64_t(blockIdx.x) * warps_per_cta + threadIdx.x / 32; row < a.rows; row += int64_t(gridDim.x) * warps_per_cta) {
        const uint8_t* src = a.x + row * a.cols * 2;
        for (int base = 0; base < vecs; base += 32 * kInFlight) {       // warp-uniform trip count: shuffles inside
            int4 raw[kInFlight];
            #pragma unroll
            for (int i = 0; i < kInFlight; ++i) {
                const int vec = base + 32 * i + lane;
                raw[i] = vec < vecs ? ptx::ld_nc_v4(src + int64_t(vec) * 16) : make_int4(0, 0, 0, 0);
            }
            #pragma unroll
            for (int i = 0; i < kInFlight; ++i) {
                const int vec = base + 32 * i + lane;
                float v[8];
                unpack8(raw[i], v);
                uint32_t byte;
                const uint2 packed = quantize8_ue8m0(v, byte);
                if (vec < vecs) {
                    *reinterpret_cast<uint2*>(a.q + row * a.cols + int64_t(vec) * 8) = packed;
                    if ((lane & 15) == 0) a.sf[row * groups + vec / 16] = static_cast<uint8_t>(byte);
                }
            }
        }
    }
}

struct SwiGLUQuantArgs {
    const uint8_t* h;          // bf16 [rows, 2 * inter]: [gate | up]
    const float* row_scale;    // fp32 [rows] or nullptr
    uint8_t* act;              // bf16 [rows, inter] or nullptr: silu(gate) * up * row_scale, rounded once
    uint8_t* q;                // e4m3 [rows, inter]: the same values quantised from fp32
    uint8_t* sf;               // UE8M0 bytes [rows, inter / 128]
    int64_t rows;
    int inter;                 // multiple of 128
};

// One warp per row, two vector pairs (gate, up) per lane in flight.
__global__ void __launch_bounds__(256) swiglu_quant_ue8m0_kernel(const __grid_constant__ SwiGLUQuantArgs a) {
    using namespace quant_detail;
    constexpr int kInFlight = 2;
    const int lane = ptx::lane_id(), warps_per_cta = blockDim.x / 32;
    const int vecs = a.inter / 8, groups = a.inter / 128;
    for (int64_t row = int64_t(blockIdx.x) * warps_per_cta + threadIdx.x / 32; row < a.rows; row += int64_t(gridDim.x) * warps_per_cta) {
        const uint8_t* gate = a.h + row * a.inter * 4;
        const uint8_t* up = gate + int64_t(a.inter) * 2;
        const float scale = a.row_scale != nullptr ? a.row_scale[row] : 1.0f;
        for (int base = 0; base < vecs; base += 32 * kInFlight) {       // warp-uniform trip count: shuffles inside
            int4 g4[kInFlight], u4[kInFlight];
            #pragma unroll
            for (int i = 0; i < kInFlight; ++i) {
                const int vec = base + 32 * i + lane;
                g4[i] = vec < vecs ? ptx::ld_nc_v4(gate + int64_t(vec) * 16) : make_int4(0, 0, 0, 0);
                u4[i] = vec < vecs ? ptx::ld_nc_v4(up + int64_t(vec) * 16) : make_int4(0, 0, 0, 0);
            }
            #pragma unroll
            for (int i = 0; i < kInFlight; ++i) {
                const int vec = base + 32 * i + lane;
                float g[8], u[8], v[8];
                unpack8(g4[i], g);
                unpack8(u4[i], u);
                #pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = g[e] / (1.0f + __expf(-g[e])) * u[e] * scale;
                uint32_t byte;
                const uint2 packed = quantize8_ue8m0(v, byte);
                if (vec < vecs) {
                    *reinterpret_cast<uint2*>(a.q + row * a.inter + int64_t(vec) * 8) = packed;
                    if ((lane & 15) == 0) a.sf[row * groups + vec / 16] = static_cast<uint8_t>(byte);
                    if (a.act != nullptr) {
                        int4 out;
                        uint32_t* w = reinterpret_cast<uint32_t*>(&out);
                        #pragma unroll
                        for (int e = 0; e < 4; ++e) w[e] = ptx::float2_to_bf16x2(v[2 * e], v[2 * e + 1]);
                        ptx::st_na_v4(a.act + (row * a.inter + int64_t(vec) * 8) * 2, out);
                    }
                }
            }
        }
    }
}

struct BlockQuantArgs {
    const uint8_t* w;          // bf16 [rows, cols]: `rows / n` matrices of n rows each, stacked
    uint8_t* q;                // e4m3 [rows, cols]
    uint8_t* sf;               // UE8M0 bytes [rows / 128, cols / 128]
    uint8_t* qt;               // e4m3 [rows / n, cols, n]: every matrix transposed, or nullptr
    uint8_t* sft;              // UE8M0 bytes [rows / n, cols / 128, n / 128] (with `qt`)
    int64_t rows;
    int cols, n;               // multiples of 128
};

// Weights: one power-of-two scale per 128 x 128 block; the transposed copy (operand of the data-gradient GEMM) comes from
// the same pass. One CTA of 256 threads per block, grid = (cols / 128, rows / 128).
__global__ void __launch_bounds__(256) block_quant_ue8m0_kernel(const __grid_constant__ BlockQuantArgs a) {
    using namespace quant_detail;
    constexpr int kStride = 132;                           // bytes per tile row: 4-byte aligned, off the 128-byte bank period
    __shared__ float warp_max[8];
    __shared__ __align__(16) uint8_t tile[128 * kStride];
    const int tid = threadIdx.x, lane = ptx::lane_id(), warp = tid / 32;
    const int64_t row0 = int64_t(blockIdx.y) * 128;
    const int col0 = blockIdx.x * 128;
    const int vc = tid % 16, r_base = tid / 16;            // this thread: vector `vc` of rows r_base + 16 * i

    int4 raw[8];
    #pragma unroll
    for (int i = 0; i < 8; ++i)
        raw[i] = ptx::ld_nc_v4(a.w + ((row0 + r_base + 16 * i) * a.cols + col0 + vc * 8) * 2);
    float amax = 0.f;
    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        float v[8];
        unpack8(raw[i], v);
        #pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    }
    #pragma unroll
    for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) warp_max[warp] = amax;
    __syncthreads();
    #pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, warp_max[i]);
    amax = fmaxf(amax, 1e-4f);
    uint32_t byte;
    float inv;
    ptx::ue8m0_ceil(__fmul_rn(amax, 1.0f / 448.0f), byte, inv);

    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        float v[8];
        unpack8(raw[i], v);
        uint2 packed;
        packed.x = ptx::float2_to_e4m3x2(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv)) |
                   (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[2], inv), __fmul_rn(v[3], inv))) << 16);
        packed.y = ptx::float2_to_e4m3x2(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv)) |
                   (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[6], inv), __fmul_rn(v[7], inv))) << 16);
        const int r = r_base + 16 * i;
        *reinterpret_cast<uint2*>(a.q + (row0 + r) * a.cols + col0 + vc * 8) = packed;
        if (a.qt != nullptr) {
            uint32_t* t = reinterpret_cast<uint32_t*>(tile + r * kStride + vc * 8);
            t[0] = packed.x, t[1] = packed.y;
        }
    }
    const int64_t matrix = row0 / a.n;
    const int row_in_matrix = static_cast<int>(row0 % a.n);
    if (tid == 0) {
        a.sf[(row0 / 128) * (a.cols / 128) + blockIdx.x] = static_cast<uint8_t>(byte);
        if (a.qt != nullptr)
            a.sft[(matrix * (a.cols / 128) + blockIdx.x) * (a.n / 128) + row_in_matrix / 128] = static_cast<uint8_t>(byte);
    }
    if (a.qt == nullptr) return;
    __syncthreads();
    // transposed tile: output row c holds tile[0 .. 127][c]; 8 vectors of 16 bytes per output row, 4 vectors per thread
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int idx = tid + 256 * j, c = idx / 8, seg = idx % 8;
        int4 out;
        uint8_t* b = reinterpret_cast<uint8_t*>(&out);
        #pragma unroll
        for (int e = 0; e < 16; ++e) b[e] = tile[(seg * 16 + e) * kStride + c];
        *reinterpret_cast<int4*>(a.qt + (matrix * a.cols + col0 + c) * a.n + row_in_matrix + seg * 16) = out;
    }
}

}  // namespace deep_ep::kernels
