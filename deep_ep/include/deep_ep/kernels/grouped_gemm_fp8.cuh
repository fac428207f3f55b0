// Grouped FP8 (e4m3) GEMM with DeepSeek-style block scales for the expert FFNs, forward direction, on the
// sm_100a tensor cores.
//
//   D[rows_e, N] = (A[rows_e, K] * sf_a[rows_e, K / 128])  x  (B_e[N, K] * sf_b[e, N / 128, K / 128])^T
//
// A is what the FP8 dispatch delivers (e4m3 rows with one fp32 scale per 128 columns), B are expert weights
// quantised per 128 x 128 block. fp32 scales cannot be given to `tcgen05.mma`, so the kernel promotes in
// software: one K block (128 e4m3 = one 128-byte swizzle row = one scale block) is multiplied into a
// tensor-memory buffer by four `kind::f8f6f4` MMAs (K = 32 each), then eight warps read the buffer with
// `tcgen05.ld` and add `sf_a[row, kb] * sf_b[block, kb] * partial` into fp32 registers while the tensor core
// already works on the next K block in the second buffer.
//
// Roles (kRegSplit = true, 384 threads; the variant without the register split has 320 and no idle warps):
//   warp 0      TMA producer (tiled `cp.async.bulk.tensor`, 128-byte swizzle, CTA-local)
//   warp 1      MMA issuer (one thread)
//   warps 2-3   idle: they complete the first warpgroup, which hands most of its registers to the other two
//               (`setmaxnreg`), so that a promotion thread can hold 128 accumulators plus 64 values in flight
//   warps 4-11  promotion + epilogue; warp w owns tensor-memory lanes 32 * (w % 4) .. +32 (one row per thread) and
//               two 64-column segments of the 256-column tile
// Epilogues: bf16 store, or SwiGLU (gate and up columns paired in one tile) with bf16 output or with e4m3 output
// re-quantised per row and 128 columns, so that the second FFN GEMM consumes it without another pass.
// The reference contains no matrix math; this kernel exists for the fused MoE layer the library is benchmarked in.
#pragma once

#include "../device/sync.cuh"
#include "../device/tcgen05.cuh"
#include "grouped_gemm.cuh"

namespace deep_ep::kernels {

namespace gemm_detail {

// acc{0,1} += f * {a0, a1} as one packed fp32x2 instruction (sm_100 issues two fp32 FMAs per slot this way).
EP_DEVICE void fma2(float& acc0, float& acc1, uint32_t a0, uint32_t a1, float f) {
    asm("{\n .reg .b64 va, vf, vc;\n"
        " mov.b64 va, {%2, %3};\n mov.b64 vf, {%4, %4};\n mov.b64 vc, {%0, %1};\n"
        " fma.rn.f32x2 vc, va, vf, vc;\n"
        " mov.b64 {%0, %1}, vc;\n}\n"
        : "+f"(acc0), "+f"(acc1) : "r"(a0), "r"(a1), "f"(f));
}

struct Fp8Tile {
    int expert, m0, n0, row_base, rows_valid, rows_written;
};

EP_DEVICE Fp8Tile locate_fp8_tile(const GroupedGemmFp8Args& a, const int* prefix, int tile, int block_n_out) {
    int lo = 0, hi = a.num_groups - 1;
    while (lo < hi) {                       // last expert whose prefix <= tile
        const int mid = (lo + hi + 1) >> 1;
        if (prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const int e = lo, local = tile - prefix[e];
    const int count = a.count[e];
    const int m_tiles = math::ceil_div(count, kGemmBlockM);
    Fp8Tile t;
    t.expert = e, t.row_base = a.psum[e] - count;
    t.m0 = (local % m_tiles) * kGemmBlockM, t.n0 = (local / m_tiles) * block_n_out;
    t.rows_valid = min(kGemmBlockM, count - t.m0);
    t.rows_written = min(kGemmBlockM, math::align(count, max(a.alignment, 1)) - t.m0);
    return t;
}

}  // namespace gemm_detail

template <bool kRegSplit>
__global__ void __launch_bounds__(kRegSplit ? kFp8ThreadsRegSplit : kFp8Threads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ GroupedGemmFp8Args a) {
    using namespace gemm_detail;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kGemmMaxStages], empty_bar[kGemmMaxStages], tmem_full_bar[2], tmem_empty_bar[2], amax_bar[4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int tile_prefix[kMaxLocalExperts + 1];
    __shared__ float amax_sm[2][2][kGemmBlockM];       // [tile parity][column half][row]
    __shared__ volatile int error_flag;

    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    const int S = a.num_stages;
    constexpr uint32_t a_bytes = kGemmBlockM * kFp8BlockK, b_bytes = kFp8BlockN * kFp8BlockK;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + size_t(S) * a_bytes;
    const bool swiglu = a.epilogue != kEpilogueStore;
    const int block_n_out = swiglu ? kFp8BlockN / 2 : kFp8BlockN;
    const int num_k_blocks = a.k / kFp8BlockK;

    // ---- setup: barriers, tile schedule, tensor memory
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) ptx::mbarrier_init(&full_bar[s], 1), ptx::mbarrier_init(&empty_bar[s], 1);
        for (int i = 0; i < 2; ++i) ptx::mbarrier_init(&tmem_full_bar[i], 1), ptx::mbarrier_init(&tmem_empty_bar[i], 8);
        for (int i = 0; i < 4; ++i) ptx::mbarrier_init(&amax_bar[i], 2);
        ptx::fence_mbarrier_init();
        error_flag = 0;
        tc::prefetch_tensormap(&map_a), tc::prefetch_tensormap(&map_b);
    }
    if (warp == 1) tc::tmem_alloc(&tmem_base_slot, 512);
    if (warp == 2) {
        int carry = 0;
        for (int base = 0; base < a.num_groups; base += 32) {
            const int e = base + lane;
            const int tiles = e < a.num_groups ? math::ceil_div(a.count[e], kGemmBlockM) * (a.n_out / block_n_out) : 0;
            int incl = tiles;
            #pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (e < a.num_groups) tile_prefix[e] = carry + incl - tiles;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) tile_prefix[a.num_groups] = carry;
    }
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = tmem_base_slot;
    const int num_tiles = tile_prefix[a.num_groups];
    constexpr int kFirstEpilogueWarp = kRegSplit ? 4 : 2;

    if (warp < kFirstEpilogueWarp) {
    // The CTA's register pool is what the launch allocated: 384 threads x 168 registers = 64512. `setmaxnreg.inc` blocks
    // until the pool has room, so the split must fit it exactly or below: 128 x 40 + 256 x 232 = 64512.
    if constexpr (kRegSplit) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x) {
                const Fp8Tile t = locate_fp8_tile(a, tile_prefix, tile, block_n_out);
                const int b_row0 = t.expert * a.n + t.n0;
                const int b_row1 = swiglu ? t.expert * a.n + a.n / 2 + t.n0 : b_row0 + 128;
                for (int kb = 0; kb < num_k_blocks; ++kb, s = (s + 1 == S ? 0 : s + 1), phase ^= (s == 0)) {
                    if (not ptx::mbarrier_wait(&empty_bar[s], phase ^ 1)) { error_flag = 1; break; }
                    ptx::mbarrier_arrive_expect_tx(&full_bar[s], a_bytes + b_bytes);
                    uint8_t* sa = smem_a + size_t(s) * a_bytes;
                    uint8_t* sb = smem_b + size_t(s) * b_bytes;
                    const int k0 = kb * kFp8BlockK;
                    tc::tma_load_2d(sa, &map_a, k0, t.row_base + t.m0, &full_bar[s]);
                    tc::tma_load_2d(sb, &map_b, k0, b_row0, &full_bar[s]);
                    tc::tma_load_2d(sb + 128 * kFp8BlockK, &map_b, k0, b_row1, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = tc::make_idesc(tc::kFormatE4M3, kGemmBlockM, kFp8BlockN, false, false);
            const uint64_t desc_a0 = tc::make_smem_desc(smem_a, 16, 1024), desc_b0 = tc::make_smem_desc(smem_b, 16, 1024);
            constexpr uint32_t a_stage_step = a_bytes >> 4, b_stage_step = b_bytes >> 4;
            int s = 0;
            uint32_t phase = 0, it = 0;         // `it` counts K blocks over all tiles: buffer = it & 1
            for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x) {
                for (int kb = 0; kb < num_k_blocks; ++kb, ++it, s = (s + 1 == S ? 0 : s + 1), phase ^= (s == 0)) {
                    const uint32_t buf = it & 1, use = it >> 1;
                    if (not ptx::mbarrier_wait(&tmem_empty_bar[buf], (use & 1) ^ 1)) { error_flag = 1; break; }
                    if (not ptx::mbarrier_wait(&full_bar[s], phase)) { error_flag = 1; break; }
                    tc::fence_after_thread_sync();
                    const uint32_t tmem_d = tmem_base + buf * kFp8BlockN;
                    const uint64_t da = desc_a0 + uint64_t(s * a_stage_step), db = desc_b0 + uint64_t(s * b_stage_step);
                    #pragma unroll
                    for (int k = 0; k < kFp8BlockK / 32; ++k)       // 32 e4m3 = 32 bytes = 2 address units per MMA
                        tc::mma_f8(tmem_d, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, k > 0);
                    tc::commit(&empty_bar[s]);              // stage is free once these MMAs have read it
                    tc::commit(&tmem_full_bar[buf]);        // partial product of this K block is complete
                }
            }
        }
    }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue (eight warps)
        if constexpr (kRegSplit) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int quarter = warp & 3;                    // tensor-memory lane quarter this warp may access
        const int half = (warp - kFirstEpilogueWarp) >> 2;   // which two 64-column segments
        const int row = quarter * 32 + lane;
        // tensor-memory columns of the two segments: plain store -> 128 consecutive columns; SwiGLU -> 64 gate
        // columns and the 64 up columns that pair with them
        const int col_a = swiglu ? half * 64 : half * 128;
        const int col_b = swiglu ? 128 + half * 64 : half * 128 + 64;
        const int sfb_stride = num_k_blocks;
        uint32_t it = 0;
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x, ++local_tile) {
            const Fp8Tile t = locate_fp8_tile(a, tile_prefix, tile, block_n_out);
            const int grow = t.row_base + t.m0 + row;
            const float* sfa = a.sf_a + size_t(min(grow, a.total_rows - 1)) * num_k_blocks;
            const int nb_a = swiglu ? t.n0 / 128 : t.n0 / 128 + half;
            const int nb_b = swiglu ? (a.n / 2 + t.n0) / 128 : nb_a;
            const float* sfb_a = a.sf_b + (size_t(t.expert) * (a.n / 128) + nb_a) * sfb_stride;
            const float* sfb_b = a.sf_b + (size_t(t.expert) * (a.n / 128) + nb_b) * sfb_stride;

            float acc[128];
            #pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.f;
            float sa_next = __ldg(sfa), sba_next = __ldg(sfb_a), sbb_next = __ldg(sfb_b);
            bool ok = true;
            for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
                const uint32_t buf = it & 1, use = it >> 1;
                const float fa = sa_next * sba_next, fb = sa_next * sbb_next;
                if (kb + 1 < num_k_blocks)
                    sa_next = __ldg(sfa + kb + 1), sba_next = __ldg(sfb_a + kb + 1), sbb_next = __ldg(sfb_b + kb + 1);
                if (not ptx::mbarrier_wait(&tmem_full_bar[buf], use & 1)) { error_flag = 1; ok = false; break; }
                tc::fence_after_thread_sync();
                const uint32_t taddr = tmem_base + buf * kFp8BlockN + (uint32_t(quarter * 32) << 16);
                if constexpr (kRegSplit) {
                    // two round trips to tensor memory per K block, 64 columns each
                    #pragma unroll
                    for (int seg = 0; seg < 2; ++seg) {
                        uint32_t r0[32], r1[32];
                        const int col = seg == 0 ? col_a : col_b;
                        tc::tmem_ld_32x32(taddr + col, r0);
                        tc::tmem_ld_32x32(taddr + col + 32, r1);
                        tc::wait_ld();
                        if (seg == 1) {
                            // every value of this buffer is in registers: hand it back before the last multiply-adds
                            tc::fence_before_thread_sync();
                            __syncwarp();
                            if (lane == 0) ptx::mbarrier_arrive(&tmem_empty_bar[buf]);
                        }
                        const float f = seg == 0 ? fa : fb;
                        #pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            fma2(acc[64 * seg + i], acc[64 * seg + i + 1], r0[i], r0[i + 1], f);
                            fma2(acc[64 * seg + 32 + i], acc[64 * seg + 32 + i + 1], r1[i], r1[i + 1], f);
                        }
                    }
                } else {
                    #pragma unroll
                    for (int seg = 0; seg < 4; ++seg) {
                        uint32_t r[32];
                        tc::tmem_ld_32x32(taddr + (seg < 2 ? col_a + 32 * seg : col_b + 32 * (seg - 2)), r);
                        tc::wait_ld();
                        if (seg == 3) {
                            tc::fence_before_thread_sync();
                            __syncwarp();
                            if (lane == 0) ptx::mbarrier_arrive(&tmem_empty_bar[buf]);
                        }
                        const float f = seg < 2 ? fa : fb;
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) acc[32 * seg + i] = fmaf(f, __uint_as_float(r[i]), acc[32 * seg + i]);
                    }
                }
            }
            if (not ok) break;

            const bool valid = row < t.rows_valid, written = row < t.rows_written;
            if (not swiglu) {
                // acc[0..128) = 128 consecutive output columns
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + size_t(grow) * a.n_out + t.n0 + half * 128;
                if (written) {
                    #pragma unroll
                    for (int v = 0; v < 16; ++v) {
                        int4 packed;
                        uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) w[i] = valid ? ptx::float2_to_bf16x2(acc[8 * v + 2 * i], acc[8 * v + 2 * i + 1]) : 0u;
                        *reinterpret_cast<int4*>(out + 8 * v) = packed;
                    }
                }
            } else {
                // acc[0..64) = gate, acc[64..128) = up of output columns n0 + half * 64 ..
                const float scale = (valid and a.row_scale != nullptr) ? a.row_scale[grow] : 1.0f;
                float amax = 0.f;
                #pragma unroll
                for (int i = 0; i < 64; ++i) {
                    acc[i] = valid ? silu(acc[i]) * acc[64 + i] * scale : 0.f;
                    amax = fmaxf(amax, fabsf(acc[i]));
                }
                if (not a.out_fp8) {
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + size_t(grow) * a.n_out + t.n0 + half * 64;
                    if (written) {
                        #pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            int4 packed;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                            #pragma unroll
                            for (int i = 0; i < 4; ++i) w[i] = ptx::float2_to_bf16x2(acc[8 * v + 2 * i], acc[8 * v + 2 * i + 1]);
                            *reinterpret_cast<int4*>(out + 8 * v) = packed;
                        }
                    }
                } else {
                    // the 128 output columns of this tile are one scale block: merge the two halves' maxima
                    const int par = local_tile & 1;
                    amax_sm[par][half][row] = amax;
                    __syncwarp();
                    if (lane == 0) ptx::mbarrier_arrive(&amax_bar[quarter]);
                    if (not ptx::mbarrier_wait(&amax_bar[quarter], par)) { error_flag = 1; break; }
                    amax = fmaxf(fmaxf(amax, amax_sm[par][half ^ 1][row]), 1e-4f);
                    const float inv = __fmul_rn(__frcp_rn(amax), 448.0f);
                    if (written) {
                        uint8_t* out = reinterpret_cast<uint8_t*>(a.d) + size_t(grow) * a.n_out + t.n0 + half * 64;
                        #pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            int4 packed;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                            #pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int j = 16 * v + 4 * i;
                                w[i] = ptx::float2_to_e4m3x2(__fmul_rn(acc[j], inv), __fmul_rn(acc[j + 1], inv)) |
                                       (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(acc[j + 2], inv), __fmul_rn(acc[j + 3], inv))) << 16);
                            }
                            *reinterpret_cast<int4*>(out + 16 * v) = packed;
                        }
                        if (half == 0) a.d_sf[size_t(grow) * (a.n_out / 128) + t.n0 / 128] = __fmul_rn(amax, 1.0f / 448.0f);
                    }
                }
            }
        }
    }

    // ---- teardown: every thread arrives here, then the allocating warp frees tensor memory
    tc::fence_before_thread_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem_base, 512);
    }
    // a bounded wait ran out: leave a mark where the host finds it (mapped host memory) before its next launch
    if (threadIdx.x == 0 and error_flag and a.status != nullptr) {
        *reinterpret_cast<volatile int*>(a.status) = 1;
        __threadfence_system();
    }
}

}  // namespace deep_ep::kernels
