// Grouped FP8 (e4m3) forward GEMM whose block scales are applied by the tensor core itself
// (`tcgen05.mma.kind::mxf8f6f4.block_scale`). Scales are UE8M0 bytes (powers of two, value 2^(byte - 127)):
//
//   D[rows_e, N] = (A[rows_e, K] * 2^(sf_a[rows_e, K / 128] - 127))  x  (B_e[N, K] * 2^(sf_b[e, N / 128, K / 128] - 127))^T
//
// Unlike the fp32-scale kernel (`grouped_gemm_fp8.cuh`) nothing has to be promoted in registers: a tile's accumulator
// stays in tensor memory over the whole K loop and the tensor core is the only consumer of the operand stream.
//
// The instruction takes one scale per row (A) / column (B) and K = 32 elements from tensor memory. A scale here covers
// 128 K elements, so the four MMAs of a K block use the same scale byte, and the four bytes of a 32-bit tensor-memory
// column hold the scales of four consecutive K blocks (a "scale group"): the scale id in the instruction descriptor is
// `kb % 4`. Per scale group one warp re-lays the scale bytes out in shared memory (rows r, r + 32, r + 64, r + 96 of a
// 128-row tile side by side in one 16-byte line, the arrangement `tcgen05.cp.32x128b.warpx4` copies into tensor
// memory), and the MMA thread copies them next to the accumulator: 4 columns for A, 8 for the 256 columns of B.
//
// 384 threads per CTA, registers re-split with `setmaxnreg` (72 / 216; with 40 the scale producer spilled):
//   warp 0      TMA producer of the operand tiles (128-byte swizzle, CTA-local loads)
//   warp 1      MMA issuer: `tcgen05.cp` of the scales, four block-scaled MMAs per K block, commits
//   warp 2      scale producer: global scale bytes -> shared-memory atoms
//   warp 3      idle
//   warps 4-11  epilogue: each thread takes its 128 accumulator values into registers in two rounds of 64, reducing the
//               first round to its results before the second arrives; tensor memory is handed back to the next tile
//               right after the second round's loads, before the re-quantisation and the stores
// K must be a multiple of 512 (whole scale groups), N a multiple of 256.
// The reference contains no matrix math; this kernel exists for the fused MoE layer the library is benchmarked in.
#pragma once

#include "grouped_gemm_fp8.cuh"

namespace deep_ep::kernels {

__global__ void __launch_bounds__(kFp8ThreadsRegSplit, 1)
grouped_gemm_fp8_hw_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const __grid_constant__ GroupedGemmFp8Args a) {
    using namespace gemm_detail;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kGemmMaxStages], empty_bar[kGemmMaxStages], sf_full_bar[kFp8SfStages], sf_empty_bar[kFp8SfStages];
    __shared__ uint64_t tmem_full_bar, tmem_empty_bar, amax_bar[4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int tile_prefix[kMaxLocalExperts + 1];
    __shared__ float amax_sm[2][2][kGemmBlockM];       // [tile parity][column half][row]
    __shared__ __align__(128) uint8_t sf_smem[kFp8SfStages][kFp8SfStageBytes];
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
    const int num_sf_groups = num_k_blocks / kFp8SfGroup;
    constexpr uint32_t kSfColumns = 16;               // tensor-memory columns per scale buffer: 4 for A, 8 for B, 4 unused

    // ---- setup: barriers, tile schedule, tensor memory (256 accumulator columns + two scale buffers -> 512 allocated)
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) ptx::mbarrier_init(&full_bar[s], 1), ptx::mbarrier_init(&empty_bar[s], 1);
        for (int s = 0; s < kFp8SfStages; ++s) ptx::mbarrier_init(&sf_full_bar[s], 1), ptx::mbarrier_init(&sf_empty_bar[s], 1);
        ptx::mbarrier_init(&tmem_full_bar, 1), ptx::mbarrier_init(&tmem_empty_bar, 8);
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

    if (warp < 4) {
    // The CTA's register pool is 384 threads x 168 registers = 64512 = 128 x 72 + 256 x 216.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
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
            const uint64_t desc_a0 = tc::make_smem_desc(smem_a, 16, 1024), desc_b0 = tc::make_smem_desc(smem_b, 16, 1024);
            constexpr uint32_t a_stage_step = a_bytes >> 4, b_stage_step = b_bytes >> 4;
            int s = 0, fs = 0, local_tile = 0;
            uint32_t phase = 0, sf_phase = 0, group_count = 0;
            for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x, ++local_tile) {
                // the epilogue of the previous tile has taken the accumulator into registers
                if (not ptx::mbarrier_wait(&tmem_empty_bar, (local_tile & 1) ^ 1)) { error_flag = 1; break; }
                tc::fence_after_thread_sync();
                for (int kb = 0; kb < num_k_blocks; ++kb, s = (s + 1 == S ? 0 : s + 1), phase ^= (s == 0)) {
                    const int in_group = kb % kFp8SfGroup;
                    const uint32_t sf_tmem = tmem_base + kFp8BlockN + (group_count & 1) * kSfColumns;
                    if (in_group == 0) {
                        if (not ptx::mbarrier_wait(&sf_full_bar[fs], sf_phase)) { error_flag = 1; break; }
                    }
                    if (not ptx::mbarrier_wait(&full_bar[s], phase)) { error_flag = 1; break; }
                    tc::fence_after_thread_sync();
                    if (in_group == 0) {
                        // scales of this group: A atom -> 4 columns, the two B atoms -> 8 columns. Earlier MMAs that read
                        // the same tensor-memory columns (two groups ago) were issued by this thread before and complete first.
                        const uint8_t* atoms = sf_smem[fs];
                        tc::tmem_cp_32x128b_warpx4(sf_tmem, tc::make_smem_desc_noswizzle(atoms, 128));
                        tc::tmem_cp_32x128b_warpx4(sf_tmem + 4, tc::make_smem_desc_noswizzle(atoms + 512, 128));
                        tc::tmem_cp_32x128b_warpx4(sf_tmem + 8, tc::make_smem_desc_noswizzle(atoms + 1024, 128));
                    }
                    const uint32_t idesc = tc::make_idesc_block_scaled(tc::kFormatE4M3, kGemmBlockM, kFp8BlockN, in_group, in_group);
                    const uint64_t da = desc_a0 + uint64_t(s * a_stage_step), db = desc_b0 + uint64_t(s * b_stage_step);
                    #pragma unroll
                    for (int k = 0; k < kFp8BlockK / 32; ++k)
                        tc::mma_mxf8_block_scaled(tmem_base, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, sf_tmem, sf_tmem + 4,
                                                  kb > 0 or k > 0);
                    tc::commit(&empty_bar[s]);              // operand stage is free once these MMAs have read it
                    if (in_group == kFp8SfGroup - 1) {
                        tc::commit(&sf_empty_bar[fs]);      // so is the scale stage (its copy completed before the MMAs)
                        fs = (fs + 1 == kFp8SfStages ? 0 : fs + 1), sf_phase ^= (fs == 0), ++group_count;
                    }
                }
                tc::commit(&tmem_full_bar);                 // accumulator of this tile is complete
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ scale producer
        int fs = 0;
        uint32_t sf_phase = 0;
        const int sf_row_words = num_k_blocks / 4;          // 32-bit words per row of scale bytes
        for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x) {
            const Fp8Tile t = locate_fp8_tile(a, tile_prefix, tile, block_n_out);
            const int nb0 = t.n0 / 128, nb1 = swiglu ? (a.n / 2 + t.n0) / 128 : nb0 + 1;
            const uint32_t* sfb0 = reinterpret_cast<const uint32_t*>(a.sf_b_e8) + (size_t(t.expert) * (a.n / 128) + nb0) * sf_row_words;
            const uint32_t* sfb1 = reinterpret_cast<const uint32_t*>(a.sf_b_e8) + (size_t(t.expert) * (a.n / 128) + nb1) * sf_row_words;
            // scales of A: UE8M0 bytes, or fp32 powers of two (what the dispatch kernel's power-of-two quantiser delivers),
            // of which only the exponent byte is kept
            const bool a_bytes_given = a.sf_a_e8 != nullptr;
            size_t sfa_row[4];
            #pragma unroll
            for (int j = 0; j < 4; ++j) sfa_row[j] = size_t(min(t.row_base + t.m0 + lane + 32 * j, a.total_rows - 1));
            for (int g = 0; g < num_sf_groups; ++g, fs = (fs + 1 == kFp8SfStages ? 0 : fs + 1), sf_phase ^= (fs == 0)) {
                uint32_t wa_[4];
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (a_bytes_given) {
                        wa_[j] = __ldg(reinterpret_cast<const uint32_t*>(a.sf_a_e8) + sfa_row[j] * sf_row_words + g);
                    } else {
                        const uint4 f = __ldg(reinterpret_cast<const uint4*>(a.sf_a + sfa_row[j] * num_k_blocks) + g);
                        wa_[j] = ((f.x >> 23) & 0xffu) | (((f.y >> 23) & 0xffu) << 8) | (((f.z >> 23) & 0xffu) << 16) | (((f.w >> 23) & 0xffu) << 24);
                    }
                }
                const uint4 wa = make_uint4(wa_[0], wa_[1], wa_[2], wa_[3]);
                const uint32_t w0 = __ldg(sfb0 + g), w1 = __ldg(sfb1 + g);
                bool ok = true;
                if (lane == 0) ok = ptx::mbarrier_wait(&sf_empty_bar[fs], sf_phase ^ 1);
                if (not __shfl_sync(0xffffffffu, int(ok), 0)) { error_flag = 1; break; }
                uint4* atoms = reinterpret_cast<uint4*>(sf_smem[fs]);
                atoms[lane] = wa;                                   // rows lane, lane + 32, lane + 64, lane + 96
                atoms[32 + lane] = make_uint4(w0, w0, w0, w0);      // every column of a 128 x 128 weight block shares its scale
                atoms[64 + lane] = make_uint4(w1, w1, w1, w1);
                ptx::fence_proxy_async_smem();                      // visible to the tensor-memory copy engine
                __syncwarp();
                if (lane == 0) ptx::mbarrier_arrive(&sf_full_bar[fs]);
            }
        }
    }
    } else {
        // ------------------------------------------------------------------ epilogue (eight warps)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int quarter = warp & 3;                    // tensor-memory lane quarter this warp may access
        const int half = (warp - 4) >> 2;                // which two 64-column segments
        const int row = quarter * 32 + lane;
        const int col_a = swiglu ? half * 64 : half * 128;
        const int col_b = swiglu ? 128 + half * 64 : half * 128 + 64;
        int local_tile = 0;
        bool stored_remotely = false;
        for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x, ++local_tile) {
            const Fp8Tile t = locate_fp8_tile(a, tile_prefix, tile, block_n_out);
            const int grow = t.row_base + t.m0 + row;
            if (not ptx::mbarrier_wait(&tmem_full_bar, local_tile & 1)) { error_flag = 1; break; }
            tc::fence_after_thread_sync();
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
            // The warp's 128 accumulator columns are taken out of tensor memory in two rounds of 64 (two 32-column loads
            // each): the values of the first round are already reduced to their results (32 SwiGLU outputs, or stored) when
            // the second round arrives, so at most about a hundred registers are live instead of two hundred. Tensor
            // memory is handed back to the MMA warp right after the second round's loads.
            const bool valid = row < t.rows_valid, written = row < t.rows_written;
            uint32_t acc[64];
            auto load_round = [&](int round) {
                // SwiGLU: 32 gate + 32 up columns of output columns [32 * round, 32 * round + 32); plain: 64 columns
                uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&acc[0]);
                uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&acc[32]);
                if (swiglu) {
                    tc::tmem_ld_32x32(taddr + col_a + 32 * round, lo);
                    tc::tmem_ld_32x32(taddr + col_b + 32 * round, hi);
                } else {
                    tc::tmem_ld_32x32(taddr + (round == 0 ? col_a : col_b), lo);
                    tc::tmem_ld_32x32(taddr + (round == 0 ? col_a : col_b) + 32, hi);
                }
                tc::wait_ld();
                if (round == 1) {
                    // everything is in registers: the next tile may overwrite tensor memory
                    tc::fence_before_thread_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbarrier_arrive(&tmem_empty_bar);
                }
            };
            if (not swiglu) {
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + size_t(grow) * a.n_out + t.n0 + half * 128;
                if (a.route != nullptr and valid) {
                    // a row that is its token's only contribution from this rank goes straight to the token's owner
                    const unsigned long long target = __ldg(a.route + grow);
                    if (target != 0) out = reinterpret_cast<__nv_bfloat16*>(target) + t.n0 + half * 128, stored_remotely = true;
                }
                #pragma unroll
                for (int round = 0; round < 2; ++round) {
                    load_round(round);
                    if (written) {
                        #pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            int4 packed;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                            #pragma unroll
                            for (int i = 0; i < 4; ++i)
                                w[i] = valid ? ptx::float2_to_bf16x2(__uint_as_float(acc[8 * v + 2 * i]), __uint_as_float(acc[8 * v + 2 * i + 1])) : 0u;
                            *reinterpret_cast<int4*>(out + 64 * round + 8 * v) = packed;
                        }
                    }
                }
            } else {
                // output columns n0 + half * 64 .. + 64 of this warp: h = silu(gate) * up * row scale
                const float scale = (valid and a.row_scale != nullptr) ? a.row_scale[grow] : 1.0f;
                float amax = 0.f;
                float h[64];
                #pragma unroll
                for (int round = 0; round < 2; ++round) {
                    load_round(round);
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float value = valid ? silu(__uint_as_float(acc[i])) * __uint_as_float(acc[32 + i]) * scale : 0.f;
                        h[32 * round + i] = value;
                        amax = fmaxf(amax, fabsf(value));
                    }
                }
                if (not a.out_fp8) {
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + size_t(grow) * a.n_out + t.n0 + half * 64;
                    if (written) {
                        #pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            int4 packed;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                            #pragma unroll
                            for (int i = 0; i < 4; ++i) w[i] = ptx::float2_to_bf16x2(h[8 * v + 2 * i], h[8 * v + 2 * i + 1]);
                            *reinterpret_cast<int4*>(out + 8 * v) = packed;
                        }
                    }
                } else {
                    // the 128 output columns of this tile are one scale block: merge the two halves' maxima, then
                    // quantise with the power-of-two scale 2^ceil(log2(amax / 448))
                    const int par = local_tile & 1;
                    amax_sm[par][half][row] = amax;
                    __syncwarp();
                    if (lane == 0) ptx::mbarrier_arrive(&amax_bar[quarter]);
                    if (not ptx::mbarrier_wait(&amax_bar[quarter], par)) { error_flag = 1; break; }
                    amax = fmaxf(fmaxf(amax, amax_sm[par][half ^ 1][row]), 1e-4f);
                    uint32_t sf_byte;
                    float inv;
                    ptx::ue8m0_ceil(__fmul_rn(amax, 1.0f / 448.0f), sf_byte, inv);
                    if (written) {
                        uint8_t* out = reinterpret_cast<uint8_t*>(a.d) + size_t(grow) * a.n_out + t.n0 + half * 64;
                        #pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            int4 packed;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                            #pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int j = 16 * v + 4 * i;
                                w[i] = ptx::float2_to_e4m3x2(h[j] * inv, h[j + 1] * inv) |
                                       (uint32_t(ptx::float2_to_e4m3x2(h[j + 2] * inv, h[j + 3] * inv)) << 16);
                            }
                            *reinterpret_cast<int4*>(out + 16 * v) = packed;
                        }
                        if (half == 0) a.d_sf_e8[size_t(grow) * (a.n_out / 128) + t.n0 / 128] = uint8_t(sf_byte);
                    }
                }
            }
        }
        if (stored_remotely) __threadfence_system();     // peer stores are performed before the kernel completes
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
