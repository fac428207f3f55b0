// Grouped BF16 GEMM on CTA pairs (`tcgen05.mma.cta_group::2`): the same three problem shapes as
// `grouped_gemm.cuh`, with a 256 x 256 output tile owned by two CTAs of a cluster. Each CTA stages 128 rows of A and
// 128 columns of B per K block (32 KB instead of 48 KB), the even CTA issues one M = 256 MMA per K = 16 for both,
// and each CTA's tensor memory holds its 128 rows of the accumulator. Halving the B traffic per SM lifts the
// shared-memory bound of the single-CTA kernel (about two thirds of the tensor peak).
//
// Synchronisation inside a pair:
//   full[s]        (even CTA)  one arrival from the even producer + the TMA bytes of BOTH CTAs
//   empty[s]       (each CTA)  committed by the even CTA's MMA thread to both CTAs when the stage has been read
//   tmem_full[a]   (each CTA)  committed by the MMA thread to both CTAs when an accumulator is complete
//   tmem_empty[a]  (even CTA)  eight arrivals: the four epilogue warps of each CTA
// No load is multicast: every CTA fetches its own operand halves.
#pragma once

#include "../device/sync.cuh"
#include "../device/tcgen05.cuh"
#include "grouped_gemm.cuh"

namespace deep_ep::kernels {

namespace gemm2_detail {

constexpr int kPairM = 256, kPairN = 256;

struct Tile {
    int expert, m0, n0, row_base, count, aligned_count, num_k_blocks;
};

EP_DEVICE Tile locate_tile(const GroupedGemmArgs& a, const int* prefix, int tile) {
    int lo = 0, hi = a.num_groups - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const int e = lo, local = tile - prefix[e];
    const int count = a.count[e];
    Tile t;
    t.expert = e, t.row_base = a.psum[e] - count, t.count = count;
    t.aligned_count = math::align(count, max(a.alignment, 1));
    if (a.mode == kModeWgrad) {
        const int m_tiles = a.m / kPairM;
        t.m0 = (local % m_tiles) * kPairM, t.n0 = (local / m_tiles) * kPairN;
        t.num_k_blocks = math::ceil_div(count, kGemmBlockK);
    } else {
        const int m_tiles = math::ceil_div(count, kPairM);
        t.m0 = (local % m_tiles) * kPairM, t.n0 = (local / m_tiles) * a.block_n_out;
        t.num_k_blocks = math::ceil_div(a.k, kGemmBlockK);
    }
    return t;
}

}  // namespace gemm2_detail

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_d, const __grid_constant__ GroupedGemmArgs a) {
    using namespace gemm2_detail;
    using gemm_detail::silu;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kGemmMaxStages], empty_bar[kGemmMaxStages], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int tile_prefix[kMaxLocalExperts + 1];
    __shared__ volatile int error_flag;

    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    const uint32_t cta_rank = tc::cluster_ctarank();            // 0 = even CTA (issues the MMAs), 1 = odd CTA
    const bool leader = cta_rank == 0;
    const int pair = blockIdx.x / 2, num_pairs = gridDim.x / 2;
    const int S = a.num_stages;
    constexpr uint32_t kHalfBytes = 128 * kGemmBlockK * 2;      // 128 rows (or columns) x 64 bf16 = 16 KB
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + size_t(S) * kHalfBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) ptx::mbarrier_init(&full_bar[s], 1), ptx::mbarrier_init(&empty_bar[s], 1);
        for (int i = 0; i < 2; ++i) ptx::mbarrier_init(&tmem_full_bar[i], 1), ptx::mbarrier_init(&tmem_empty_bar[i], 8);
        ptx::fence_mbarrier_init();
        error_flag = 0;
        tc::prefetch_tensormap(&map_a), tc::prefetch_tensormap(&map_b);
    }
    if (warp == 2) {
        int carry = 0;
        for (int base = 0; base < a.num_groups; base += 32) {
            const int e = base + lane;
            int tiles = 0;
            if (e < a.num_groups) {
                const int count = a.count[e];
                if (a.mode == kModeWgrad) tiles = (count > 0 or not a.accumulate) ? (a.m / kPairM) * (a.n / kPairN) : 0;
                else tiles = math::ceil_div(count, kPairM) * (a.n_out / a.block_n_out);
            }
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
    __syncthreads();
    tc::cluster_sync();                      // both CTAs' barriers exist before anyone signals across the pair
    if (warp == 1) tc::tmem_alloc_pair(&tmem_base_slot, 512);
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = tmem_base_slot;
    const int num_tiles = tile_prefix[a.num_groups];

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            for (int tile = pair; tile < num_tiles and not error_flag; tile += num_pairs) {
                const Tile t = locate_tile(a, tile_prefix, tile);
                for (int kb = 0; kb < t.num_k_blocks; ++kb, s = (s + 1 == S ? 0 : s + 1), phase ^= (s == 0)) {
                    if (not ptx::mbarrier_wait(&empty_bar[s], phase ^ 1)) { error_flag = 1; break; }
                    // the bytes of both CTAs are counted on the even CTA's barrier
                    const uint32_t bar = tc::map_to_cta(&full_bar[s], 0);
                    if (leader) ptx::mbarrier_arrive_expect_tx(&full_bar[s], 4 * kHalfBytes);
                    uint8_t* sa = smem_a + size_t(s) * kHalfBytes;
                    uint8_t* sb = smem_b + size_t(s) * kHalfBytes;
                    const int k0 = kb * kGemmBlockK;
                    const int m_half = t.m0 + 128 * int(cta_rank);
                    if (a.mode == kModeWgrad) {
                        const int n_half = t.n0 + 128 * int(cta_rank);
                        for (int i = 0; i < 2; ++i) {
                            tc::tma_load_2d_pair(sa + i * 8192, &map_a, m_half + 64 * i, t.row_base + k0, bar);
                            tc::tma_load_2d_pair(sb + i * 8192, &map_b, n_half + 64 * i, t.row_base + k0, bar);
                        }
                    } else {
                        tc::tma_load_2d_pair(sa, &map_a, k0, t.row_base + m_half, bar);
                        if (a.mode == kModeForward) {
                            // accumulator columns [0,128) come from the even CTA's B half, [128,256) from the odd CTA's;
                            // with SwiGLU those are 128 gate rows and the matching 128 up rows of the weight
                            const int row = t.expert * a.n + (a.epilogue != kEpilogueStore
                                                                  ? t.n0 + int(cta_rank) * (a.n / 2)
                                                                  : t.n0 + 128 * int(cta_rank));
                            tc::tma_load_2d_pair(sb, &map_b, k0, row, bar);
                        } else {
                            const int n_half = t.n0 + 128 * int(cta_rank);
                            for (int i = 0; i < 2; ++i)
                                tc::tma_load_2d_pair(sb + i * 8192, &map_b, n_half + 64 * i, t.expert * a.k + k0, bar);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (even CTA only)
        if (leader and lane == 0) {
            const bool a_mn = a.mode == kModeWgrad, b_mn = a.mode != kModeForward;
            const uint32_t idesc = tc::make_idesc(tc::kFormatBF16, kPairM, kPairN, a_mn, b_mn);
            const uint32_t a_lead = a_mn ? 8192 : 16, b_lead = b_mn ? 8192 : 16;
            const uint32_t a_kstep = a_mn ? 2048 : 32, b_kstep = b_mn ? 2048 : 32;
            const uint64_t desc_a0 = tc::make_smem_desc(smem_a, a_lead, 1024), desc_b0 = tc::make_smem_desc(smem_b, b_lead, 1024);
            const uint32_t stage_step = kHalfBytes >> 4, a_k = a_kstep >> 4, b_k = b_kstep >> 4;
            int s = 0, local_tile = 0;
            uint32_t phase = 0;
            for (int tile = pair; tile < num_tiles and not error_flag; tile += num_pairs, ++local_tile) {
                const Tile t = locate_tile(a, tile_prefix, tile);
                const int acc = local_tile & 1, use = local_tile >> 1;
                if (not ptx::mbarrier_wait(&tmem_empty_bar[acc], (use & 1) ^ 1)) { error_flag = 1; break; }
                tc::fence_after_thread_sync();
                const uint32_t tmem_d = tmem_base + acc * 256;
                for (int kb = 0; kb < t.num_k_blocks; ++kb, s = (s + 1 == S ? 0 : s + 1), phase ^= (s == 0)) {
                    if (not ptx::mbarrier_wait(&full_bar[s], phase)) { error_flag = 1; break; }
                    tc::fence_after_thread_sync();
                    const uint64_t da = desc_a0 + uint64_t(s * stage_step), db = desc_b0 + uint64_t(s * stage_step);
                    #pragma unroll
                    for (int k = 0; k < kGemmBlockK / 16; ++k)
                        tc::mma_f16_pair(tmem_d, da + uint64_t(k * a_k), db + uint64_t(k * b_k), idesc, kb > 0 or k > 0);
                    tc::commit_pair(&empty_bar[s]);      // the stage is free in both CTAs once these MMAs have read it
                }
                if (t.num_k_blocks > 0) {
                    tc::commit_pair(&tmem_full_bar[acc]);
                } else {
                    tc::mbarrier_arrive_cluster(tc::map_to_cta(&tmem_full_bar[acc], 0));
                    tc::mbarrier_arrive_cluster(tc::map_to_cta(&tmem_full_bar[acc], 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                       // row inside this CTA's 128-row half
        int local_tile = 0;
        bool stored_remotely = false;
        // fp32 weight gradients: two staging buffers per warp behind the operand ring (see gemm_detail::WgradStaging)
        gemm_detail::WgradStaging staging;
        staging.num_buffers = max(a.staging_buffers, 1);
        staging.buffers = smem_b + size_t(S) * kHalfBytes + size_t(quarter) * staging.num_buffers * gemm_detail::WgradStaging::kChunkBytes;
        const bool use_tma = a.staging_buffers > 0;
        for (int tile = pair; tile < num_tiles and not error_flag; tile += num_pairs, ++local_tile) {
            const Tile t = locate_tile(a, tile_prefix, tile);
            const int acc = local_tile & 1, use = local_tile >> 1;
            const int m = t.m0 + 128 * int(cta_rank) + row;        // row inside the expert's region (or of the per-expert output)
            const bool wgrad_fp32 = a.mode == kModeWgrad and not a.out_bf16;
            const size_t wgrad_index = a.mode == kModeWgrad ? (size_t(t.expert) * a.m + m) * a.n + t.n0 : 0;
            if (not ptx::mbarrier_wait(&tmem_full_bar[acc], use & 1)) { error_flag = 1; break; }
            tc::fence_after_thread_sync();
            const uint32_t taddr = tmem_base + acc * 256 + (uint32_t(quarter * 32) << 16);
            if (wgrad_fp32) {
                staging.store_rows(&map_d, taddr, kPairN / 32, t.n0, t.expert * a.m + t.m0 + 128 * int(cta_rank) + quarter * 32,
                                   t.num_k_blocks > 0, a.accumulate, lane);
            } else if (a.mode == kModeWgrad and use_tma) {
                staging.store_rows_bf16(&map_d, taddr, kPairN / 64, t.n0, t.expert * a.m + t.m0 + 128 * int(cta_rank) + quarter * 32,
                                        t.num_k_blocks > 0, true, lane);
            } else if (a.mode == kModeWgrad) {
                __nv_bfloat16* out16 = reinterpret_cast<__nv_bfloat16*>(a.d) + wgrad_index;
                for (int c = 0; c < kPairN; c += 32) {
                    uint32_t r[32];
                    if (t.num_k_blocks > 0) {
                        tc::tmem_ld_32x32(taddr + c, r);
                        tc::wait_ld();
                    } else {
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = 0;
                    }
                    #pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        int4 packed;
                        uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                        #pragma unroll
                        for (int i = 0; i < 4; ++i)
                            w[i] = ptx::float2_to_bf16x2(__uint_as_float(r[8 * v + 2 * i]), __uint_as_float(r[8 * v + 2 * i + 1]));
                        *reinterpret_cast<int4*>(out16 + c + 8 * v) = packed;
                    }
                }
            } else {
                const bool valid = m < t.count, written = m < t.aligned_count;
                const size_t grow = size_t(t.row_base + m);
                if (a.epilogue != kEpilogueStore) {
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + grow * a.n_out + t.n0;
                    __nv_bfloat16* keep = a.epilogue == kEpilogueSwiGLUKeep ? reinterpret_cast<__nv_bfloat16*>(a.d2) + grow * a.n + t.n0 : nullptr;
                    const float scale = (valid and a.row_scale != nullptr) ? a.row_scale[grow] : 1.0f;
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t g[32], u[32];
                        tc::tmem_ld_32x32(taddr + c, g);
                        tc::tmem_ld_32x32(taddr + 128 + c, u);
                        tc::wait_ld();
                        if (not written) continue;
                        #pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            int4 packed, pg, pu;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                            uint32_t* wg = reinterpret_cast<uint32_t*>(&pg);
                            uint32_t* wu = reinterpret_cast<uint32_t*>(&pu);
                            #pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int j = 8 * v + 2 * i;
                                const float g0 = valid ? __uint_as_float(g[j]) : 0.f, g1 = valid ? __uint_as_float(g[j + 1]) : 0.f;
                                const float u0 = valid ? __uint_as_float(u[j]) : 0.f, u1 = valid ? __uint_as_float(u[j + 1]) : 0.f;
                                w[i] = ptx::float2_to_bf16x2(silu(g0) * u0 * scale, silu(g1) * u1 * scale);
                                wg[i] = ptx::float2_to_bf16x2(g0, g1), wu[i] = ptx::float2_to_bf16x2(u0, u1);
                            }
                            *reinterpret_cast<int4*>(out + c + 8 * v) = packed;
                            if (keep != nullptr) {
                                *reinterpret_cast<int4*>(keep + c + 8 * v) = pg;
                                *reinterpret_cast<int4*>(keep + a.n / 2 + c + 8 * v) = pu;
                            }
                        }
                    }
                } else if (use_tma and a.route == nullptr and t.m0 + 128 * int(cta_rank) + quarter * 32 + 32 <= t.aligned_count) {
                    // all 32 rows of this warp are written (values, or zeros for padding rows): whole chunks through the TMA
                    staging.store_rows_bf16(&map_d, taddr, kPairN / 64, t.n0, t.row_base + t.m0 + 128 * int(cta_rank) + quarter * 32,
                                            true, valid, lane);
                } else {
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + grow * a.n_out + t.n0;
                    if (a.route != nullptr and valid) {
                        // a row that is its token's only contribution from this rank goes straight to the token's owner
                        const unsigned long long target = __ldg(a.route + grow);
                        if (target != 0) out = reinterpret_cast<__nv_bfloat16*>(target) + t.n0, stored_remotely = true;
                    }
                    for (int c = 0; c < kPairN; c += 32) {
                        uint32_t r[32];
                        tc::tmem_ld_32x32(taddr + c, r);
                        tc::wait_ld();
                        if (not written) continue;
                        #pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            int4 packed;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
                            #pragma unroll
                            for (int i = 0; i < 4; ++i)
                                w[i] = valid ? ptx::float2_to_bf16x2(__uint_as_float(r[8 * v + 2 * i]), __uint_as_float(r[8 * v + 2 * i + 1])) : 0u;
                            *reinterpret_cast<int4*>(out + c + 8 * v) = packed;
                        }
                    }
                }
            }
            tc::fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) tc::mbarrier_arrive_cluster(tc::map_to_cta(&tmem_empty_bar[acc], 0));
        }
        if (stored_remotely) __threadfence_system();     // peer stores are performed before the kernel completes
        staging.drain(lane);
    }

    // ---- teardown: no CTA leaves while its partner may still signal its barriers or read its shared memory
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::cluster_sync();
    if (warp == 1) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc_pair(tmem_base, 512);
    }
    // a bounded wait ran out: leave a mark where the host finds it (mapped host memory) before its next launch
    if (threadIdx.x == 0 and error_flag and a.status != nullptr) {
        *reinterpret_cast<volatile int*>(a.status) = 1;
        __threadfence_system();
    }
}

}  // namespace deep_ep::kernels
