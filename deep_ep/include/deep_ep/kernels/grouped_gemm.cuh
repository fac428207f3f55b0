// Grouped BF16 GEMM for the expert FFNs of an MoE layer on sm_100a tensor cores.
//
// One persistent kernel, 192 threads per CTA, three roles:
//   warp 0   TMA producer   tiled `cp.async.bulk.tensor` loads of A and B tiles (128-byte swizzle) into a
//                           shared-memory ring, completion on mbarriers
//   warp 1   MMA issuer     one elected thread issues `tcgen05.mma` (M = 128, N = BLOCK_N, K = 16 per
//                           instruction) with the accumulator in tensor memory, double buffered so that
//                           the epilogue of tile i overlaps the main loop of tile i + 1
//   warps 2-5 epilogue      `tcgen05.ld` the accumulator (one row per thread), optional SwiGLU or fp32
//                           accumulate, vector stores to global memory
//
// Three problem shapes, all over the expanded dispatch layout (expert e owns rows
// `[psum[e] - count[e], psum[e])`, regions padded to the expert alignment):
//   kModeForward   D[rows_e, N]  = A[rows_e, K] * B_e[N, K]^T          (A and B K-major)
//   kModeDgrad     D[rows_e, N]  = A[rows_e, K] * B_e[K, N]            (B MN-major: the weight as stored)
//   kModeWgrad     D_e[M, N]    += A[rows_e, M]^T * B[rows_e, N]       (both MN-major, K = tokens of expert e)
// The reference contains no matrix math; this kernel exists for the fused MoE layer that the library is
// benchmarked in.
#pragma once

#include "../device/sync.cuh"
#include "../device/tcgen05.cuh"
#include "grouped_gemm_args.hpp"

namespace deep_ep::kernels {

namespace gemm_detail {

EP_DEVICE float silu(float x) { return x / (1.0f + __expf(-x)); }

struct Tile {
    int expert, m0, n0, row_base, rows_valid, rows_written, num_k_blocks;
};

// tile index -> (expert, m block, n block). `prefix` holds the exclusive prefix of tiles per expert.
EP_DEVICE Tile locate_tile(const GroupedGemmArgs& a, const int* prefix, int tile) {
    int lo = 0, hi = a.num_groups - 1;
    while (lo < hi) {                       // last expert whose prefix <= tile
        const int mid = (lo + hi + 1) >> 1;
        if (prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const int e = lo, local = tile - prefix[e];
    const int count = a.count[e], start = a.psum[e] - count;
    Tile t;
    t.expert = e, t.row_base = start;
    if (a.mode == kModeWgrad) {
        const int m_tiles = a.m / kGemmBlockM;
        t.m0 = (local % m_tiles) * kGemmBlockM, t.n0 = (local / m_tiles) * a.block_n;
        t.rows_valid = t.rows_written = kGemmBlockM, t.num_k_blocks = math::ceil_div(count, kGemmBlockK);
    } else {
        const int m_tiles = math::ceil_div(count, kGemmBlockM);
        t.m0 = (local % m_tiles) * kGemmBlockM, t.n0 = (local / m_tiles) * a.block_n_out;
        t.rows_valid = min(kGemmBlockM, count - t.m0), t.num_k_blocks = math::ceil_div(a.k, kGemmBlockK);
        // padding rows of the expert's aligned region that fall into this tile are written as zeros
        t.rows_written = min(kGemmBlockM, math::align(count, max(a.alignment, 1)) - t.m0);
    }
    return t;
}

// fp32 weight-gradient tiles leave the CTA through shared memory and the TMA. An epilogue thread holds one accumulator row
// (`tcgen05.ld` 32x32b), so a warp-wide store from registers would touch 32 different rows, 16 bytes each, per instruction,
// and with `accumulate` every 16 bytes would also be a round trip for the previous contents. Instead each warp writes its
// 32 rows x 32 columns chunk (4 KB) into a staging buffer, laid out in the 128-byte swizzle the tensor map expects (which
// also makes the writes bank-conflict free), and one lane hands it to the TMA: a plain tiled store, or a tiled
// reduce-add (`cp.reduce.async.bulk.tensor ... .add`) that performs the fp32 accumulation at the memory side with no
// load in the SM at all. Two buffers per warp alternate; a buffer is reused once the copy that read it has done so.
struct WgradStaging {
    static constexpr int kChunkBytes = 32 * 128;          // 32 rows x 32 fp32 (or x 64 bf16)
    uint8_t* buffers;                                     // this warp's chunk buffers (1024-byte aligned)
    int num_buffers = 2;                                  // 1 or 2
    unsigned issued = 0;

    // one chunk: wait until the buffer is free, write `units[8]` (the row's 128 bytes) swizzled, hand it to the TMA
    EP_DEVICE void push(const CUtensorMap* map_d, const uint4 (&units)[8], int x, int y, bool accumulate, int lane) {
        uint8_t* buffer = buffers + (num_buffers == 2 ? (issued & 1) : 0) * kChunkBytes;
        // the copy that last read this buffer has done so (lane 0 owns the bulk groups)
        if (lane == 0) {
            if (num_buffers == 2) ptx::bulk_wait_read<1>();
            else ptx::bulk_wait_read<0>();
        }
        __syncwarp();
        #pragma unroll
        for (int v = 0; v < 8; ++v)             // 16-byte unit v of row `lane` sits at unit v ^ (row % 8) of its 128-byte line
            *reinterpret_cast<uint4*>(buffer + lane * 128 + ((v ^ (lane & 7)) << 4)) = units[v];
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            if (accumulate) tc::tma_reduce_add_2d(map_d, x, y, buffer);
            else tc::tma_store_2d(map_d, x, y, buffer);
            ptx::bulk_commit();
        }
        ++issued;
    }

    // bf16 rows: `num_chunks` chunks of 64 columns; rows whose `valid` is false are written as zeros
    EP_DEVICE void store_rows_bf16(const CUtensorMap* map_d, uint32_t taddr, int num_chunks, int x0, int y0, bool has_accumulator,
                                   bool valid, int lane) {
        for (int i = 0; i < num_chunks; ++i) {
            uint32_t lo[32], hi[32];
            if (has_accumulator) {
                tc::tmem_ld_32x32(taddr + 64 * i, lo);
                tc::tmem_ld_32x32(taddr + 64 * i + 32, hi);
                tc::wait_ld();
            }
            uint4 units[8];
            #pragma unroll
            for (int v = 0; v < 4; ++v) {
                uint32_t* w = reinterpret_cast<uint32_t*>(&units[v]);
                uint32_t* w2 = reinterpret_cast<uint32_t*>(&units[4 + v]);
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const bool keep = valid and has_accumulator;
                    w[j] = keep ? ptx::float2_to_bf16x2(__uint_as_float(lo[8 * v + 2 * j]), __uint_as_float(lo[8 * v + 2 * j + 1])) : 0u;
                    w2[j] = keep ? ptx::float2_to_bf16x2(__uint_as_float(hi[8 * v + 2 * j]), __uint_as_float(hi[8 * v + 2 * j + 1])) : 0u;
                }
            }
            push(map_d, units, x0 + 64 * i, y0, false, lane);
        }
    }

    EP_DEVICE void store_rows(const CUtensorMap* map_d, uint32_t taddr, int num_chunks, int x0, int y0, bool has_accumulator,
                              bool accumulate, int lane) {
        for (int i = 0; i < num_chunks; ++i) {
            uint32_t r[32];
            if (has_accumulator) {
                tc::tmem_ld_32x32(taddr + 32 * i, r);
                tc::wait_ld();
            } else {
                #pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0;
            }
            uint4 units[8];
            #pragma unroll
            for (int v = 0; v < 8; ++v) units[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            push(map_d, units, x0 + 32 * i, y0, accumulate, lane);
        }
    }
    // every copy has been performed (call before the kernel ends)
    EP_DEVICE void drain(int lane) {
        if (lane == 0) ptx::bulk_wait<0>();
        __syncwarp();
    }
};

// TMA boxes of one K block of a tile into the shared-memory stage (`sa`, `sb`, completion on `bar`).
EP_DEVICE void load_k_block(const GroupedGemmArgs& a, const CUtensorMap& map_a, const CUtensorMap& map_b, const Tile& t, int kb,
                            int BN, uint8_t* sa, uint8_t* sb, uint64_t* bar) {
    auto box = [&](uint8_t* dst, const CUtensorMap* map, int x, int y) { tc::tma_load_2d(dst, map, x, y, bar); };
    const int k0 = kb * kGemmBlockK;
    if (a.mode == kModeWgrad) {
        // A = dY^T: source rows are K, columns (contiguous) are M
        for (int i = 0; i < kGemmBlockM / 64; ++i) box(sa + i * 8192, &map_a, t.m0 + 64 * i, t.row_base + k0);
        for (int i = 0; i < BN / 64; ++i) box(sb + i * 8192, &map_b, t.n0 + 64 * i, t.row_base + k0);
        return;
    }
    box(sa, &map_a, k0, t.row_base + t.m0);
    if (a.mode == kModeForward) {
        // K-major weights [G * N, K]; with SwiGLU the tile pairs 128 gate rows with 128 up rows
        const int row = t.expert * a.n;
        if (a.epilogue != kEpilogueStore) {
            box(sb, &map_b, k0, row + t.n0);
            box(sb + 128 * 128, &map_b, k0, row + a.n / 2 + t.n0);
        } else {
            for (int i = 0; i < BN / 128; ++i) box(sb + i * 128 * 128, &map_b, k0, row + t.n0 + 128 * i);
        }
    } else {
        // MN-major weights [G * K, N]
        for (int i = 0; i < BN / 64; ++i) box(sb + i * 8192, &map_b, t.n0 + 64 * i, t.expert * a.k + k0);
    }
}

}  // namespace gemm_detail

__global__ void __launch_bounds__(192, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_d, const __grid_constant__ GroupedGemmArgs a) {
    using namespace gemm_detail;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kGemmMaxStages], empty_bar[kGemmMaxStages], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int tile_prefix[kMaxLocalExperts + 1];
    __shared__ volatile int error_flag;

    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    const int S = a.num_stages, BN = a.block_n;
    const uint32_t a_bytes = kGemmBlockM * kGemmBlockK * 2, b_bytes = uint32_t(BN) * kGemmBlockK * 2;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + size_t(S) * a_bytes;

    // ---- setup: barriers, tile schedule, tensor memory
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) ptx::mbarrier_init(&full_bar[s], 1), ptx::mbarrier_init(&empty_bar[s], 1);
        for (int i = 0; i < 2; ++i) ptx::mbarrier_init(&tmem_full_bar[i], 1), ptx::mbarrier_init(&tmem_empty_bar[i], 4);
        ptx::fence_mbarrier_init();
        error_flag = 0;
        tc::prefetch_tensormap(&map_a), tc::prefetch_tensormap(&map_b);
    }
    if (warp == 1) tc::tmem_alloc(&tmem_base_slot, 512);
    if (warp == 2) {
        // exclusive prefix of tiles per expert (one warp, chunks of 32 experts)
        int carry = 0;
        for (int base = 0; base < a.num_groups; base += 32) {
            const int e = base + lane;
            int tiles = 0;
            if (e < a.num_groups) {
                const int count = a.count[e];
                if (a.mode == kModeWgrad) tiles = (count > 0 or not a.accumulate) ? (a.m / kGemmBlockM) * (a.n / BN) : 0;
                else tiles = math::ceil_div(count, kGemmBlockM) * (a.n_out / a.block_n_out);
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
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = tmem_base_slot;
    const int num_tiles = tile_prefix[a.num_groups];

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // ring position: stage index and phase bit, advanced without divisions (this loop is one thread's
            // critical path: it must stay shorter than the 512 cycles a K block occupies the tensor core)
            int s = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x) {
                const Tile t = locate_tile(a, tile_prefix, tile);
                for (int kb = 0; kb < t.num_k_blocks; ++kb, s = (s + 1 == S ? 0 : s + 1), phase ^= (s == 0)) {
                    if (not ptx::mbarrier_wait(&empty_bar[s], phase ^ 1)) { error_flag = 1; break; }
                    ptx::mbarrier_arrive_expect_tx(&full_bar[s], a_bytes + b_bytes);
                    load_k_block(a, map_a, map_b, t, kb, BN, smem_a + size_t(s) * a_bytes, smem_b + size_t(s) * b_bytes, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const bool a_mn = a.mode == kModeWgrad, b_mn = a.mode != kModeForward;
            const uint32_t idesc = tc::make_idesc(tc::kFormatBF16, kGemmBlockM, BN, a_mn, b_mn);
            // descriptor strides: K-major -> 8-row groups 1024 B apart; MN-major -> K atoms 1024 B apart, 64-wide blocks 8192 B apart
            const uint32_t a_lead = a_mn ? 8192 : 16, b_lead = b_mn ? 8192 : 16;
            const uint32_t a_kstep = a_mn ? 2048 : 32, b_kstep = b_mn ? 2048 : 32;     // bytes per K = 16
            // descriptors of stage 0; other stages and K steps differ only in the 14-bit address field (units of 16 bytes)
            const uint64_t desc_a0 = tc::make_smem_desc(smem_a, a_lead, 1024), desc_b0 = tc::make_smem_desc(smem_b, b_lead, 1024);
            const uint32_t a_stage_step = a_bytes >> 4, b_stage_step = b_bytes >> 4;
            const uint32_t a_k = a_kstep >> 4, b_k = b_kstep >> 4;
            int s = 0, local_tile = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x, ++local_tile) {
                const Tile t = locate_tile(a, tile_prefix, tile);
                const int acc = local_tile & 1, use = local_tile >> 1;
                if (not ptx::mbarrier_wait(&tmem_empty_bar[acc], (use & 1) ^ 1)) { error_flag = 1; break; }
                tc::fence_after_thread_sync();
                const uint32_t tmem_d = tmem_base + acc * 256;
                for (int kb = 0; kb < t.num_k_blocks; ++kb, s = (s + 1 == S ? 0 : s + 1), phase ^= (s == 0)) {
                    if (not ptx::mbarrier_wait(&full_bar[s], phase)) { error_flag = 1; break; }
                    tc::fence_after_thread_sync();
                    const uint64_t da = desc_a0 + uint64_t(s * a_stage_step), db = desc_b0 + uint64_t(s * b_stage_step);
                    #pragma unroll
                    for (int k = 0; k < kGemmBlockK / 16; ++k)
                        tc::mma_f16(tmem_d, da + uint64_t(k * a_k), db + uint64_t(k * b_k), idesc, kb > 0 or k > 0);
                    tc::commit(&empty_bar[s]);          // stage is free once these MMAs have read it
                }
                if (t.num_k_blocks > 0) tc::commit(&tmem_full_bar[acc]);        // accumulator complete
                else ptx::mbarrier_arrive(&tmem_full_bar[acc]);                 // nothing to wait for: the epilogue writes zeros
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;                    // tensor-memory lane quarter this warp may access
        const int row = quarter * 32 + lane;
        int local_tile = 0;
        bool stored_remotely = false;
        // results that leave through the TMA: staging buffers of this warp behind the operand ring (see WgradStaging)
        WgradStaging staging;
        staging.num_buffers = max(a.staging_buffers, 1);
        staging.buffers = smem_b + size_t(S) * b_bytes + size_t(quarter) * staging.num_buffers * WgradStaging::kChunkBytes;
        const bool use_tma = a.staging_buffers > 0;
        for (int tile = blockIdx.x; tile < num_tiles and not error_flag; tile += gridDim.x, ++local_tile) {
            const Tile t = locate_tile(a, tile_prefix, tile);
            const int acc = local_tile & 1, use = local_tile >> 1;
            const bool wgrad_fp32 = a.mode == kModeWgrad and not a.out_bf16;
            if (not ptx::mbarrier_wait(&tmem_full_bar[acc], use & 1)) { error_flag = 1; break; }
            tc::fence_after_thread_sync();
            const uint32_t taddr = tmem_base + acc * 256 + (uint32_t(quarter * 32) << 16);
            const bool valid = row < t.rows_valid;
            if (wgrad_fp32) {
                staging.store_rows(&map_d, taddr, BN / 32, t.n0, t.expert * a.m + t.m0 + quarter * 32, t.num_k_blocks > 0,
                                   a.accumulate, lane);
            } else if (a.mode == kModeWgrad and use_tma) {
                staging.store_rows_bf16(&map_d, taddr, BN / 64, t.n0, t.expert * a.m + t.m0 + quarter * 32, t.num_k_blocks > 0, true, lane);
            } else if (a.mode == kModeWgrad) {
                const size_t out_index = (size_t(t.expert) * a.m + t.m0 + row) * a.n + t.n0;
                __nv_bfloat16* out16 = reinterpret_cast<__nv_bfloat16*>(a.d) + out_index;
                for (int c = 0; c < BN; c += 32) {
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
            } else if (a.epilogue != kEpilogueStore) {
                const size_t grow = size_t(t.row_base + t.m0 + row);
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + grow * a.n_out + t.n0;
                __nv_bfloat16* keep = a.epilogue == kEpilogueSwiGLUKeep ? reinterpret_cast<__nv_bfloat16*>(a.d2) + grow * a.n + t.n0 : nullptr;
                const bool written = row < t.rows_written;
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
            } else if (use_tma and a.route == nullptr and not a.out_fp32 and quarter * 32 + 32 <= t.rows_written) {
                // all 32 rows of this warp are written (values, or zeros for padding rows): whole chunks through the TMA
                staging.store_rows_bf16(&map_d, taddr, BN / 64, t.n0, t.row_base + t.m0 + quarter * 32, true, valid, lane);
            } else {
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.d) + size_t(t.row_base + t.m0 + row) * a.n_out + t.n0;
                if (a.route != nullptr and valid) {
                    // a row that is its token's only contribution from this rank goes straight to the token's owner
                    const unsigned long long target = __ldg(a.route + t.row_base + t.m0 + row);
                    if (target != 0) out = reinterpret_cast<__nv_bfloat16*>(target) + t.n0, stored_remotely = true;
                }
                const bool written = row < t.rows_written;
                float* out32 = reinterpret_cast<float*>(a.d) + size_t(t.row_base + t.m0 + row) * a.n_out + t.n0;
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(taddr + c, r);
                    tc::wait_ld();
                    if (not written) continue;
                    if (a.out_fp32) {
                        // fp32 result (router logits): the accumulator is stored as it is
                        #pragma unroll
                        for (int v = 0; v < 8; ++v)
                            *reinterpret_cast<uint4*>(out32 + c + 4 * v) =
                                valid ? make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]) : make_uint4(0, 0, 0, 0);
                        continue;
                    }
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
            tc::fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) ptx::mbarrier_arrive(&tmem_empty_bar[acc]);
        }
        if (stored_remotely) __threadfence_system();     // peer stores are performed before the kernel completes
        staging.drain(lane);
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
