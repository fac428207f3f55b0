// Expert-parallel combine for sm_100a.
//   `ep_combine_kernel` (issue): for every token this rank received, gather its expanded rows,
//       reduce them in fp32 in top-k order, round once to bf16 and push the partial (plus the
//       positionally routed top-k weights) into the owner rank's landing buffer with one
//       `cp.async.bulk` store. Single-row tokens go global -> shared -> peer without touching registers.
//   `ep_combine_reduce_kernel` (epilogue): after every peer's "push finished" flag, the owner sums
//       bias + partials in top-k slot order in fp32 and rounds once to bf16.
// Roles of the reference's `impls/ep/combine.hpp:25-364` and `impls/ep/combine_reduce_epilogue.hpp:19-155`;
// the accumulation order is the one its oracle demands bit for bit (`deep_ep/utils/refs.py:178-247`).
#pragma once

#include "../device/sync.cuh"
#include "ep_args.hpp"
#include "ep_dispatch.cuh"

namespace deep_ep::kernels {



namespace combine_detail {

constexpr int kSiteEntryBarrier = 30, kSiteGridSync = 31, kSiteLoad = 32, kSiteArrival = 33, kSitePush = 34;
constexpr int kUnroll = 8;


EP_DEVICE void accumulate(float (&acc)[8], const int4& v) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = ptx::bf16x2_to_float2(w[i]);
        acc[2 * i] += f.x, acc[2 * i + 1] += f.y;
    }
}

EP_DEVICE int4 pack(const float (&acc)[8]) {
    int4 out;
    uint32_t* w = reinterpret_cast<uint32_t*>(&out);
    #pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = ptx::float2_to_bf16x2(acc[2 * i], acc[2 * i + 1]);
    return out;
}

// index (0-based) of the q-th set bit of m; requires q < popc(m)
EP_DEVICE int nth_set_bit(unsigned m, int q) { return __fns(m, 0, q + 1); }

// fp32 sum, in top-k order, of `count` expanded rows (slots held one per lane, `valid` = lanes that hold one)
// into a bf16 row in shared memory. Several 16-byte chunks per lane are loaded before the first add so that
// enough requests are in flight to cover memory latency.
template <int kSlots, int kChunks>
EP_DEVICE void reduce_rows_impl(const uint8_t* x, int hidden_bytes, int c_begin, int chunks, const int (&sl)[kSlots], uint8_t* stage, int lane) {
    for (int c0 = c_begin + lane; c0 < chunks; c0 += 32 * kChunks) {
        int4 v[kChunks][kSlots];
        #pragma unroll
        for (int i = 0; i < kChunks; ++i)
            #pragma unroll
            for (int u = 0; u < kSlots; ++u)
                if (c0 + 32 * i < chunks and sl[u] >= 0) v[i][u] = ptx::ld_nc_v4(x + int64_t(sl[u]) * hidden_bytes + (c0 + 32 * i) * 16);
        #pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            if (c0 + 32 * i >= chunks) break;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            #pragma unroll
            for (int u = 0; u < kSlots; ++u)
                if (sl[u] >= 0) accumulate(acc, v[i][u]);
            *reinterpret_cast<int4*>(stage + (c0 + 32 * i) * 16) = pack(acc);
        }
    }
}

// Works on the 16-byte chunks [c_begin, chunks) of the row (several warps may split a row between them).
EP_DEVICE void reduce_rows(const uint8_t* x, int hidden_bytes, int c_begin, int chunks, int my_slot, unsigned valid, int count,
                           uint8_t* stage, int lane) {
    if (count <= 4) {
        int sl[4];
        unsigned left = valid;
        #pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = __shfl_sync(0xffffffffu, my_slot, left != 0 ? __ffs(left) - 1 : 0);
            sl[u] = left != 0 ? v : -1;
            left &= left - 1;
        }
        if (count == 2) {
            const int s2[2] = {sl[0], sl[1]};
            reduce_rows_impl<2, 4>(x, hidden_bytes, c_begin, chunks, s2, stage, lane);
        } else {
            reduce_rows_impl<4, 4>(x, hidden_bytes, c_begin, chunks, sl, stage, lane);
        }
    } else if (count <= 8) {
        int sl[8];
        unsigned left = valid;
        #pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int v = __shfl_sync(0xffffffffu, my_slot, left != 0 ? __ffs(left) - 1 : 0);
            sl[u] = left != 0 ? v : -1;
            left &= left - 1;
        }
        reduce_rows_impl<8, 2>(x, hidden_bytes, c_begin, chunks, sl, stage, lane);
    } else {
        for (int base = c_begin; base < chunks; base += 32) {       // warp-uniform trip count: shuffles inside
            const int c = base + lane;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int u = 0; u < count; ++u) {
                const int slot = __shfl_sync(0xffffffffu, my_slot, nth_set_bit(valid, u));
                if (c < chunks) accumulate(acc, ptx::ld_nc_v4(x + int64_t(slot) * hidden_bytes + c * 16));
            }
            if (c < chunks) *reinterpret_cast<int4*>(stage + c * 16) = pack(acc);
        }
    }
}

EP_DEVICE void accumulate_scaled(float (&acc)[8], const int4& v, float scale) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = ptx::bf16x2_to_float2(w[i]);
        acc[2 * i] = fmaf(scale, f.x, acc[2 * i]), acc[2 * i + 1] = fmaf(scale, f.y, acc[2 * i + 1]);
    }
}

// Opt-in weighted variant: fp32 sum of `weight_j * row_j` in top-k order, one rounding to bf16 (lane j holds the slot and
// the weight of top-k position j). Four chunks per lane are in flight per row.
EP_DEVICE void reduce_rows_weighted(const uint8_t* x, int hidden_bytes, int c_begin, int chunks, int my_slot, float my_weight,
                                    unsigned valid, int count, uint8_t* stage, int lane) {
    for (int base = c_begin; base < chunks; base += 32 * 4) {           // warp-uniform trip count: shuffles inside
        float acc[4][8];
        #pragma unroll
        for (int i = 0; i < 4; ++i)
            #pragma unroll
            for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
        for (int u = 0; u < count; ++u) {
            const int src_lane = nth_set_bit(valid, u);
            const int slot = __shfl_sync(0xffffffffu, my_slot, src_lane);
            const float weight = __shfl_sync(0xffffffffu, my_weight, src_lane);
            int4 v[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = base + 32 * i + lane;
                if (c < chunks) v[i] = ptx::ld_nc_v4(x + int64_t(slot) * hidden_bytes + c * 16);
            }
            #pragma unroll
            for (int i = 0; i < 4; ++i)
                if (base + 32 * i + lane < chunks) accumulate_scaled(acc[i], v[i], weight);
        }
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = base + 32 * i + lane;
            if (c < chunks) *reinterpret_cast<int4*>(stage + c * 16) = pack(acc[i]);
        }
    }
}

// Owner-side reduction of one token: fp32 sum of the rows `part[0..kParts)` (null entries skipped) in index order, one
// rounding to bf16. The caller lists bias_0, bias_1 and then the partials in slot order. `kChunks` 16-byte chunks per lane
// and row are in flight before the first add.
template <int kParts, int kChunks>
EP_DEVICE void reduce_token(const uint8_t* const (&part)[kParts], uint8_t* out, int c_begin, int chunks, int lane) {
    for (int c0 = c_begin + lane; c0 < chunks; c0 += 32 * kChunks) {
        int4 v[kChunks][kParts];
        #pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            const int c = c0 + 32 * i;
            if (c >= chunks) continue;
            #pragma unroll
            for (int u = 0; u < kParts; ++u)
                if (part[u] != nullptr) v[i][u] = ptx::ld_v4(part[u] + c * 16);
        }
        #pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            const int c = c0 + 32 * i;
            if (c >= chunks) continue;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            #pragma unroll
            for (int u = 0; u < kParts; ++u)
                if (part[u] != nullptr) accumulate(acc, v[i][u]);
            ptx::st_na_v4(out + c * 16, pack(acc));
        }
    }
}

}  // namespace combine_detail

// Kernel body; non-zero template arguments replace the corresponding run-time shape values by compile-time constants
// (see `ep_dispatch_body`): zeros for the ahead-of-time kernel below, the shapes in use for run-time specialised kernels.
template <int kNumRanks, int kNumTopk, int kHiddenBytes>
EP_DEVICE void ep_combine_body(const CombineArgs& a) {
    using namespace combine_detail;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int psum_rank_smem[kMaxRanks];

    const int num_ranks = kNumRanks > 0 ? kNumRanks : a.peers.num_ranks, rank = a.peers.rank;
    const int hidden_bytes = kHiddenBytes > 0 ? kHiddenBytes : a.hidden_bytes;
    const int num_ctas = gridDim.x, cta = blockIdx.x;
    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    const int W = a.num_warps, S = a.num_stages, k = kNumTopk > 0 ? kNumTopk : a.num_topk;
    layout::CommonSignals* cs = &a.ws->common;
    layout::HostStatus* hs = a.host ? &a.host->status : nullptr;
    const layout::CombineTokenLayout tl(hidden_bytes, k);
    const int token_bytes = tl.num_bytes();
    const int num_groups = min(k, num_ranks);
    const layout::BufferLayout bl(token_bytes, num_groups, a.num_max_tokens);

    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint64_t* mbar = reinterpret_cast<uint64_t*>(base) + warp * S;
    uint8_t* stages = base + math::align<int64_t>(int64_t(W) * S * 8, 128) + int64_t(warp) * S * token_bytes;

    if (not dev::healthy(cs)) return;
    const unsigned epoch = a.ws->combine_epoch + 1;
    const bool tracer = cta == 0 and threadIdx.x == 0;
    if (tracer) dev::trace_point(a.trace, kTrCombStart);
    if (threadIdx.x == 0) {
        for (int i = 0; i < W * S; ++i) ptx::mbarrier_init(reinterpret_cast<uint64_t*>(base) + i, 1);
        ptx::fence_mbarrier_init();
    }
    for (int s = threadIdx.x; s < num_ranks; s += blockDim.x) psum_rank_smem[s] = a.psum_rank[s];
    __syncthreads();

    // Entry barrier: every peer has finished the dispatch epilogue that read the shared buffer.
    if (cta == 0 and warp == 0) dev::rank_barrier_warp(cs, hs, a.peers, a.timeout_ns, kSiteEntryBarrier);
    if (tracer) dev::trace_point(a.trace, kTrCombEntryBarrier);
    if (not dev::grid_sync(cs, hs, num_ctas, a.timeout_ns, rank, kSiteGridSync)) return;
    if (tracer) dev::trace_point(a.trace, kTrCombGridSync);

    const int gw = cta * W + warp, num_gw = num_ctas * W;
    const int meta_cols = k + 2;
    const int chunks = hidden_bytes / 16;
    int n = 0;            // rows processed by this warp (stage / parity counter)
    int num_loads[4] = {0, 0, 0, 0};   // bulk loads issued per stage (mbarrier parity)
    bool failed = false;

    // Decode-sized calls leave most warps without a row while the few busy ones walk through a row in a dozen
    // dependent round trips. With `coop`, P warps of a CTA (a power of two, the same in the whole CTA) share every
    // row: each reduces 1/P of the 16-byte chunks into the group's stage and the group's first warp sends it.
    // all received rows, and the first row of the source after this rank (where this rank starts, so that the ranks of a
    // node begin with different destinations)
    const int total_rows = min(psum_rank_smem[num_ranks - 1], a.num_metadata_rows);
    const int next_rank = (rank + 1) % num_ranks;
    const int first_row = total_rows > 0 ? (next_rank == 0 ? 0 : min(psum_rank_smem[next_rank - 1], total_rows)) % total_rows : 0;
    int P = 1;
    if (a.coop) {
        while (2 * P <= W and W % (2 * P) == 0 and int64_t(total_rows) * (2 * P) <= num_gw) P *= 2;
    }
    if (P > 1) {
        const int group = warp / P, part = warp % P, groups_per_cta = W / P;
        const int gg = cta * groups_per_cta + group, num_gg = num_ctas * groups_per_cta;
        uint8_t* group_stages = base + math::align<int64_t>(int64_t(W) * S * 8, 128) + int64_t(group * P) * S * token_bytes;
        const int c_begin = chunks * part / P, c_end = chunks * (part + 1) / P;
        const int bar_id = 1 + group, bar_threads = 32 * P;
        // rows are scarce here: one flat walk over all received rows (see the note at the loop of the other path)
        for (int i = gg; i < total_rows; i += num_gg, ++n) {
            const int row = (i + first_row) % total_rows;
            int s = 0;
            while (s < num_ranks - 1 and row >= psum_rank_smem[s]) ++s;
            {
                // every warp of the group reads the same metadata and therefore takes the same branches
                uint8_t* stage = group_stages + (n % S) * token_bytes;
                const int my_slot = lane < k ? a.recv_src_metadata[int64_t(row) * meta_cols + lane] : -1;
                int src_global = 0, master = 0;
                if (lane == 0) {
                    src_global = a.recv_src_metadata[int64_t(row) * meta_cols + k];
                    master = a.recv_src_metadata[int64_t(row) * meta_cols + k + 1];
                }
                src_global = __shfl_sync(0xffffffffu, src_global, 0);
                master = __shfl_sync(0xffffffffu, master, 0);
                const unsigned valid = __ballot_sync(0xffffffffu, my_slot >= 0);
                const int count = __popc(valid);
                const int token = src_global - s * a.num_max_tokens;
                if (count == 0 or token < 0 or token >= a.num_max_tokens or master < 0) {
                    if (part == 0) ptx::bulk_commit();
                    continue;
                }
                if (count == 1 and a.skip_single) {
                    // payload already delivered by the producing GEMM: the group's first warp sends the weights alone
                    if (part == 0) {
                        dispatch_detail::wait_read_pending(S - 1);
                        __syncwarp();
                        if (a.topk_weights != nullptr) {
                            if (lane < k)
                                reinterpret_cast<float*>(stage + tl.weight_offset())[lane] = my_slot >= 0 ? a.topk_weights[my_slot] : 0.f;
                            ptx::fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                const int dst_group = num_ranks >= k ? master : rank;
                                dev::store_message(cs, hs, a.peers, s, a.buffer_offset, a.buffer_bytes, bl.offset(dst_group, token) + tl.weight_offset(),
                                                   stage + tl.weight_offset(), token_bytes - tl.weight_offset(), kSitePush);
                            }
                        }
                        ptx::bulk_commit();
                    }
                    continue;
                }
                if (part == 0) dispatch_detail::wait_read_pending(S - 1);     // the store issued S rows ago has read the stage
                ptx::named_barrier(bar_id, bar_threads);
                if (a.weighted and a.topk_weights != nullptr)
                    reduce_rows_weighted(a.x, hidden_bytes, c_begin, c_end, my_slot, my_slot >= 0 ? a.topk_weights[my_slot] : 0.f,
                                         valid, count, stage, lane);
                else
                    reduce_rows(a.x, hidden_bytes, c_begin, c_end, my_slot, valid, count, stage, lane);
                if (part == 0 and lane < k)
                    reinterpret_cast<float*>(stage + tl.weight_offset())[lane] =
                        (my_slot >= 0 and a.topk_weights != nullptr) ? a.topk_weights[my_slot] : 0.f;
                ptx::fence_proxy_async_smem();
                ptx::named_barrier(bar_id, bar_threads);
                if (part == 0) {
                    if (lane == 0) {
                        const int dst_group = num_ranks >= k ? master : rank;
                        dev::store_message(cs, hs, a.peers, s, a.buffer_offset, a.buffer_bytes, bl.offset(dst_group, token), stage, token_bytes, kSitePush);
                    }
                    ptx::bulk_commit();
                }
            }
        }
    }

    // Two ways to hand rows to warps. Plenty of rows (bandwidth-bound calls): every warp visits the sources in an order
    // rotated by rank and warp and takes every `num_gw`-th row of each, so that at any moment the ranks of the node spread
    // their pushes over all destinations. Few rows (decode-sized calls): that scheme gives the first warps one row PER
    // SOURCE, eight rows one after the other, while most warps have none; a flat walk over all rows gives every warp at
    // most a few.
    const bool flat_walk = total_rows <= 4 * num_gw;
    const int num_outer = flat_walk ? 1 : num_ranks;
    for (int q = 0; q < num_outer and not failed and P == 1; ++q) {
        const int source = (rank + 1 + gw + q) % num_ranks;
        const int begin = flat_walk ? 0 : (source == 0 ? 0 : psum_rank_smem[source - 1]);
        const int end = flat_walk ? total_rows : min(psum_rank_smem[source], a.num_metadata_rows);
        for (int walk = begin + gw; walk < end; walk += num_gw, ++n) {
            int row = walk, s = source;
            if (flat_walk) {
                row = (walk + first_row) % total_rows;
                s = 0;
                while (s < num_ranks - 1 and row >= psum_rank_smem[s]) ++s;
            }
            const int stage_idx = n % S;
            uint8_t* stage = stages + stage_idx * token_bytes;
            const int my_slot = lane < k ? a.recv_src_metadata[int64_t(row) * meta_cols + lane] : -1;
            int src_global = 0, master = 0;
            if (lane == 0) {
                src_global = a.recv_src_metadata[int64_t(row) * meta_cols + k];
                master = a.recv_src_metadata[int64_t(row) * meta_cols + k + 1];
            }
            src_global = __shfl_sync(0xffffffffu, src_global, 0);
            master = __shfl_sync(0xffffffffu, master, 0);
            const unsigned valid = __ballot_sync(0xffffffffu, my_slot >= 0);
            const int count = __popc(valid);
            const int token = src_global - s * a.num_max_tokens;
            if (count == 0 or token < 0 or token >= a.num_max_tokens or master < 0) { ptx::bulk_commit(); continue; }

            // the stage may still be read by the store issued S rows ago
            dispatch_detail::wait_read_pending(S - 1);
            __syncwarp();

            if (count == 1 and a.skip_single) {
                // the row itself already sits in the owner's landing slot (stored there by the GEMM that produced it):
                // only the routed weights behind it are sent
                if (a.topk_weights != nullptr) {
                    if (lane < k)
                        reinterpret_cast<float*>(stage + tl.weight_offset())[lane] = my_slot >= 0 ? a.topk_weights[my_slot] : 0.f;
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const int group = num_ranks >= k ? master : rank;
                        dev::store_message(cs, hs, a.peers, s, a.buffer_offset, a.buffer_bytes, bl.offset(group, token) + tl.weight_offset(),
                                           stage + tl.weight_offset(), token_bytes - tl.weight_offset(), kSitePush);
                    }
                }
                ptx::bulk_commit();
                continue;
            }

            // opt-in: rows are multiplied by their routing weights before the sum (single rows too, so no plain copy)
            const bool weighted = a.weighted and a.topk_weights != nullptr;
            const bool single_copy = count == 1 and not weighted;
            if (single_copy) {
                const int slot = __shfl_sync(0xffffffffu, my_slot, __ffs(valid) - 1);
                if (lane == 0) {
                    ptx::mbarrier_arrive_expect_tx(&mbar[stage_idx], hidden_bytes);
                    ptx::bulk_load(stage, a.x + int64_t(slot) * hidden_bytes, hidden_bytes, &mbar[stage_idx]);
                }
            } else if (weighted) {
                reduce_rows_weighted(a.x, hidden_bytes, 0, chunks, my_slot, my_slot >= 0 ? a.topk_weights[my_slot] : 0.f, valid,
                                     count, stage, lane);
            } else {
                reduce_rows(a.x, hidden_bytes, 0, chunks, my_slot, valid, count, stage, lane);
            }
            if (lane < k)
                reinterpret_cast<float*>(stage + tl.weight_offset())[lane] =
                    (my_slot >= 0 and a.topk_weights != nullptr) ? a.topk_weights[my_slot] : 0.f;
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (single_copy) {
                if (not ptx::mbarrier_wait(&mbar[stage_idx], num_loads[stage_idx] & 1)) failed = true;
                ++num_loads[stage_idx];
                if (__any_sync(0xffffffffu, failed)) {
                    if (lane == 0) dev::report_status(cs, hs, kStatusMbarrierTimeout, rank, s, kSiteLoad, row, 0);
                    break;
                }
            }
            if (lane == 0) {
                const int group = num_ranks >= k ? master : rank;
                dev::store_message(cs, hs, a.peers, s, a.buffer_offset, a.buffer_bytes, bl.offset(group, token), stage, token_bytes, kSitePush);
            }
            ptx::bulk_commit();
        }
    }

    // completion: all stores performed, then one flag per destination from the last CTA
    if (tracer) dev::trace_point(a.trace, kTrCombPushed);
    ptx::bulk_wait<0>();
    ptx::fence_proxy_async();
    __threadfence_system();
    __syncthreads();
    if (tracer) dev::trace_point(a.trace, kTrCombStoresDone);
    if (warp == 0) {
        unsigned last = 0;
        if (lane == 0) {
            last = atomicAdd(&cs->done_ctas, 1u) == unsigned(num_ctas - 1);
            if (last) cs->done_ctas = 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            __threadfence_system();
            for (int r = lane; r < num_ranks; r += 32)
                ptx::st_release_sys(a.peers.sym(&a.ws->combine_done[rank], r), static_cast<unsigned long long>(epoch));
            if (lane == 0) a.ws->combine_epoch = epoch;
            if (a.wait_arrival) {
                const dev::Deadline deadline(a.timeout_ns);
                for (int s = lane; s < num_ranks; s += 32) {
                    unsigned long long w = 0;
                    if (not dev::spin_until(deadline, [&]() { return (w = ptx::ld_acquire_sys(&a.ws->combine_done[s])) == epoch; }))
                        dev::report_status(cs, hs, kStatusArrivalTimeout, rank, s, kSiteArrival, epoch, w);
                }
            }
            __syncwarp();
            if (lane == 0) dev::trace_point(a.trace, kTrCombEnd);       // the CTA that finished last
        }
    }
}

__global__ void __launch_bounds__(32 * 8, 1) ep_combine_kernel(const __grid_constant__ CombineArgs a) {
    ep_combine_body<0, 0, 0>(a);
}

// Kernel body; non-zero template arguments replace the corresponding run-time shape values by compile-time constants
// (see `ep_dispatch_body`): zeros for the ahead-of-time kernel below, the shapes in use for run-time specialised kernels.
template <int kNumRanks, int kNumTopk, int kHiddenBytes, int kNumExperts, bool kFewRows>
EP_DEVICE void ep_combine_reduce_body(const CombineReduceArgs& a) {
    using namespace combine_detail;
    const int num_ranks = kNumRanks > 0 ? kNumRanks : a.num_ranks;
    const int num_experts = kNumExperts > 0 ? kNumExperts : a.num_experts;
    const int hidden_bytes = kHiddenBytes > 0 ? kHiddenBytes : a.hidden_bytes;
    const int num_local_experts = num_experts / num_ranks;
    const int warps_per_cta = blockDim.x / 32;
    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    const int k = kNumTopk > 0 ? kNumTopk : a.num_topk;
    layout::CommonSignals* cs = &a.ws->common;
    layout::HostStatus* hs = a.host ? &a.host->status : nullptr;
    const layout::CombineTokenLayout tl(hidden_bytes, k);
    const int token_bytes = tl.num_bytes();
    const layout::BufferLayout bl(token_bytes, min(k, num_ranks), a.num_max_tokens);

    if (not dev::healthy(cs)) return;
    const unsigned epoch = a.ws->combine_epoch;
    const bool tracer = blockIdx.x == 0 and threadIdx.x == 0;
    if (tracer) dev::trace_point(a.trace, kTrRedStart);
    if (a.wait_arrival and warp == 0) {
        const dev::Deadline deadline(a.timeout_ns);
        for (int s = lane; s < num_ranks; s += 32) {
            unsigned long long w = 0;
            if (not dev::spin_until(deadline, [&]() { return (w = ptx::ld_acquire_sys(&a.ws->combine_done[s])) == epoch; }))
                dev::report_status(cs, hs, kStatusArrivalTimeout, a.rank, s, kSiteArrival, epoch, w);
        }
    }
    __syncthreads();
    if (not dev::healthy(cs)) return;
    if (tracer) dev::trace_point(a.trace, kTrRedArrived);

    const int chunks = hidden_bytes / 16;
    // With `coop` and fewer tokens than warps, P consecutive warps share a token (1 / P of the chunks each).
    const int total_warps = gridDim.x * warps_per_cta;
    int P = 1;
    if (a.coop)
        while (P < 8 and int64_t(a.num_tokens) * (2 * P) <= total_warps) P *= 2;
    for (int unit = blockIdx.x * warps_per_cta + warp; unit < a.num_tokens * P; unit += total_warps) {
        const int t = unit / P, part_idx = unit % P;
        const int c_begin = chunks * part_idx / P, c_end = chunks * (part_idx + 1) / P;
        // lane j owns top-k position j
        int r = -1;
        if (lane < k) {
            const int64_t e = a.topk_idx[int64_t(t) * k + lane];
            if (e >= 0 and e < num_experts) r = int(e) / num_local_experts;
        }
        // master position of a rank = last top-k position that selects it
        bool is_master = r >= 0;
        for (int d = 1; d < k; ++d) {
            const int other = __shfl_down_sync(0xffffffffu, r, d);
            if (lane + d < k and other == r) is_master = false;
        }
        const int group = num_ranks >= k ? lane : r;
        const unsigned masters = __ballot_sync(0xffffffffu, is_master);
        const int count = __popc(masters);

        const uint8_t* b0 = a.bias_0 != nullptr ? a.bias_0 + int64_t(t) * hidden_bytes : nullptr;
        const uint8_t* b1 = a.bias_1 != nullptr ? a.bias_1 + int64_t(t) * hidden_bytes : nullptr;
        uint8_t* out = a.combined_x + int64_t(t) * hidden_bytes;
        // rows to add, in the order of the sum: bias_0, bias_1, then the partials in slot order
        const int num_bias = (b0 != nullptr) + (b1 != nullptr), total = num_bias + count;
        const uint8_t* part[kUnroll];
        unsigned left = masters;                // master positions not yet listed (the same in every lane)
        #pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (u < num_bias) {
                part[u] = (u == 0 and b0 != nullptr) ? b0 : b1;
            } else {
                const bool have = left != 0;
                const int g = __shfl_sync(0xffffffffu, group, have ? __ffs(left) - 1 : 0);
                left &= left - 1;
                part[u] = have ? a.buffer + bl.offset(g, t) : nullptr;
            }
        }
        // Register budget first: with one row per load round the kernel needs about 80 registers, so three CTAs (24 warps)
        // fit on an SM and the rows of a token (3 to 6 at eight ranks) are in flight together in each of them. When a
        // token can have at most two partials (`kFewRows`: one or two ranks, or top-1/top-2 routing) that would leave one or
        // two loads per lane, so that variant fetches four chunks of each row per round instead (128 registers, 16 warps).
        if (kFewRows and total <= 2) {
            const uint8_t* p2[2] = {part[0], part[1]};
            reduce_token<2, 4>(p2, out, c_begin, c_end, lane);
        } else if (total <= kUnroll) {
            reduce_token<kUnroll, 1>(part, out, c_begin, c_end, lane);
        } else {
            for (int base = c_begin; base < c_end; base += 32) {      // warp-uniform trip count: shuffles inside
                const int c = base + lane;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (c < c_end and b0 != nullptr) accumulate(acc, ptx::ld_nc_v4(b0 + c * 16));
                if (c < c_end and b1 != nullptr) accumulate(acc, ptx::ld_nc_v4(b1 + c * 16));
                for (int u = 0; u < count; ++u) {
                    const int g = __shfl_sync(0xffffffffu, group, nth_set_bit(masters, u));
                    if (c < c_end) accumulate(acc, ptx::ld_v4(a.buffer + bl.offset(g, t) + c * 16));
                }
                if (c < c_end) ptx::st_na_v4(out + c * 16, pack(acc));
            }
        }
        if (a.combined_topk_weights != nullptr and part_idx == 0) {
            // position j reads its weight from the partial produced by the rank that owns expert j
            int master_group = -1;
            for (int j = 0; j < k; ++j) {
                const int rj = __shfl_sync(0xffffffffu, r, j);
                const int gj = __shfl_sync(0xffffffffu, group, j);
                if ((masters >> j) & 1 and rj == r) master_group = gj;
            }
            if (lane < k) {
                float w = 0.f;
                if (r >= 0 and master_group >= 0)
                    w = *reinterpret_cast<const float*>(a.buffer + bl.offset(master_group, t) + tl.weight_offset() + 4 * lane);
                a.combined_topk_weights[int64_t(t) * k + lane] = w;
            }
        }
    }
    // CTA 0's share is done (the other CTAs work on as many tokens each, give or take one)
    __syncthreads();
    if (tracer) dev::trace_point(a.trace, kTrRedEnd);
}

__global__ void __launch_bounds__(32 * 8, 3) ep_combine_reduce_kernel(const __grid_constant__ CombineReduceArgs a) {
    ep_combine_reduce_body<0, 0, 0, 0, false>(a);
}

// Variant for tokens with at most two partials (min(top-k, ranks) <= 2), see the note on the register budget above.
__global__ void __launch_bounds__(32 * 8, 2) ep_combine_reduce_few_rows_kernel(const __grid_constant__ CombineReduceArgs a) {
    ep_combine_reduce_body<0, 0, 0, 0, true>(a);
}

}  // namespace deep_ep::kernels
