// Dispatch epilogue for sm_100a: waits for every source rank's "push finished" flag, then turns the
// per-source receive regions into the expert-major *expanded* layout. Each received message is
// loaded once into shared memory with a bulk copy and stored once per local expert it selected;
// rows of an expert appear in (source rank, source token) order, so the layout is deterministic.
// Role of the reference's `impls/ep/dispatch_copy_epilogue.hpp:176-621`.
#pragma once

#include "../device/sync.cuh"
#include "ep_args.hpp"
#include "ep_dispatch.cuh"      // `dispatch_detail::wait_read_pending`

namespace deep_ep::kernels {


namespace expand_detail {

constexpr int kSiteArrival = 20, kSiteGridSync = 21, kSiteLoad = 22;


// Position i of the compact receive stream -> (source rank, slot inside that source's region).
EP_DEVICE void locate(const int* psum_rank_smem, int num_ranks, int i, int& src, int& slot) {
    int s = 0;
    while (s < num_ranks - 1 and i >= psum_rank_smem[s]) ++s;
    src = s, slot = i - (s == 0 ? 0 : psum_rank_smem[s - 1]);
}

}  // namespace expand_detail

// Kernel body; non-zero template arguments replace the corresponding run-time shape values by compile-time constants
// (see `ep_dispatch_body`): zeros for the ahead-of-time kernel below, the shapes in use for run-time specialised kernels.
template <int kNumRanks, int kNumTopk, int kHiddenBytes, int kNumExperts>
EP_DEVICE void ep_dispatch_expand_body(const ExpandArgs& a) {
    using namespace expand_detail;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int psum_rank_smem[kMaxRanks];

    const int num_ranks = kNumRanks > 0 ? kNumRanks : a.num_ranks;
    const int num_experts = kNumExperts > 0 ? kNumExperts : a.num_experts;
    const int hidden_bytes = kHiddenBytes > 0 ? kHiddenBytes : a.hidden_bytes;
    const int num_local_experts = num_experts / num_ranks;
    const int expert_begin = a.rank * num_local_experts;
    const int num_ctas = gridDim.x, cta = blockIdx.x;
    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    const int W = a.num_warps, S = a.num_stages, k = kNumTopk > 0 ? kNumTopk : a.num_topk;
    layout::CommonSignals* cs = &a.ws->common;
    layout::HostStatus* hs = a.host ? &a.host->status : nullptr;
    const layout::DispatchTokenLayout tl(hidden_bytes, a.sf_bytes, k);
    const int token_bytes = tl.num_bytes();
    const layout::BufferLayout bl(token_bytes, num_ranks, a.num_max_tokens);

    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t* p = base;
    uint64_t* mbar_all = reinterpret_cast<uint64_t*>(p);
    p += int64_t(W) * S * 8;
    int* run_all = reinterpret_cast<int*>(p);
    p += int64_t(W) * num_local_experts * 4;
    unsigned* hit_all = reinterpret_cast<unsigned*>(p);
    p += int64_t(W) * num_local_experts * 4;
    int* slots_all = reinterpret_cast<int*>(p);
    p += int64_t(W) * 32 * (k + 1) * 4;
    int* psum_sm = reinterpret_cast<int*>(p);          // end of every local expert's rows
    p += int64_t(num_local_experts) * 4;
    int* base_sm = reinterpret_cast<int*>(p);          // first row this CTA writes for every local expert
    p += int64_t(num_local_experts) * 4;
    p = base + math::align<int64_t>(p - base, 128);
    uint8_t* stages_all = p;

    if (not dev::healthy(cs)) return;
    const unsigned epoch = a.ws->dispatch_epoch;
    const bool tracer = cta == 0 and threadIdx.x == 0;
    if (tracer) dev::trace_point(a.trace, kTrExpStart);

    if (threadIdx.x == 0) {
        for (int i = 0; i < W * S; ++i) ptx::mbarrier_init(&mbar_all[i], 1);
        ptx::fence_mbarrier_init();
    }
    for (int i = threadIdx.x; i < W * num_local_experts; i += blockDim.x) run_all[i] = 0, hit_all[i] = 0;

    // ---- wait until every source rank has finished pushing to this rank
    if (a.wait_arrival and warp == 0) {
        const dev::Deadline deadline(a.timeout_ns);
        for (int s = lane; s < num_ranks; s += 32) {
            unsigned long long w = 0;
            if (not dev::spin_until(deadline, [&]() { return (w = ptx::ld_acquire_sys(&a.ws->dispatch_done[s])) == epoch; }))
                dev::report_status(cs, hs, kStatusArrivalTimeout, a.rank, s, kSiteArrival, epoch, w);
        }
    }
    for (int s = threadIdx.x; s < num_ranks; s += blockDim.x) psum_rank_smem[s] = a.psum_rank[s];
    for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x) psum_sm[e] = a.psum_expert[e];
    __syncthreads();
    if (not dev::healthy(cs)) return;
    if (tracer) dev::trace_point(a.trace, kTrExpArrived);

    const int num_recv = min(psum_rank_smem[num_ranks - 1], a.num_metadata_rows);
    const int per_cta = math::ceil_div(num_recv, num_ctas);
    const int cta_begin = min(cta * per_cta, num_recv), cta_end = min(cta_begin + per_cta, num_recv);
    const int per_warp = math::ceil_div(cta_end - cta_begin, W);
    const int warp_begin = min(cta_begin + warp * per_warp, cta_end), warp_end = min(warp_begin + per_warp, cta_end);

    int* run = run_all + warp * num_local_experts;
    unsigned* hit = hit_all + warp * num_local_experts;
    int* slots = slots_all + warp * 32 * (k + 1);

    // ------------------------------------------------------------------ pass 1: per-expert histogram
    if (not a.cached) {
        for (int g = warp_begin; g < warp_end; g += 32) {
            const int i = g + lane;
            if (i < warp_end) {
                int src, slot;
                locate(psum_rank_smem, num_ranks, i, src, slot);
                const int* idx = reinterpret_cast<const int*>(a.buffer + bl.offset(src, slot) + tl.idx_offset());
                for (int j = 0; j < k; ++j) {
                    const int e = idx[j] - expert_begin;
                    if (e >= 0 and e < num_local_experts and idx[j] >= 0) atomicAdd(&run[e], 1);
                }
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x) {
            int total = 0;
            for (int w = 0; w < W; ++w) total += run_all[w * num_local_experts + e];
            a.ws->cta_expert_count[cta][e] = total;
        }
        if (not dev::grid_sync(cs, hs, num_ctas, a.timeout_ns, a.rank, kSiteGridSync)) return;
        if (tracer) dev::trace_point(a.trace, kTrExpLaidOut);
        // rows written by earlier CTAs: one warp per expert, lanes split the CTAs so that the loads overlap
        for (int e = warp; e < num_local_experts; e += W) {
            int partial = 0;
            for (int c = lane; c < cta; c += 32) partial += __ldcg(&a.ws->cta_expert_count[c][e]);
            #pragma unroll
            for (int o = 16; o >= 1; o >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, o);
            // aligned start of the expert's region (previous expert's end, rounded up) + rows of earlier CTAs
            if (lane == 0) base_sm[e] = (e == 0 ? 0 : math::align(psum_sm[e - 1], a.expert_alignment)) + partial;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x) {
            int b = base_sm[e];
            for (int w = 0; w < W; ++w) {
                const int cnt = run_all[w * num_local_experts + e];
                run_all[w * num_local_experts + e] = b, b += cnt;
            }
        }
        __syncthreads();
    }

    // ------------------------------------------------------------------ pass 2: assign rows and copy
    uint64_t* mbar = mbar_all + warp * S;
    uint8_t* stages = stages_all + int64_t(warp) * S * token_bytes;
    const int meta_cols = k + 2;
    bool failed = false;

    auto issue_load = [&](int n, int src, int slot) {    // lane 0
        ptx::mbarrier_arrive_expect_tx(&mbar[n % S], token_bytes);
        ptx::bulk_load(stages + (n % S) * token_bytes, a.buffer + bl.offset(src, slot), token_bytes, &mbar[n % S]);
    };

    // S - 1 message loads are in flight while the oldest message is being copied out: message n + D reuses the stage of
    // message n + D - S, whose stores must have read it (at most S - D - 1 = 0 committed groups may still be reading).
    const int D = S - 1;
    if (lane == 0)
        for (int i = warp_begin; i < min(warp_begin + D, warp_end); ++i) {
            int src, slot;
            locate(psum_rank_smem, num_ranks, i, src, slot);
            issue_load(i - warp_begin, src, slot);
        }

    for (int i = warp_begin; i < warp_end; ++i) {
        const int n = i - warp_begin, tl_idx = n & 31;
        if (tl_idx == 0) {
            const int row = i + lane;
            int src = 0, slot = 0;
            const int* idx = nullptr;
            if (row < warp_end) {
                locate(psum_rank_smem, num_ranks, row, src, slot);
                idx = reinterpret_cast<const int*>(a.buffer + bl.offset(src, slot) + tl.idx_offset());
            }
            if (a.cached) {
                if (row < warp_end)
                    for (int j = 0; j < k; ++j) slots[lane * (k + 1) + j] = a.recv_src_metadata[int64_t(row) * meta_cols + j];
            } else {
                if (row < warp_end) {
                    for (int j = 0; j < k; ++j) {
                        const int e = idx[j] - expert_begin;
                        if (idx[j] >= 0 and e >= 0 and e < num_local_experts) atomicOr(&hit[e], 1u << lane);
                    }
                }
                __syncwarp();
                if (row < warp_end) {
                    int master = -1;
                    for (int j = 0; j < k; ++j) {
                        const int e = idx[j] - expert_begin;
                        int out = -1;
                        if (idx[j] >= 0 and e >= 0 and e < num_local_experts) {
                            out = run[e] + __popc(hit[e] & ptx::lanemask_lt());
                            if (out >= a.num_expanded_rows) out = -1;
                            master = j;
                        }
                        slots[lane * (k + 1) + j] = out;
                        a.recv_src_metadata[int64_t(row) * meta_cols + j] = out;
                    }
                    a.recv_src_metadata[int64_t(row) * meta_cols + k] =
                        *reinterpret_cast<const int*>(a.buffer + bl.offset(src, slot) + tl.src_offset());
                    a.recv_src_metadata[int64_t(row) * meta_cols + k + 1] = master;
                }
                __syncwarp();
                if (row < warp_end) {
                    // every (token, expert) pair is unique, so each lane retires its own hits
                    for (int j = 0; j < k; ++j) {
                        const int e = idx[j] - expert_begin;
                        if (idx[j] >= 0 and e >= 0 and e < num_local_experts) {
                            const unsigned h = hit[e];
                            if ((h & ptx::lanemask_lt()) == 0) run[e] += __popc(h);   // lowest lane of the group updates
                        }
                    }
                }
                __syncwarp();
                if (row < warp_end)
                    for (int j = 0; j < k; ++j) {
                        const int e = idx[j] - expert_begin;
                        if (idx[j] >= 0 and e >= 0 and e < num_local_experts) hit[e] = 0;
                    }
            }
            __syncwarp();
        }

        // prefetch the next message
        if (i + D < warp_end) {
            dispatch_detail::wait_read_pending(S - D - 1);
            __syncwarp();
            if (lane == 0) {
                int src, slot;
                locate(psum_rank_smem, num_ranks, i + D, src, slot);
                issue_load(n + D, src, slot);
            }
        }

        uint8_t* stage = stages + (n % S) * token_bytes;
        if (not ptx::mbarrier_wait(&mbar[n % S], (n / S) & 1)) failed = true;
        if (__any_sync(0xffffffffu, failed)) {
            if (lane == 0) dev::report_status(cs, hs, kStatusMbarrierTimeout, a.rank, -1, kSiteLoad, i, 0);
            break;
        }

        // hidden row: one bulk store per expanded slot (lane j owns top-k position j)
        const int my_out = lane < k ? slots[tl_idx * (k + 1) + lane] : -1;
        if (my_out >= 0) {
            ptx::bulk_store(a.recv_x + int64_t(my_out) * hidden_bytes, stage, hidden_bytes);
            if (a.recv_topk_weights != nullptr)
                a.recv_topk_weights[my_out] = reinterpret_cast<const float*>(stage + tl.weight_offset())[lane];
        }
        // scale factors of a row-major destination: each row's packs are contiguous, one more bulk store per copy
        const bool sf_rows_bulk = a.recv_sf != nullptr and a.recv_sf_pack_stride == 1 and a.sf_bytes % 16 == 0 and
                                  (a.recv_sf_token_stride * 2) % 16 == 0;
        if (sf_rows_bulk and my_out >= 0)
            ptx::bulk_store(a.recv_sf + int64_t(my_out) * a.recv_sf_token_stride, stage + tl.sf_offset(), a.sf_bytes);
        ptx::bulk_commit();
        // otherwise: strided 2-byte packs (column-major destination, or rows that are no multiple of 16 bytes)
        if (a.recv_sf != nullptr and not sf_rows_bulk) {
            const unsigned valid = __ballot_sync(0xffffffffu, my_out >= 0);
            const sf_pack_t* src_sf = reinterpret_cast<const sf_pack_t*>(stage + tl.sf_offset());
            for (unsigned m = valid; m != 0; m &= m - 1) {
                const int out = __shfl_sync(0xffffffffu, my_out, __ffs(m) - 1);
                for (int q = lane; q < a.sf_bytes / 2; q += 32)
                    a.recv_sf[int64_t(out) * a.recv_sf_token_stride + int64_t(q) * a.recv_sf_pack_stride] = src_sf[q];
            }
        }
    }
    ptx::bulk_wait<0>();

    // ------------------------------------------------------------------ zero the alignment padding
    if (a.do_zero_padding and a.expert_alignment > 1) {
        const int gw = cta * W + warp, num_gw = num_ctas * W;
        const int4 zero = make_int4(0, 0, 0, 0);
        for (int e = 0; e < num_local_experts; ++e) {
            const int end = psum_sm[e];
            const int pad_end = min(math::align(end, a.expert_alignment), a.num_expanded_rows);
            for (int row = end + gw; row < pad_end; row += num_gw) {
                for (int c = lane; c < hidden_bytes / 16; c += 32)
                    ptx::st_na_v4(a.recv_x + int64_t(row) * hidden_bytes + c * 16, zero);
                if (a.recv_sf != nullptr)
                    for (int q = lane; q < a.sf_bytes / 2; q += 32)
                        a.recv_sf[int64_t(row) * a.recv_sf_token_stride + int64_t(q) * a.recv_sf_pack_stride] = 0;
                if (a.recv_topk_weights != nullptr and lane == 0) a.recv_topk_weights[row] = 0.f;
            }
        }
    }
    // CTA 0's share is done (every CTA copies the same number of messages, give or take one)
    __syncthreads();
    if (tracer) dev::trace_point(a.trace, kTrExpEnd);
}

__global__ void __launch_bounds__(32 * 8, 1) ep_dispatch_expand_kernel(const __grid_constant__ ExpandArgs a) {
    ep_dispatch_expand_body<0, 0, 0, 0>(a);
}

}  // namespace deep_ep::kernels
