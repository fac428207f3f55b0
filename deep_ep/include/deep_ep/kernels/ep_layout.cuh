// Standalone routing-layout kernel: the count/assign passes of the dispatch kernel without any
// communication. For every token it computes the slot it will occupy in each destination rank's
// per-source receive region (token order, one slot per destination rank, stored at the last top-k position
// that selects the rank), plus the per-rank and per-expert send counts. Useful to plan buffers, to inspect
// load balance, and as the sender half of the handle semantics (`EPHandle.dst_buffer_slot_idx`).
// Role of the routing scan in the reference's `impls/ep/dispatch.hpp:167-292`.
#pragma once

#include "../device/sync.cuh"
#include "ep_layout_args.hpp"

namespace deep_ep::kernels {

// Body of the kernel; each translation unit that launches it wraps it in its own `__global__` function
// (256 threads per CTA, cooperative launch, at most `kLayoutMaxCtas` CTAs).
EP_DEVICE void ep_layout_body(const LayoutArgs& a) {
    __shared__ int warp_rank[8][kMaxRanks];
    __shared__ unsigned hit_all[8][kMaxRanks];
    __shared__ int expert_hist[kMaxExperts];

    const int num_local_experts = a.num_experts / a.num_ranks;
    const int num_ctas = gridDim.x, cta = blockIdx.x;
    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    constexpr int W = 8;
    const int k = a.num_topk;
    layout::CommonSignals* cs = &a.scratch->sync;

    for (int i = threadIdx.x; i < a.num_experts; i += blockDim.x) expert_hist[i] = 0;
    for (int i = threadIdx.x; i < W * kMaxRanks; i += blockDim.x) (&warp_rank[0][0])[i] = 0, (&hit_all[0][0])[i] = 0;
    __syncthreads();

    const int per_cta = math::ceil_div(a.num_tokens, num_ctas);
    const int cta_begin = min(cta * per_cta, a.num_tokens), cta_end = min(cta_begin + per_cta, a.num_tokens);
    const int per_warp = math::ceil_div(cta_end - cta_begin, W);
    const int warp_begin = min(cta_begin + warp * per_warp, cta_end), warp_end = min(warp_begin + per_warp, cta_end);
    unsigned* hit = hit_all[warp];
    int* run = warp_rank[warp];

    // pass 1: counts
    for (int g = warp_begin; g < warp_end; g += 32) {
        const int t = g + lane;
        if (t < warp_end) {
            for (int j = 0; j < k; ++j) {
                const int64_t e = a.topk_idx[int64_t(t) * k + j];
                if (e >= 0 and e < a.num_experts) {
                    atomicOr(&hit[int(e) / num_local_experts], 1u << lane);
                    atomicAdd(&expert_hist[e], 1);
                }
            }
        }
        __syncwarp();
        for (int r = lane; r < a.num_ranks; r += 32) run[r] += __popc(hit[r]), hit[r] = 0;
        __syncwarp();
    }
    __syncthreads();
    for (int r = threadIdx.x; r < a.num_ranks; r += blockDim.x) {
        int total = 0;
        for (int w = 0; w < W; ++w) total += warp_rank[w][r];
        a.scratch->cta_rank_count[cta][r] = total;
    }
    for (int e = threadIdx.x; e < a.num_experts; e += blockDim.x)
        if (expert_hist[e] != 0) atomicAdd(&a.scratch->expert_count[e], expert_hist[e]);

    const bool ok = dev::grid_sync(cs, nullptr, num_ctas, a.timeout_ns, 0, /*where=*/60);
    if (not ok) {
        if (threadIdx.x == 0 and a.status != nullptr) *a.status = kStatusGridSyncTimeout;
        if (threadIdx.x == 0) cs->status = 0;       // standalone kernel: the failure is reported, not sticky
        return;
    }

    // totals (CTA 0); the expert histogram is cleared for the next launch
    if (cta == 0) {
        for (int r = threadIdx.x; r < a.num_ranks; r += blockDim.x) {
            int total = 0;
            for (int c = 0; c < num_ctas; ++c) total += __ldcg(&a.scratch->cta_rank_count[c][r]);
            a.num_tokens_per_rank[r] = total;
        }
        for (int e = threadIdx.x; e < a.num_experts; e += blockDim.x) {
            a.num_tokens_per_expert[e] = __ldcg(&a.scratch->expert_count[e]);
            a.scratch->expert_count[e] = 0;
        }
    }

    // pass 2: slots in token order
    for (int r = threadIdx.x; r < a.num_ranks; r += blockDim.x) {
        int base = 0;
        for (int c = 0; c < cta; ++c) base += __ldcg(&a.scratch->cta_rank_count[c][r]);
        for (int w = 0; w < W; ++w) {
            const int cnt = warp_rank[w][r];
            warp_rank[w][r] = base, base += cnt;
        }
    }
    __syncthreads();
    for (int g = warp_begin; g < warp_end; g += 32) {
        const int t = g + lane;
        if (t < warp_end) {
            for (int j = 0; j < k; ++j) {
                const int64_t e = a.topk_idx[int64_t(t) * k + j];
                if (e >= 0 and e < a.num_experts) atomicOr(&hit[int(e) / num_local_experts], 1u << lane);
            }
        }
        __syncwarp();
        if (t < warp_end) {
            unsigned long long seen = 0;
            for (int j = k - 1; j >= 0; --j) {
                const int64_t e = a.topk_idx[int64_t(t) * k + j];
                int slot = -1;
                if (e >= 0 and e < a.num_experts) {
                    const int r = int(e) / num_local_experts;
                    if (not((seen >> r) & 1)) slot = run[r] + __popc(hit[r] & ptx::lanemask_lt());
                    seen |= 1ull << r;
                }
                a.dst_slot_idx[int64_t(t) * k + j] = slot;
            }
        }
        __syncwarp();
        for (int r = lane; r < a.num_ranks; r += 32) run[r] += __popc(hit[r]), hit[r] = 0;
        __syncwarp();
    }
}

}  // namespace deep_ep::kernels
