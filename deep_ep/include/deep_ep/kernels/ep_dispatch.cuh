// Expert-parallel dispatch for sm_100a: one persistent, cooperatively launched kernel that
//   (1) computes the routing layout (per-rank de-duplicated slots in token order, per-expert
//       histogram) with a two-pass count/assign scheme, so the result is deterministic,
//   (2) exchanges counts with every peer through epoch-tagged words in peer memory,
//   (3) optionally quantises BF16 rows to e4m3 with one fp32 scale per 128 columns, and
//   (4) pushes every token once per destination rank as ONE contiguous message with a
//       `cp.async.bulk` store from shared memory straight into the peer's receive region.
// It plays the role of the reference's `impls/ep/dispatch.hpp:75-863` (routing scan, count exchange,
// metadata packing, URMA payload push); the transport and the pipeline are NVLink/TMA specific.
#pragma once

#include "../device/sync.cuh"
#include "ep_args.hpp"

namespace deep_ep::kernels {


namespace dispatch_detail {

constexpr int kSiteEntryBarrier = 10, kSiteGridSync1 = 11, kSiteRankCount = 12, kSiteExpertCount = 13,
              kSiteLoad = 14, kSiteArrival = 15, kSitePush = 16;

struct Smem {
    uint64_t* mbar;          // [W][S + 2]  (S message stages + 2 quantiser source stages)
    int* warp_rank;          // [W][kMaxRanks]  pass-1 counts, then running slot bases
    unsigned* hit;           // [W][kMaxRanks]  per-group token bitmaps
    int* expert_hist;        // [num_experts]
    int* slots;              // [W][32][k]
    uint8_t* stages;         // [W][S][token_bytes]
    uint8_t* src_stages;     // [W][2][src_row_bytes]   (fused quantisation only)
};


EP_DEVICE Smem carve(uint8_t* base, const DispatchArgs& a, int token_bytes, int src_row_bytes) {
    Smem s;
    base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(base) + 127) & ~uintptr_t(127));
    uint8_t* p = base;
    s.mbar = reinterpret_cast<uint64_t*>(p), p += int64_t(a.num_warps) * (a.num_stages + 2) * 8;
    s.warp_rank = reinterpret_cast<int*>(p), p += int64_t(a.num_warps) * kMaxRanks * 4;
    s.hit = reinterpret_cast<unsigned*>(p), p += int64_t(a.num_warps) * kMaxRanks * 4;
    s.expert_hist = reinterpret_cast<int*>(p), p += int64_t(a.num_experts) * 4;
    s.slots = reinterpret_cast<int*>(p), p += int64_t(a.num_warps) * 32 * a.num_topk * 4;
    p = base + math::align<int64_t>(p - base, 128);
    s.stages = p, p += int64_t(a.num_warps) * a.num_stages * token_bytes;
    p = base + math::align<int64_t>(p - base, 128);
    s.src_stages = p;
    return s;
}

// Token range of this CTA and of one pusher warp inside it (contiguous, in token order).
EP_DEVICE void token_range(int num_tokens, int num_parts, int part, int& begin, int& end) {
    const int per = math::ceil_div(num_tokens, num_parts);
    begin = min(part * per, num_tokens), end = min(begin + per, num_tokens);
}

template <int N>
EP_DEVICE void wait_read_le() { ptx::bulk_wait_read<N>(); }

EP_DEVICE void wait_read_pending(int n) {
    // `n` most recent groups may still be reading shared memory
    switch (n) {
        case 0: ptx::bulk_wait_read<0>(); break;
        case 1: ptx::bulk_wait_read<1>(); break;
        case 2: ptx::bulk_wait_read<2>(); break;
        default: ptx::bulk_wait_read<3>(); break;
    }
}

// Quantise one BF16 row held in shared memory into e4m3 + fp32 scales in the message stage.
// Bit-compatible with `x * (448 * (1 / max(amax, 1e-4)))` rounded to e4m3 and `scale = amax * (1/448)`.
// With `pow2` the scale is rounded up to a power of two (`2^ceil(log2(amax / 448))`, still sent as fp32), the form
// the tensor core can apply itself as a UE8M0 block scale.
EP_DEVICE void quantize_row(const uint8_t* src, uint8_t* dst_fp8, float* dst_sf, int hidden, int lane, bool pow2) {
    const int num_iters = math::ceil_div(hidden, 256);
    for (int it = 0; it < num_iters; ++it) {
        const int col = it * 256 + lane * 8;
        const bool active = col < hidden;
        int4 raw = make_int4(0, 0, 0, 0);
        if (active) raw = *reinterpret_cast<const int4*>(src + col * 2);
        float v[8];
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
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
        float inv = __fmul_rn(__frcp_rn(amax), 448.0f), sf = __fmul_rn(amax, 1.0f / 448.0f);
        if (pow2) {
            uint32_t byte;
            ptx::ue8m0_ceil(sf, byte, inv);
            sf = __uint_as_float(byte << 23);
        }
        if (active) {
            uint2 packed;
            packed.x = ptx::float2_to_e4m3x2(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv)) |
                       (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[2], inv), __fmul_rn(v[3], inv))) << 16);
            packed.y = ptx::float2_to_e4m3x2(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv)) |
                       (uint32_t(ptx::float2_to_e4m3x2(__fmul_rn(v[6], inv), __fmul_rn(v[7], inv))) << 16);
            *reinterpret_cast<uint2*>(dst_fp8 + col) = packed;
            if ((lane & 15) == 0) dst_sf[col / 128] = sf;
        }
    }
}

}  // namespace dispatch_detail

// Kernel body. Non-zero template arguments replace the corresponding run-time values (`a.peers.num_ranks`, `a.num_topk`,
// `a.hidden_bytes`, `a.num_experts`) by compile-time constants: the ahead-of-time kernel below passes zeros, kernels
// specialised at run time for the shapes in use (`csrc/runtime/specialize.hpp`) pass the shapes, which unrolls the top-k
// and per-rank loops and folds the message layout into constants (the reference instantiates its kernels the same way,
// `csrc/kernels/ep/dispatch.hpp:52-81`). The host guarantees that the arguments match the constants.
template <int kNumRanks, int kNumTopk, int kHiddenBytes, int kNumExperts>
EP_DEVICE void ep_dispatch_body(const DispatchArgs& a) {
    using namespace dispatch_detail;
    extern __shared__ uint8_t smem_raw[];

    const int num_ranks = kNumRanks > 0 ? kNumRanks : a.peers.num_ranks, rank = a.peers.rank;
    const int num_experts = kNumExperts > 0 ? kNumExperts : a.num_experts;
    const int num_local_experts = num_experts / num_ranks;
    const int num_ctas = gridDim.x, cta = blockIdx.x;
    const int warp = threadIdx.x / 32, lane = ptx::lane_id();
    const int W = a.num_warps, S = a.num_stages, k = kNumTopk > 0 ? kNumTopk : a.num_topk;
    const int hidden_bytes = kHiddenBytes > 0 ? kHiddenBytes : a.hidden_bytes;
    const bool is_aux = warp == W;
    const int num_pushers = W * 32;
    layout::CommonSignals* cs = &a.ws->common;
    layout::HostStatus* hs = a.host ? &a.host->status : nullptr;

    const layout::DispatchTokenLayout tl(hidden_bytes, a.sf_bytes, k);
    const int token_bytes = tl.num_bytes();
    const int hidden = a.fused_quant ? hidden_bytes : 0;               // fp8 elements when quantising
    const int src_row_bytes = a.fused_quant ? hidden_bytes * 2 : 0;
    const Smem sm = carve(smem_raw, a, token_bytes, src_row_bytes);

    if (not dev::healthy(cs)) return;
    const unsigned epoch = a.ws->dispatch_epoch + 1;
    const bool tracer = cta == 0 and threadIdx.x == 0;
    if (tracer) dev::trace_point(a.trace, kTrDispStart);

    if (threadIdx.x == 0) {
        for (int i = 0; i < W * (S + 2); ++i) ptx::mbarrier_init(&sm.mbar[i], 1);
        ptx::fence_mbarrier_init();
    }
    for (int i = threadIdx.x; i < num_experts; i += blockDim.x) sm.expert_hist[i] = 0;
    for (int i = threadIdx.x; i < W * kMaxRanks; i += blockDim.x) sm.warp_rank[i] = 0, sm.hit[i] = 0;
    __syncthreads();

    int cta_begin, cta_end, warp_begin = 0, warp_end = 0;
    token_range(a.num_tokens, num_ctas, cta, cta_begin, cta_end);
    if (not is_aux) {
        int b, e;
        token_range(cta_end - cta_begin, W, warp, b, e);
        warp_begin = cta_begin + b, warp_end = cta_begin + e;
    }
    unsigned* hit = sm.hit + warp * kMaxRanks;       // (aux warp never touches these)
    int* run = sm.warp_rank + warp * kMaxRanks;

    // ------------------------------------------------------------------ pass 1: count
    if (not a.cached and not is_aux) {
        for (int g = warp_begin; g < warp_end; g += 32) {
            const int t = g + lane;
            if (t < warp_end) {
                for (int j = 0; j < k; ++j) {
                    const int64_t e = a.topk_idx[int64_t(t) * k + j];
                    if (e >= 0 and e < num_experts) {
                        atomicOr(&hit[int(e) / num_local_experts], 1u << lane);
                        atomicAdd(&sm.expert_hist[e], 1);
                    }
                }
            }
            __syncwarp();
            for (int r = lane; r < num_ranks; r += 32) run[r] += __popc(hit[r]), hit[r] = 0;
            __syncwarp();
        }
    }
    __syncthreads();
    if (not a.cached) {
        for (int r = threadIdx.x; r < num_ranks; r += blockDim.x) {
            int total = 0;
            for (int w = 0; w < W; ++w) total += sm.warp_rank[w * kMaxRanks + r];
            a.ws->cta_rank_count[cta][r] = total;
        }
        for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
            if (sm.expert_hist[e] != 0) atomicAdd(&a.ws->send_expert_count[e], sm.expert_hist[e]);
    }

    // ------------------------------------------------------------------ entry barrier + grid sync
    // Every rank has finished consuming the previous contents of the receive buffers once the
    // barrier completes; no remote write is issued before the grid sync below.
    if (tracer) dev::trace_point(a.trace, kTrDispCounted);
    if (cta == 0 and is_aux) {
        dev::rank_barrier_warp(cs, hs, a.peers, a.timeout_ns, kSiteEntryBarrier);
        if (lane == 0) dev::trace_point(a.trace, kTrDispEntryBarrier);
    }
    if (not dev::grid_sync(cs, hs, num_ctas, a.timeout_ns, rank, kSiteGridSync1)) return;
    if (tracer) dev::trace_point(a.trace, kTrDispGridSync);

    // ------------------------------------------------------------------ aux warp: count exchange
    if (is_aux) {
        if (cta != 0 or a.cached) return;
        // rank counts -> peers
        for (int r0 = 0; r0 < num_ranks; r0 += 32) {
            // per-rank totals over all CTAs: lanes split the CTAs of one rank at a time so that the loads overlap
            int total = 0;
            for (int rr = r0; rr < min(r0 + 32, num_ranks); ++rr) {
                int partial = 0;
                for (int c = lane; c < num_ctas; c += 32) partial += __ldcg(&a.ws->cta_rank_count[c][rr]);
                #pragma unroll
                for (int o = 16; o >= 1; o >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, o);
                if (rr - r0 == lane) total = partial;
            }
            const int r = r0 + lane;
            if (r >= num_ranks) continue;
            // count words validate themselves through their epoch tag: no ordering against other stores is needed
            ptx::st_relaxed_sys(&a.peers.sym(&a.ws->recv_rank_count[rank], r)[0], layout::pack_tagged(epoch, total));
        }
        // expert counts -> owners (and clean the local histogram for the next call)
        for (int e = lane; e < num_experts; e += 32) {
            const int v = __ldcg(&a.ws->send_expert_count[e]);
            a.ws->send_expert_count[e] = 0;
            ptx::st_relaxed_sys(a.peers.sym(&a.ws->recv_expert_count[rank][e % num_local_experts], e / num_local_experts),
                                layout::pack_tagged(epoch, v));
        }
        // wait for every source's rank count, inclusive prefix
        const dev::Deadline deadline(a.timeout_ns);
        int carry = 0;
        bool ok = true;
        for (int base = 0; base < num_ranks; base += 32) {
            const int s = base + lane;
            int c = 0;
            if (s < num_ranks) {
                unsigned long long w = 0;
                const bool got = dev::spin_until(deadline, [&]() {
                    w = ptx::ld_relaxed_sys(&a.ws->recv_rank_count[s]);
                    return layout::tagged_epoch(w) == epoch;
                });
                if (not got) dev::report_status(cs, hs, kStatusCountTimeout, rank, s, kSiteRankCount, epoch, layout::tagged_epoch(w));
                ok = ok and got;
                c = layout::tagged_value(w);
            }
            int incl = c;
            #pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            if (s < num_ranks) a.psum_rank[s] = carry + incl;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        const int num_recv_tokens = carry;
        // per local expert: sum over sources, aligned prefix
        int expanded = 0;
        for (int base = 0; base < num_local_experts; base += 32) {
            const int e = base + lane;
            int c = 0;
            if (e < num_local_experts) {
                for (int s = 0; s < num_ranks; ++s) {
                    unsigned long long w = 0;
                    const bool got = dev::spin_until(deadline, [&]() {
                        w = ptx::ld_relaxed_sys(&a.ws->recv_expert_count[s][e]);
                        return layout::tagged_epoch(w) == epoch;
                    });
                    if (not got) dev::report_status(cs, hs, kStatusCountTimeout, rank, s, kSiteExpertCount, epoch, layout::tagged_epoch(w));
                    ok = ok and got;
                    c += layout::tagged_value(w);
                }
            }
            const int aligned = math::align(c, a.expert_alignment);
            int incl = aligned;
            #pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            if (e < num_local_experts) {
                a.psum_expert[e] = expanded + incl - aligned + c;
                a.num_unaligned[e] = c;
                if (a.cumulative_stats != nullptr) a.cumulative_stats[e] += c;
                if (a.do_cpu_sync) a.host->aligned_recv_per_expert[e] = aligned;
            }
            expanded += __shfl_sync(0xffffffffu, incl, 31);
        }
        __syncwarp();
        if (a.do_cpu_sync and lane == 0) {
            __threadfence_system();
            a.host->num_expanded_tokens = layout::pack_tagged(epoch, expanded);
            a.host->num_recv_tokens = layout::pack_tagged(epoch, num_recv_tokens);
            __threadfence_system();
        }
        if (lane == 0) dev::trace_point(a.trace, kTrDispCountsExchanged);
        return;
    }

    // ------------------------------------------------------------------ pusher warps
    // running slot base per (warp, rank): tokens of earlier CTAs + earlier warps of this CTA
    if (not a.cached) {
        // tokens of earlier CTAs: one warp per rank, lanes split the CTAs so that the loads overlap
        __shared__ int cta_base[kMaxRanks];
        for (int r = warp; r < num_ranks; r += W) {
            int partial = 0;
            for (int c = lane; c < cta; c += 32) partial += __ldcg(&a.ws->cta_rank_count[c][r]);
            #pragma unroll
            for (int o = 16; o >= 1; o >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, o);
            if (lane == 0) cta_base[r] = partial;
        }
        ptx::named_barrier(1, num_pushers);
        for (int r = threadIdx.x; r < num_ranks; r += num_pushers) {
            int base = cta_base[r];
            for (int w = 0; w < W; ++w) {
                const int cnt = sm.warp_rank[w * kMaxRanks + r];
                sm.warp_rank[w * kMaxRanks + r] = base, base += cnt;
            }
        }
    }
    ptx::named_barrier(1, num_pushers);

    uint64_t* mbar = sm.mbar + warp * (S + 2);
    uint8_t* stages = sm.stages + int64_t(warp) * S * token_bytes;
    uint8_t* src_stages = sm.src_stages + int64_t(warp) * 2 * src_row_bytes;
    int* slots = sm.slots + warp * 32 * k;
    const int load_bytes = a.fused_quant ? src_row_bytes : hidden_bytes;
    bool failed = false;

    auto issue_load = [&](int i) {   // token index i of this warp's range; executed by lane 0
        const int n = i - warp_begin;
        uint8_t* dst = a.fused_quant ? src_stages + (n & 1) * src_row_bytes : stages + (n % S) * token_bytes;
        uint64_t* bar = a.fused_quant ? &mbar[S + (n & 1)] : &mbar[n % S];
        ptx::mbarrier_arrive_expect_tx(bar, load_bytes);
        ptx::bulk_load(dst, a.x + int64_t(i) * load_bytes, load_bytes, bar);
    };

    // Look-ahead of the row loads: with quantisation one row (two source stages), otherwise S - 1 rows, so that S - 1
    // loads are in flight while the oldest row is being sent. Row n + D goes into the stage that row n + D - S used, whose
    // store must have read it: at most S - D - 1 of the committed groups may still be reading.
    const int D = a.fused_quant ? 1 : S - 1;
    if (lane == 0)
        for (int i = warp_begin; i < min(warp_begin + D, warp_end); ++i) issue_load(i);

    for (int i = warp_begin; i < warp_end; ++i) {
        const int n = i - warp_begin, tl_idx = n & 31;
        // ---- slots of the next 32 tokens (pass 2 of the layout), in token order
        if (tl_idx == 0) {
            const int t = i + lane;
            if (a.cached) {
                if (t < warp_end)
                    for (int j = 0; j < k; ++j) slots[lane * k + j] = a.dst_slot_idx[int64_t(t) * k + j];
            } else {
                if (t < warp_end) {
                    for (int j = 0; j < k; ++j) {
                        const int64_t e = a.topk_idx[int64_t(t) * k + j];
                        if (e >= 0 and e < num_experts) atomicOr(&hit[int(e) / num_local_experts], 1u << lane);
                    }
                }
                __syncwarp();
                if (t < warp_end) {
                    unsigned long long seen = 0;
                    for (int j = k - 1; j >= 0; --j) {
                        const int64_t e = a.topk_idx[int64_t(t) * k + j];
                        int slot = -1;
                        if (e >= 0 and e < num_experts) {
                            const int r = int(e) / num_local_experts;
                            if (not((seen >> r) & 1)) slot = run[r] + __popc(hit[r] & ptx::lanemask_lt());
                            seen |= 1ull << r;
                        }
                        slots[lane * k + j] = slot;
                        a.dst_slot_idx[int64_t(t) * k + j] = slot;
                    }
                }
                __syncwarp();
                for (int r = lane; r < num_ranks; r += 32) run[r] += __popc(hit[r]), hit[r] = 0;
            }
            __syncwarp();
        }

        // ---- prefetch the next row
        if (i + D < warp_end) {
            if (a.fused_quant) {
                // the source stage was read with ordinary loads two tokens ago
                ptx::fence_proxy_async_smem();
            } else {
                wait_read_pending(S - D - 1);
            }
            __syncwarp();
            if (lane == 0) issue_load(i + D);
        }

        // ---- assemble the message
        uint8_t* stage = stages + (n % S) * token_bytes;
        if (a.fused_quant) {
            wait_read_pending(S - 1);     // the message stage may still be read by an earlier store
            __syncwarp();
            if (not ptx::mbarrier_wait(&mbar[S + (n & 1)], (n >> 1) & 1)) failed = true;
            quantize_row(src_stages + (n & 1) * src_row_bytes, stage, reinterpret_cast<float*>(stage + tl.sf_offset()),
                         hidden, lane, a.fused_quant == 2);
        } else if (a.sf_bytes > 0) {
            sf_pack_t* dst = reinterpret_cast<sf_pack_t*>(stage + tl.sf_offset());
            for (int p = lane; p < a.sf_bytes / 2; p += 32)
                dst[p] = a.sf[int64_t(i) * a.sf_token_stride + int64_t(p) * a.sf_pack_stride];
        }
        int my_slot = -1, my_rank = 0;
        if (lane < k) {
            const int64_t e = a.topk_idx[int64_t(i) * k + lane];
            const bool valid = e >= 0 and e < num_experts;
            reinterpret_cast<int*>(stage + tl.idx_offset())[lane] = valid ? int(e) : -1;
            reinterpret_cast<float*>(stage + tl.weight_offset())[lane] =
                a.topk_weights != nullptr ? a.topk_weights[int64_t(i) * k + lane] : 0.f;
            my_slot = slots[tl_idx * k + lane];
            my_rank = valid ? int(e) / num_local_experts : 0;
        }
        if (lane == 0) *reinterpret_cast<int*>(stage + tl.src_offset()) = rank * a.num_max_tokens + i;
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (not a.fused_quant and not ptx::mbarrier_wait(&mbar[n % S], (n / S) & 1)) failed = true;
        if (__any_sync(0xffffffffu, failed)) {
            if (lane == 0) dev::report_status(cs, hs, kStatusMbarrierTimeout, rank, -1, kSiteLoad, i, 0);
            break;
        }

        // ---- one bulk store per destination rank, issued by the lane that owns the slot
        if (my_slot >= 0 and my_slot < a.num_max_tokens)
            dev::store_message(cs, hs, a.peers, my_rank, a.buffer_offset, a.buffer_bytes,
                               layout::BufferLayout(token_bytes, num_ranks, a.num_max_tokens).offset(rank, my_slot), stage,
                               token_bytes, kSitePush);
        ptx::bulk_commit();
    }

    // ------------------------------------------------------------------ completion
    if (tracer) dev::trace_point(a.trace, kTrDispPushed);
    ptx::bulk_wait<0>();
    ptx::fence_proxy_async();
    __threadfence_system();
    ptx::named_barrier(1, num_pushers);
    if (tracer) dev::trace_point(a.trace, kTrDispStoresDone);
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
                ptx::st_release_sys(a.peers.sym(&a.ws->dispatch_done[rank], r), static_cast<unsigned long long>(epoch));
            if (lane == 0) a.ws->dispatch_epoch = epoch;
            if (a.wait_arrival) {
                const dev::Deadline deadline(a.timeout_ns);
                for (int s = lane; s < num_ranks; s += 32) {
                    unsigned long long w = 0;
                    if (not dev::spin_until(deadline, [&]() { return (w = ptx::ld_acquire_sys(&a.ws->dispatch_done[s])) == epoch; }))
                        dev::report_status(cs, hs, kStatusArrivalTimeout, rank, s, kSiteArrival, epoch, w);
                }
            }
            __syncwarp();
            if (lane == 0) dev::trace_point(a.trace, kTrDispEnd);       // the CTA that finished last
        }
    }
}

__global__ void __launch_bounds__(32 * 9, 1) ep_dispatch_kernel(const __grid_constant__ DispatchArgs a) {
    ep_dispatch_body<0, 0, 0, 0>(a);
}

}  // namespace deep_ep::kernels
