// Barrier, Engram fetch, batched all-gather and pipeline send/recv kernels for sm_100a.
// Reference roles: `impls/comm/barrier.hpp:13-21`, `impls/engram/engram_fetch.hpp:15-138`,
// `impls/bucket/all_gather/urma.hpp:9-48`, `impls/pp/pp_send_recv.hpp:14-166`. All of them move data
// with ordinary peer loads/stores (or NVLS `multimem.st`) issued by the SMs over NVLink.
#pragma once

#include <cuda_fp16.h>

#include "../device/bulk_copy.cuh"
#include "../device/sync.cuh"
#include "misc_args.hpp"

namespace deep_ep::kernels {

// ---------------------------------------------------------------------------------------- barrier
__global__ void __launch_bounds__(32) rank_barrier_kernel(const __grid_constant__ BarrierArgs a) {
    if (not dev::healthy(a.cs)) return;
    // `repeats` > 1: that many barriers back to back inside one launch, which is how the barrier's own latency is timed
    // (a loop of launches measures the host's launch rate instead); every rank must pass the same count
    for (int i = 0; i < max(a.repeats, 1); ++i)
        if (not dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, /*where=*/1)) return;
}

// ---------------------------------------------------------------------------------------- engram
// One warp per (layer, token, entry); four entries are kept in flight per warp so that small
// (512 B) remote reads overlap. Negative indices are skipped and leave the destination untouched.
__global__ void __launch_bounds__(256) engram_fetch_kernel(const __grid_constant__ EngramFetchArgs a) {
    constexpr int kInflight = 4;
    const int lane = ptx::lane_id();
    const int64_t gw = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
    const int64_t num_gw = int64_t(gridDim.x) * blockDim.x / 32;
    const int64_t per_layer = int64_t(a.num_tokens) * a.num_entries_per_token;
    const int64_t total = per_layer * a.num_layers;
    const int chunks = a.hidden_bytes / 16;

    for (int64_t base = gw * kInflight; base < total; base += num_gw * kInflight) {
        const uint8_t* src[kInflight];
        uint8_t* dst[kInflight];
        #pragma unroll
        for (int u = 0; u < kInflight; ++u) {
            src[u] = nullptr, dst[u] = nullptr;
            const int64_t i = base + u;
            if (i >= total) continue;
            const int layer = int(i / per_layer);
            const int64_t in_layer = i % per_layer;
            const int idx = a.indices[i];
            if (idx < 0) continue;
            const int entries = a.table.num_entries_per_rank[layer];
            const int owner = idx / entries, entry = idx % entries;
            if (owner >= a.peers.num_ranks) continue;
            src[u] = a.peers.base[owner] + a.table.storage_offset[layer] + int64_t(entry) * a.hidden_bytes;
            const int64_t token = in_layer / a.num_entries_per_token, p = in_layer % a.num_entries_per_token;
            dst[u] = a.recv + ((int64_t(layer) * a.num_max_tokens + token) * a.num_entries_per_token + p) * a.hidden_bytes;
            if (a.sf_out != nullptr) {
                const sf_pack_t* sf_src = reinterpret_cast<const sf_pack_t*>(
                    a.peers.base[owner] + a.table.sf_offset[layer]) + int64_t(entry) * a.num_sf_packs;
                sf_pack_t* sf_dst = a.sf_out + layer * a.sf_layer_stride + token * a.sf_token_stride;
                for (int q = lane; q < a.num_sf_packs; q += 32)
                    sf_dst[(p * a.num_sf_packs + q) * a.sf_pack_stride] = sf_src[q];
            }
        }
        for (int c = lane; c < chunks; c += 32) {
            int4 v[kInflight];
            #pragma unroll
            for (int u = 0; u < kInflight; ++u)
                if (src[u] != nullptr) v[u] = ptx::ld_nc_v4(src[u] + c * 16);
            #pragma unroll
            for (int u = 0; u < kInflight; ++u)
                if (src[u] != nullptr) ptx::st_na_v4(dst[u] + c * 16, v[u]);
        }
    }
}

// ---------------------------------------------------------------------------------------- all-gather
namespace ag_detail {

EP_DEVICE void multimem_st_v4(void* mc_ptr, const int4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 ::"l"(mc_ptr), "f"(__int_as_float(v.x)), "f"(__int_as_float(v.y)), "f"(__int_as_float(v.z)),
                   "f"(__int_as_float(v.w)) : "memory");
}

}  // namespace ag_detail

// Every rank writes its shard of every bucket into all peers at `dst_offset + rank * num_bytes`.
// Work is cut into 32 KiB tiles spread over all CTAs; each tile is read once and written to every
// destination (peer order rotated by rank), or written once through the NVLS multicast mapping.
__global__ void __launch_bounds__(512) bucket_all_gather_kernel(const __grid_constant__ AllGatherArgs a) {
    constexpr int64_t kTileBytes = 32 * 1024;
    extern __shared__ uint8_t ag_smem[];
    const int rank = a.peers.rank, num_ranks = a.peers.num_ranks;
    const int warp = threadIdx.x / 32, lane = ptx::lane_id(), warps_per_cta = blockDim.x / 32;
    dev::WarpCopier copier;
    copier.init(ag_smem, warps_per_cta, warp, lane);

    // "destinations have been consumed" barrier, then release the other CTAs
    if (not dev::healthy(a.cs)) return;
    if (blockIdx.x == 0 and threadIdx.x < 32)
        dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, /*where=*/40);
    if (not dev::grid_sync(a.cs, a.host_status, gridDim.x, a.timeout_ns, rank, /*where=*/41)) return;

    int64_t tile_base = 0;
    for (int b = 0; b < a.list.num_buckets; ++b) {
        const layout::Bucket& bucket = a.list.buckets[b];
        const int64_t num_tiles = math::ceil_div(bucket.num_bytes, kTileBytes);
        const int64_t dst_off = bucket.dst_offset + int64_t(rank) * bucket.num_bytes;
        // widest access that keeps source and every destination aligned (bases are 2 MiB aligned)
        const uint64_t mis = reinterpret_cast<uint64_t>(bucket.src) | uint64_t(dst_off) | uint64_t(bucket.num_bytes);
        const bool vec16 = (mis & 15) == 0;
        for (int64_t tile = (blockIdx.x + gridDim.x - tile_base % gridDim.x) % gridDim.x; tile < num_tiles; tile += gridDim.x) {
            const int64_t begin = tile * kTileBytes, end = min(begin + kTileBytes, bucket.num_bytes);
            if (vec16 and not a.use_multicast) {
                // read each 8 KiB chunk once into shared memory, store it to every destination with the TMA engine
                for (int64_t o = begin + int64_t(warp) * dev::kCopyChunkBytes; o < end; o += int64_t(warps_per_cta) * dev::kCopyChunkBytes) {
                    const int bytes = int(min(int64_t(dev::kCopyChunkBytes), end - o));
                    const int num_dsts = a.skip_local ? num_ranks - 1 : num_ranks;
                    copier.copy_chunk(bucket.src + o, bytes, num_dsts, [&](int i) {
                        return a.peers.base[(rank + 1 + i) % num_ranks] + dst_off + o;      // rotation: the local rank comes last
                    }, lane);
                }
            } else if (vec16) {
                for (int64_t o = begin + threadIdx.x * 16; o < end; o += blockDim.x * 16) {
                    const int4 v = ptx::ld_nc_v4(bucket.src + o);
                    if (a.use_multicast) {
                        ag_detail::multimem_st_v4(a.peers.mc_base + dst_off + o, v);
                    } else {
                        for (int i = 0; i < num_ranks; ++i) {
                            const int p = (rank + 1 + i) % num_ranks;
                            if (p == rank and a.skip_local) continue;
                            ptx::st_na_v4(a.peers.base[p] + dst_off + o, v);
                        }
                    }
                }
            } else {
                // odd sizes or unaligned addresses: byte granularity (rare, small tensors)
                for (int64_t o = begin + threadIdx.x; o < end; o += blockDim.x) {
                    const uint8_t v = bucket.src[o];
                    for (int i = 0; i < num_ranks; ++i) {
                        const int p = (rank + 1 + i) % num_ranks;
                        if (p == rank and a.skip_local) continue;
                        a.peers.base[p][dst_off + o] = v;
                    }
                }
            }
        }
        tile_base += num_tiles;
    }
    copier.drain();
    if (copier.failed and lane == 0) dev::report_status(a.cs, a.host_status, kStatusMbarrierTimeout, rank, -1, 42, 0, 0);
    __threadfence_system();
}

// ---------------------------------------------------------------------------------------- reduce-scatter / all-reduce
// One pass over this rank's shard of every tensor: each 16-byte vector is pulled from all ranks (plain peer loads,
// all in flight together), summed in fp32 in rank order (so the result does not depend on who reduces), scaled,
// rounded to the tensor's dtype and stored in place on the owner; for an all-reduce the same registers are then stored
// to the shard's position on every peer. Nobody else reads or writes shard `rank` positions, so the operation is in
// place without staging. It starts with a rank barrier (every source is complete) and ends with one (every read and
// write has been performed), so sources may be reused as soon as the kernel has completed.
// The reference declares these two collectives without a kernel (`csrc/buffers/bucket.hpp:66-75`).
namespace reduce_detail {

template <int kDtype>
EP_DEVICE void accumulate(float (&acc)[8], const int4& v) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
    if constexpr (kDtype == kReduceFP32) {
        #pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += __uint_as_float(w[i]);
    } else if constexpr (kDtype == kReduceBF16) {
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = ptx::bf16x2_to_float2(w[i]);
            acc[2 * i] += f.x, acc[2 * i + 1] += f.y;
        }
    } else {
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            acc[2 * i] += f.x, acc[2 * i + 1] += f.y;
        }
    }
}

template <int kDtype>
EP_DEVICE int4 finish(const float (&acc)[8], float scale) {
    int4 out;
    uint32_t* w = reinterpret_cast<uint32_t*>(&out);
    if constexpr (kDtype == kReduceFP32) {
        #pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = __float_as_uint(acc[i] * scale);
    } else if constexpr (kDtype == kReduceBF16) {
        #pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = ptx::float2_to_bf16x2(acc[2 * i] * scale, acc[2 * i + 1] * scale);
    } else {
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(acc[2 * i] * scale, acc[2 * i + 1] * scale);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    return out;
}

EP_DEVICE void store_result(const BucketReduceArgs& a, int64_t offset, const int4& out) {
    const int rank = a.peers.rank, num_ranks = a.peers.num_ranks;
    if (a.all_reduce) {
        for (int i = 0; i < num_ranks; ++i)       // the local copy comes last
            ptx::st_na_v4(a.peers.base[(rank + 1 + i) % num_ranks] + offset, out);
    } else {
        ptx::st_v4(a.peers.base[rank] + offset, out);
    }
}

// NVLS variants: one instruction fetches the 16-byte vector from every GPU of the multicast group and returns the sum
// (accumulated in fp32 inside the switch), one instruction stores a vector to every GPU.
template <int kDtype>
EP_DEVICE int4 multimem_ld_reduce_v4(const void* mc_ptr) {
    int4 v;
    if constexpr (kDtype == kReduceFP32) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
    } else if constexpr (kDtype == kReduceBF16) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
    } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
    }
    return v;
}

template <int kDtype>
EP_DEVICE void reduce_bucket_multicast(const BucketReduceArgs& a, const layout::Bucket& bucket, int64_t& tile_base) {
    constexpr int64_t kTileBytes = 64 * 1024;
    constexpr int kUnroll = 4;
    const int rank = a.peers.rank, num_ranks = a.peers.num_ranks;
    const int64_t shard_bytes = bucket.num_bytes / num_ranks;
    const int64_t base_off = bucket.dst_offset + int64_t(rank) * shard_bytes;
    const int64_t num_tiles = math::ceil_div(shard_bytes, kTileBytes);
    const int64_t step = int64_t(blockDim.x) * 16;
    for (int64_t tile = (blockIdx.x + gridDim.x - tile_base % gridDim.x) % gridDim.x; tile < num_tiles; tile += gridDim.x) {
        const int64_t begin = tile * kTileBytes, end = min(begin + kTileBytes, shard_bytes);
        for (int64_t o = begin + threadIdx.x * 16; o < end; o += step * kUnroll) {
            int4 v[kUnroll];
            #pragma unroll
            for (int u = 0; u < kUnroll; ++u)
                v[u] = multimem_ld_reduce_v4<kDtype>(a.peers.mc_base + base_off + (o + u * step < end ? o + u * step : o));
            #pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (o + u * step >= end) break;
                int4 out = v[u];
                if (a.scale != 1.0f) {
                    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    accumulate<kDtype>(acc, v[u]);
                    out = finish<kDtype>(acc, a.scale);
                }
                if (a.all_reduce) ag_detail::multimem_st_v4(a.peers.mc_base + base_off + o + u * step, out);
                else ptx::st_v4(a.peers.base[rank] + base_off + o + u * step, out);
            }
        }
    }
    tile_base += num_tiles;
}

// `kNumRanks` > 0: the group size is a compile-time constant and a thread keeps `16 / kNumRanks` vectors x `kNumRanks`
// loads in flight (16 outstanding 16-byte loads: what covers the NVLink latency with one 256-thread CTA per SM).
// `kNumRanks` == 0: any group size, one vector at a time, eight ranks per round of loads.
template <int kDtype, int kNumRanks>
EP_DEVICE void reduce_bucket(const BucketReduceArgs& a, const layout::Bucket& bucket, int64_t& tile_base) {
    constexpr int64_t kTileBytes = 64 * 1024;
    constexpr int kUnroll = kNumRanks == 0 ? 1 : (kNumRanks >= 8 ? 2 : 16 / (kNumRanks < 2 ? 2 : kNumRanks));
    const int rank = a.peers.rank, num_ranks = a.peers.num_ranks;
    const int64_t shard_bytes = bucket.num_bytes / num_ranks;
    const int64_t base_off = bucket.dst_offset + int64_t(rank) * shard_bytes;
    const int64_t num_tiles = math::ceil_div(shard_bytes, kTileBytes);
    const int64_t step = int64_t(blockDim.x) * 16;
    for (int64_t tile = (blockIdx.x + gridDim.x - tile_base % gridDim.x) % gridDim.x; tile < num_tiles; tile += gridDim.x) {
        const int64_t begin = tile * kTileBytes, end = min(begin + kTileBytes, shard_bytes);
        for (int64_t o = begin + threadIdx.x * 16; o < end; o += step * kUnroll) {
            if constexpr (kNumRanks > 0) {
                int4 v[kUnroll][kNumRanks];
                #pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    // vectors past the end of the tile re-read its first vector and are not stored
                    const int64_t ou = o + u * step < end ? o + u * step : o;
                    #pragma unroll
                    for (int i = 0; i < kNumRanks; ++i) v[u][i] = ptx::ld_v4(a.peers.base[i] + base_off + ou);
                }
                #pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    #pragma unroll
                    for (int i = 0; i < kNumRanks; ++i) accumulate<kDtype>(acc, v[u][i]);
                    if (o + u * step < end) store_result(a, base_off + o + u * step, finish<kDtype>(acc, a.scale));
                }
            } else {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int p0 = 0; p0 < num_ranks; p0 += 8) {
                    int4 v[8];
                    #pragma unroll
                    for (int i = 0; i < 8; ++i)
                        v[i] = ptx::ld_v4(a.peers.base[min(p0 + i, num_ranks - 1)] + base_off + o);
                    #pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (p0 + i < num_ranks) accumulate<kDtype>(acc, v[i]);
                }
                store_result(a, base_off + o, finish<kDtype>(acc, a.scale));
            }
        }
    }
    tile_base += num_tiles;
}

}  // namespace reduce_detail

template <int kNumRanks>
__global__ void __launch_bounds__(256) bucket_reduce_kernel(const __grid_constant__ BucketReduceArgs a) {
    const int rank = a.peers.rank;
    if (not dev::healthy(a.cs)) return;
    if (blockIdx.x == 0 and threadIdx.x < 32) dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, /*where=*/44);
    if (not dev::grid_sync(a.cs, a.host_status, gridDim.x, a.timeout_ns, rank, /*where=*/45)) return;
    int64_t tile_base = 0;
    for (int b = 0; b < a.list.num_buckets; ++b) {
        const layout::Bucket& bucket = a.list.buckets[b];
        if (a.dtype[b] == kReduceFP32) reduce_detail::reduce_bucket<kReduceFP32, kNumRanks>(a, bucket, tile_base);
        else if (a.dtype[b] == kReduceBF16) reduce_detail::reduce_bucket<kReduceBF16, kNumRanks>(a, bucket, tile_base);
        else reduce_detail::reduce_bucket<kReduceFP16, kNumRanks>(a, bucket, tile_base);
    }
    __threadfence_system();
    if (not dev::grid_sync(a.cs, a.host_status, gridDim.x, a.timeout_ns, rank, /*where=*/46)) return;
    if (blockIdx.x == 0 and threadIdx.x < 32) dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, /*where=*/47);
}

// The same collective through the NVLink multicast mapping (`peers.mc_base`, present on the NVLS route only).
__global__ void __launch_bounds__(256) bucket_reduce_multicast_kernel(const __grid_constant__ BucketReduceArgs a) {
    const int rank = a.peers.rank;
    if (not dev::healthy(a.cs)) return;
    if (blockIdx.x == 0 and threadIdx.x < 32) dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, /*where=*/48);
    if (not dev::grid_sync(a.cs, a.host_status, gridDim.x, a.timeout_ns, rank, /*where=*/49)) return;
    int64_t tile_base = 0;
    for (int b = 0; b < a.list.num_buckets; ++b) {
        const layout::Bucket& bucket = a.list.buckets[b];
        if (a.dtype[b] == kReduceFP32) reduce_detail::reduce_bucket_multicast<kReduceFP32>(a, bucket, tile_base);
        else if (a.dtype[b] == kReduceBF16) reduce_detail::reduce_bucket_multicast<kReduceBF16>(a, bucket, tile_base);
        else reduce_detail::reduce_bucket_multicast<kReduceFP16>(a, bucket, tile_base);
    }
    __threadfence_system();
    if (not dev::grid_sync(a.cs, a.host_status, gridDim.x, a.timeout_ns, rank, /*where=*/50)) return;
    if (blockIdx.x == 0 and threadIdx.x < 32) dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, /*where=*/51);
}

// ---------------------------------------------------------------------------------------- load balancing
// Collective over the NVLink domain. Mode 0 pushes this rank's expert weights into every redundant slot that a
// peer assigned to one of them; mode 1 pulls the gradients of those redundant copies and adds them to the
// owner's fp32 gradient. Both start with a rank barrier (slots / gradients are ready everywhere) and end with
// one (all transfers have landed), so the data is usable once the kernel has completed on every rank.
// The reference exposes this API without a kernel behind it (`csrc/buffers/ep.hpp:75-86`).
__global__ void __launch_bounds__(512) lb_exchange_kernel(const __grid_constant__ LBArgs a) {
    const int rank = a.peers.rank, num_ranks = a.peers.num_ranks;
    if (not dev::healthy(a.cs)) return;
    if (blockIdx.x == 0 and threadIdx.x < 32) dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, 70);
    if (not dev::grid_sync(a.cs, a.host_status, gridDim.x, a.timeout_ns, rank, 71)) return;

    const int num_slots = num_ranks * a.num_redundant;
    if (a.mode == 0) {
        int task = 0;
        for (int s = 0; s < num_slots; ++s) {
            const int e = a.mapping[s];
            if (e < 0 or e / a.num_local_experts != rank) continue;
            const int r = s / a.num_redundant, c = s % a.num_redundant, local = e % a.num_local_experts;
            for (int i = 0; i < a.num_tensors; ++i, ++task) {
                if (task % gridDim.x != blockIdx.x) continue;
                const int64_t bytes = a.bytes_per_expert[i];
                const uint8_t* src = a.src[i] + local * bytes;
                uint8_t* dst = a.peers.base[r] + a.dst_offset[i] + c * bytes;
                for (int64_t o = threadIdx.x * 16; o < bytes; o += blockDim.x * 16)
                    ptx::st_na_v4(dst + o, ptx::ld_nc_v4(src + o));
            }
        }
    } else {
        // one thread owns a column of one local expert, so additions to an element are ordered
        const int64_t total = int64_t(a.num_local_experts) * a.hidden;
        for (int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
            const int local = int(idx / a.hidden);
            const int64_t col = idx % a.hidden;
            float acc = a.expert_grads[idx];
            for (int s = 0; s < num_slots; ++s) {
                if (a.mapping[s] != rank * a.num_local_experts + local) continue;
                const int r = s / a.num_redundant, c = s % a.num_redundant;
                acc += *reinterpret_cast<const float*>(a.peers.base[r] + a.dst_offset[0] + (int64_t(c) * a.hidden + col) * 4);
            }
            a.expert_grads[idx] = acc;
        }
    }
    __threadfence_system();
    if (not dev::grid_sync(a.cs, a.host_status, gridDim.x, a.timeout_ns, rank, 72)) return;
    if (blockIdx.x == 0 and threadIdx.x < 32) dev::rank_barrier_warp(a.cs, a.host_status, a.peers, a.timeout_ns, 73);
}

// ---------------------------------------------------------------------------------------- pipeline
namespace pp_detail {

// Grid-wide copy. 16-byte aligned ranges go through the TMA ring of `copier`; the tail and unaligned ranges use
// ordinary loads and stores.
EP_DEVICE void copy_bytes(uint8_t* dst, const uint8_t* src, int64_t n, dev::WarpCopier& copier) {
    const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x, nthreads = int64_t(gridDim.x) * blockDim.x;
    if (((reinterpret_cast<uint64_t>(dst) | reinterpret_cast<uint64_t>(src)) & 15) == 0 and n >= dev::kCopyChunkBytes) {
        const int lane = ptx::lane_id();
        const int64_t gw = tid / 32, num_gw = nthreads / 32;
        const int64_t body = n / 16 * 16;
        for (int64_t o = gw * dev::kCopyChunkBytes; o < body; o += num_gw * dev::kCopyChunkBytes) {
            const int bytes = int(min(int64_t(dev::kCopyChunkBytes), body - o));
            copier.copy_chunk(src + o, bytes, 1, [&](int) { return dst + o; }, lane);
        }
        copier.drain();
        for (int64_t i = body + tid; i < n; i += nthreads) dst[i] = src[i];
    } else if (((reinterpret_cast<uint64_t>(dst) | reinterpret_cast<uint64_t>(src)) & 15) == 0) {
        const int64_t nvec = n / 16;
        for (int64_t i = tid; i < nvec; i += nthreads) ptx::st_na_v4(dst + i * 16, ptx::ld_v4(src + i * 16));
        for (int64_t i = nvec * 16 + tid; i < n; i += nthreads) dst[i] = src[i];
    } else {
        for (int64_t i = tid; i < n; i += nthreads) dst[i] = src[i];
    }
}

// true for exactly one CTA: the last one to arrive
EP_DEVICE bool last_cta(layout::CommonSignals* cs) {
    __shared__ int is_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        is_last = atomicAdd(&cs->done_ctas, 1u) == gridDim.x - 1;
        if (is_last) cs->done_ctas = 0;
    }
    __syncthreads();
    return is_last != 0;
}

}  // namespace pp_detail

// Buffered send to a ring neighbour: wait for a free slot (credit), copy the tensor into the
// neighbour's landing slot, then publish the arrival counter with release semantics.
__global__ void __launch_bounds__(512) pp_send_kernel(const __grid_constant__ PPArgs a) {
    extern __shared__ uint8_t pp_smem[];
    layout::CommonSignals* cs = &a.ws->common;
    if (not dev::healthy(cs)) return;
    dev::WarpCopier copier;
    copier.init(pp_smem, blockDim.x / 32, threadIdx.x / 32, ptx::lane_id());
    const int d = a.direction;
    const unsigned long long n = a.ws->send_count[d];
    __shared__ int ok_smem;
    if (threadIdx.x == 0) {
        const dev::Deadline deadline(a.timeout_ns);
        unsigned long long freed = 0;
        const bool ok = dev::spin_until(deadline, [&]() {
            freed = ptx::ld_acquire_sys(&a.ws->release[d]);
            return freed + a.num_inflight >= n + 1;
        });
        if (not ok) dev::report_status(cs, a.host_status, kStatusCreditTimeout, a.peers.rank, a.peer, 50, n + 1, freed);
        ok_smem = ok;
    }
    __syncthreads();
    if (not ok_smem) return;
    // the receiver sees data from its previous rank in region 1 and from its next rank in region 0
    const int region = 1 - d;
    uint8_t* slot = a.peers.base[a.peer] + a.storage_offset + (int64_t(region) * a.num_inflight + n % a.num_inflight) * a.slot_bytes;
    pp_detail::copy_bytes(slot, a.x, a.num_bytes, copier);
    if (copier.failed and ptx::lane_id() == 0) dev::report_status(cs, a.host_status, kStatusMbarrierTimeout, a.peers.rank, a.peer, 52, 0, 0);
    if (pp_detail::last_cta(cs) and threadIdx.x == 0) {
        ptx::st_release_sys(a.peers.sym(&a.ws->arrival[region], a.peer), n + 1);
        a.ws->send_count[d] = n + 1;
    }
}

// Matching receive: wait for the arrival counter, copy out of the landing slot, return the credit.
__global__ void __launch_bounds__(512) pp_recv_kernel(const __grid_constant__ PPArgs a) {
    extern __shared__ uint8_t pp_smem[];
    layout::CommonSignals* cs = &a.ws->common;
    if (not dev::healthy(cs)) return;
    dev::WarpCopier copier;
    copier.init(pp_smem, blockDim.x / 32, threadIdx.x / 32, ptx::lane_id());
    const int d = a.direction;            // region index == direction of the source
    const unsigned long long n = a.ws->recv_count[d];
    __shared__ int ok_smem;
    if (threadIdx.x == 0) {
        const dev::Deadline deadline(a.timeout_ns);
        unsigned long long arrived = 0;
        const bool ok = dev::spin_until(deadline, [&]() { return (arrived = ptx::ld_acquire_sys(&a.ws->arrival[d])) >= n + 1; });
        if (not ok) dev::report_status(cs, a.host_status, kStatusArrivalTimeout, a.peers.rank, a.peer, 51, n + 1, arrived);
        ok_smem = ok;
    }
    __syncthreads();
    if (not ok_smem) return;
    const uint8_t* slot = a.peers.base[a.peers.rank] + a.storage_offset + (int64_t(d) * a.num_inflight + n % a.num_inflight) * a.slot_bytes;
    pp_detail::copy_bytes(a.x, slot, a.num_bytes, copier);
    if (copier.failed and ptx::lane_id() == 0) dev::report_status(cs, a.host_status, kStatusMbarrierTimeout, a.peers.rank, a.peer, 53, 0, 0);
    if (pp_detail::last_cta(cs) and threadIdx.x == 0) {
        // the sender addressed me through its direction 1 - d
        ptx::st_release_sys(a.peers.sym(&a.ws->release[1 - d], a.peer), n + 1);
        a.ws->recv_count[d] = n + 1;
    }
}

}  // namespace deep_ep::kernels
