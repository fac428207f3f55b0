// Destination table that lets a GEMM epilogue take over the combine push of "single-row" tokens.
//
// In the expanded layout a received token owns up to k rows, one per local expert it selected. Combine sends the owner
// of the token ONE message per rank: the fp32 sum of those rows, rounded to bf16. For a token with exactly one row here
// that message is the row itself, so the kernel that produces the row (the second expert GEMM in the forward pass, the
// data-gradient GEMM of the first one in the backward pass) can store it straight into the owner's combine landing slot
// tile by tile, while it is still computing other tiles, and the combine kernel only has to send the routed weights.
// `route[r]` is that landing address (local or peer memory) for such rows and 0 for every other row.
// The reference has no counterpart (it contains no matrix math); the slot arithmetic mirrors `ep_combine.cuh`.
#pragma once

#include "../device/ptx.cuh"
#include "ep_args.hpp"

namespace deep_ep::kernels {

__global__ void __launch_bounds__(256) ep_combine_route_kernel(const __grid_constant__ CombineRouteArgs a) {
    const int num_ranks = a.peers.num_ranks, rank = a.peers.rank, k = a.num_topk;
    const layout::CombineTokenLayout tl(a.hidden_bytes, k);
    const layout::BufferLayout bl(tl.num_bytes(), min(k, num_ranks), a.num_max_tokens);
    const int num_recv = min(a.psum_rank[num_ranks - 1], a.num_metadata_rows);
    for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < num_recv; row += gridDim.x * blockDim.x) {
        int s = 0;
        while (s < num_ranks - 1 and row >= a.psum_rank[s]) ++s;          // source rank of this received token
        const int* meta = a.recv_src_metadata + int64_t(row) * (k + 2);
        int count = 0, slot = -1;
        for (int j = 0; j < k; ++j)
            if (meta[j] >= 0) ++count, slot = meta[j];
        const int token = meta[k] - s * a.num_max_tokens, master = meta[k + 1];
        // the same validity rules as the combine kernel, which skips the payload of exactly these rows
        if (count != 1 or token < 0 or token >= a.num_max_tokens or master < 0 or slot >= a.num_expanded_rows) continue;
        const int group = num_ranks >= k ? master : rank;
        a.route[slot] = reinterpret_cast<unsigned long long>(a.peers.base[s] + a.buffer_offset + bl.offset(group, token));
    }
}

}  // namespace deep_ep::kernels
