// Plain-data argument blocks of the expert-parallel kernels and their shared-memory sizing, usable
// from the host runtime (g++) and from device code. The kernels themselves live in the `.cuh` files
// next to this header.
#pragma once

#include "../layout/ep.hpp"

namespace deep_ep::kernels {

// Phase trace: when a kernel gets a non-null `trace`, single threads of CTA 0 (and of the CTA that finishes last) store
// `%globaltimer` at the phase boundaries named below; the host subtracts neighbouring stamps. Each kernel owns 16 slots.
constexpr int kTraceSlots = 16;
enum DispatchTrace : int { kTrDispStart = 0, kTrDispCounted, kTrDispEntryBarrier, kTrDispGridSync, kTrDispCountsExchanged,
                           kTrDispPushed, kTrDispStoresDone, kTrDispEnd };
enum ExpandTrace : int { kTrExpStart = 0, kTrExpArrived, kTrExpLaidOut, kTrExpEnd };
enum CombineTrace : int { kTrCombStart = 0, kTrCombEntryBarrier, kTrCombGridSync, kTrCombPushed, kTrCombStoresDone, kTrCombEnd };
enum ReduceTrace : int { kTrRedStart = 0, kTrRedArrived, kTrRedEnd };

struct DispatchArgs {
    // inputs
    const uint8_t* x;               // [T, row_bytes]: wire bytes, or BF16 source rows when fused_quant
    const sf_pack_t* sf;            // [T, sf_bytes / 2] packs with strides below, or nullptr
    int64_t sf_token_stride, sf_pack_stride;
    const int64_t* topk_idx;        // [T, k]
    const float* topk_weights;      // [T, k] or nullptr
    int num_tokens, hidden_bytes, sf_bytes, num_topk, num_experts, num_max_tokens, expert_alignment;
    int cached, fused_quant, do_cpu_sync, wait_arrival;
    // handle tensors
    int* dst_slot_idx;              // [T, k]
    int* psum_rank;                 // [R]
    int* psum_expert;               // [E_local]
    int* num_unaligned;             // [E_local]
    int* cumulative_stats;          // [E_local] or nullptr
    // communication
    layout::EPSignals* ws;
    int64_t buffer_offset;          // receive buffer offset inside the symmetric allocation
    int64_t buffer_bytes;           // size of the receive buffer (bounds-checked build)
    layout::PeerTable peers;
    layout::EPHostCounts* host;
    long long timeout_ns;
    int num_warps, num_stages;      // pusher warps per CTA, message stages per warp
    unsigned long long* trace;      // optional [kTraceSlots] `%globaltimer` stamps of the phases (CTA 0 and the last CTA), or nullptr
};

struct ExpandArgs {
    layout::EPSignals* ws;
    const uint8_t* buffer;            // local receive buffer ([source rank][max tokens] messages)
    layout::EPHostCounts* host;
    const int* psum_rank;             // [R] inclusive
    const int* psum_expert;           // [E_local]
    const int* num_unaligned;         // [E_local]
    uint8_t* recv_x;                  // [num_expanded, hidden_bytes]
    sf_pack_t* recv_sf;               // strided, or nullptr
    int64_t recv_sf_token_stride, recv_sf_pack_stride;
    float* recv_topk_weights;         // [num_expanded] or nullptr
    int* recv_src_metadata;           // [num_recv_rows, k + 2]
    int num_metadata_rows, num_expanded_rows;   // capacities of the output tensors
    int rank, num_ranks, num_max_tokens, num_experts, num_topk, expert_alignment;
    int hidden_bytes, sf_bytes;
    int cached, do_zero_padding, wait_arrival;
    long long timeout_ns;
    int num_warps, num_stages;
    unsigned long long* trace;        // optional phase stamps, see DispatchArgs
};

struct CombineArgs {
    const uint8_t* x;                 // [num_expanded, hidden_bytes] bf16
    const float* topk_weights;        // [num_expanded] or nullptr
    const int* recv_src_metadata;     // [rows, k + 2]
    const int* psum_rank;             // [R]
    int num_metadata_rows;
    int num_topk, num_max_tokens, hidden_bytes;
    int wait_arrival;
    layout::EPSignals* ws;
    int64_t buffer_offset;
    int64_t buffer_bytes;             // size of the landing buffer (bounds-checked build)
    layout::PeerTable peers;
    layout::EPHostCounts* host;
    long long timeout_ns;
    int num_warps, num_stages;
    unsigned long long* trace;        // optional phase stamps, see DispatchArgs
    int coop;                         // 1: when rows are scarce, several warps of a CTA share a row (decode-sized calls)
    int weighted;                     // 1: every expanded row is multiplied by its entry of `topk_weights` before the sum
    int skip_single;                  // 1: rows that are their token's only one were already stored into the owner's landing
                                      //    slot by a GEMM epilogue (`ep_route.cuh`); only their routed weights are sent
};

struct CombineReduceArgs {
    layout::EPSignals* ws;
    const uint8_t* buffer;            // local landing buffer
    layout::EPHostCounts* host;
    const int64_t* topk_idx;          // [T, k]
    const uint8_t* bias_0;            // [T, hidden_bytes] bf16 or nullptr
    const uint8_t* bias_1;
    uint8_t* combined_x;              // [T, hidden_bytes]
    float* combined_topk_weights;     // [T, k] or nullptr
    int num_tokens, num_topk, num_experts, num_max_tokens, hidden_bytes;
    int rank, num_ranks;
    int wait_arrival;
    long long timeout_ns;
    unsigned long long* trace;        // optional phase stamps, see DispatchArgs
    int coop;                         // 1: when tokens are scarce, several warps share a token
};

// Destination table for GEMM epilogues that take over the combine push of single-row tokens (`ep_route.cuh`).
struct CombineRouteArgs {
    const int* recv_src_metadata;     // [rows, k + 2]: expanded row per top-k position (-1 = none), source token, master position
    const int* psum_rank;             // [R] inclusive prefix of received tokens per source rank
    int num_metadata_rows, num_expanded_rows;
    int num_topk, num_max_tokens, hidden_bytes;
    int64_t buffer_offset;            // landing buffer offset inside every rank's allocation
    layout::PeerTable peers;
    unsigned long long* route;        // [num_expanded_rows], zero-initialised by the caller
};

namespace dispatch_detail {
EP_HOST_DEVICE int64_t smem_bytes(int num_warps, int num_stages, int num_topk, int num_experts, int token_bytes,
                                  int src_row_bytes) {
    int64_t n = 0;
    n += int64_t(num_warps) * (num_stages + 2) * 8;
    n += int64_t(num_warps) * kMaxRanks * 4 * 2;
    n += int64_t(num_experts) * 4;
    n += int64_t(num_warps) * 32 * num_topk * 4;
    n = math::align<int64_t>(n, 128);
    n += int64_t(num_warps) * num_stages * token_bytes;
    n = math::align<int64_t>(n, 128);
    n += int64_t(num_warps) * 2 * src_row_bytes;
    return n + 128;
}
}  // namespace dispatch_detail

namespace expand_detail {
EP_HOST_DEVICE int64_t smem_bytes(int num_warps, int num_stages, int num_topk, int num_local_experts, int token_bytes) {
    int64_t n = int64_t(num_warps) * num_stages * 8;
    n += int64_t(num_warps) * num_local_experts * 4 * 2;      // running bases + hit bitmaps
    n += int64_t(num_local_experts) * 4 * 2;                  // expert region ends and per-CTA bases
    n += int64_t(num_warps) * 32 * (num_topk + 1) * 4;        // slots (+ source row index)
    n = math::align<int64_t>(n, 128);
    n += int64_t(num_warps) * num_stages * token_bytes;
    return n + 128;
}
}  // namespace expand_detail

namespace combine_detail {
EP_HOST_DEVICE int64_t smem_bytes(int num_warps, int num_stages, int token_bytes) {
    return int64_t(num_warps) * num_stages * 8 + 128 + int64_t(num_warps) * num_stages * token_bytes + 128;
}
}  // namespace combine_detail

}  // namespace deep_ep::kernels
