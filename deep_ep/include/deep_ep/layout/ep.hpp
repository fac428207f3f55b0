// Wire formats and workspace of the expert-parallel buffer, shared by host sizing code and the
// kernels. Same role as the reference's `layout/ep/token.hpp:9-130` and `layout/ep/workspace.hpp:8-68`,
// with a B200 wire format: every message is one contiguous, 16-byte aligned block so a single
// `cp.async.bulk` store moves it (the reference gathers two segments per token instead).
#pragma once

#include "../common/math.hpp"
#include "signals.hpp"

namespace deep_ep::layout {

// Dispatch message: [hidden bytes][scale-factor bytes ^16][topk_idx i32 x k][topk_weights f32 x k][src_token_global_idx i32] ^16
struct DispatchTokenLayout {
    int hidden_bytes, sf_bytes, num_topk;

    EP_HOST_DEVICE DispatchTokenLayout(int hidden_bytes, int sf_bytes, int num_topk)
        : hidden_bytes(hidden_bytes), sf_bytes(sf_bytes), num_topk(num_topk) {}
    EP_HOST_DEVICE int sf_offset() const { return hidden_bytes; }
    EP_HOST_DEVICE int idx_offset() const { return hidden_bytes + math::align(sf_bytes, kBulkAlignmentBytes); }
    EP_HOST_DEVICE int weight_offset() const { return idx_offset() + 4 * num_topk; }
    EP_HOST_DEVICE int src_offset() const { return weight_offset() + 4 * num_topk; }
    EP_HOST_DEVICE int num_bytes() const { return math::align(src_offset() + 4, kBulkAlignmentBytes); }
};

// Combine message: [hidden bf16][topk_weights f32 x k] ^16
struct CombineTokenLayout {
    int hidden_bytes, num_topk;

    EP_HOST_DEVICE CombineTokenLayout(int hidden_bytes, int num_topk) : hidden_bytes(hidden_bytes), num_topk(num_topk) {}
    EP_HOST_DEVICE int weight_offset() const { return hidden_bytes; }
    EP_HOST_DEVICE int num_bytes() const { return math::align(hidden_bytes + 4 * num_topk, kBulkAlignmentBytes); }
};

// A receive buffer is `[num_groups][num_max_tokens_per_rank]` messages. Dispatch: group = source
// rank. Combine: group = master top-k position (or producer rank when num_ranks < num_topk).
struct BufferLayout {
    int64_t token_bytes;
    int num_groups, num_max_tokens;

    EP_HOST_DEVICE BufferLayout(int64_t token_bytes, int num_groups, int num_max_tokens)
        : token_bytes(token_bytes), num_groups(num_groups), num_max_tokens(num_max_tokens) {}
    EP_HOST_DEVICE int64_t offset(int group, int token) const {
        return (static_cast<int64_t>(group) * num_max_tokens + token) * token_bytes;
    }
    EP_HOST_DEVICE int64_t num_bytes() const { return offset(num_groups, 0); }
};

// `[offset, offset + bytes)` lies inside the landing area `[0, area_bytes)` and obeys the bulk-copy rule (16-byte aligned
// start and size). Used by the bounds-checked build of the kernels (`EP_DEBUG`) and testable on the host.
EP_HOST_DEVICE bool landing_range_ok(int64_t offset, int64_t bytes, int64_t area_bytes) {
    return offset >= 0 and bytes > 0 and offset + bytes <= area_bytes and offset % kBulkAlignmentBytes == 0 and
           bytes % kBulkAlignmentBytes == 0;
}

// Count words that cross ranks carry the call's epoch in the high half so that nothing has to be
// cleared between calls: `[epoch:32 | value:32]`.
EP_HOST_DEVICE uint64_t pack_tagged(uint32_t epoch, uint32_t value) {
    return (static_cast<uint64_t>(epoch) << 32) | value;
}
EP_HOST_DEVICE uint32_t tagged_epoch(uint64_t w) { return static_cast<uint32_t>(w >> 32); }
EP_HOST_DEVICE uint32_t tagged_value(uint64_t w) { return static_cast<uint32_t>(w); }

struct EPSignals {
    CommonSignals common;
    // ---- local only ----
    unsigned int dispatch_epoch;    // epoch of the last completed dispatch issue kernel
    unsigned int combine_epoch;     // epoch of the last completed combine issue kernel
    unsigned int pad0[30];
    int send_expert_count[kMaxExperts];                 // this rank's per-expert histogram (self-cleaning)
    int cta_rank_count[kMaxCtas][kMaxRanks];            // dispatch layout pass 1
    int cta_expert_count[kMaxCtas][kMaxLocalExperts];   // expand epilogue pass 1
    // ---- written by peers ----
    alignas(128) unsigned long long recv_rank_count[kMaxRanks];                       // tagged
    alignas(128) unsigned long long recv_expert_count[kMaxRanks][kMaxLocalExperts];   // tagged
    alignas(128) unsigned long long dispatch_done[kMaxRanks];                          // epoch of the finished push
    alignas(128) unsigned long long combine_done[kMaxRanks];
};

// Mapped pinned host memory: the dispatch kernel publishes exact counts here for `do_cpu_sync`.
struct EPHostCounts {
    volatile unsigned long long num_recv_tokens;       // tagged
    volatile unsigned long long num_expanded_tokens;   // tagged (sum of aligned per-expert counts)
    volatile int aligned_recv_per_expert[kMaxLocalExperts];
    HostStatus status;
};

constexpr int64_t kEPWorkspaceBytes = math::align<int64_t>(sizeof(EPSignals), kNumAllocationAlignmentBytes);

}  // namespace deep_ep::layout
