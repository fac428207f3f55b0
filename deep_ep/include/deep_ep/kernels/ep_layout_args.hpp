// Arguments and scratch block of the standalone dispatch-layout kernel (usable from g++ and nvcc).
#pragma once

#include "../layout/signals.hpp"

namespace deep_ep::kernels {

constexpr int kLayoutMaxCtas = 32;

// Scratch memory of the layout kernel: grid-sync words, per-CTA rank counts and the expert histogram.
// Must be zero before the first launch; the kernel leaves it zeroed again where that is required.
struct LayoutScratch {
    layout::CommonSignals sync;                         // grid_count / grid_gen / status
    int cta_rank_count[kLayoutMaxCtas][kMaxRanks];      // fully rewritten by every launch
    int expert_count[kMaxExperts];                      // accumulated with atomics, cleared by the kernel after use
};

struct LayoutArgs {
    const int64_t* topk_idx;        // [T, k]
    int num_tokens, num_topk, num_experts, num_ranks;
    int* dst_slot_idx;              // [T, k] slot inside the destination rank's per-source region, -1 for duplicates / masked
    int* num_tokens_per_rank;       // [R] rank-deduplicated tokens sent to each rank
    int* num_tokens_per_expert;     // [E] selections per expert
    LayoutScratch* scratch;
    long long timeout_ns;
    int* status;                    // optional: receives a StatusCode when a bounded wait ran out
};

}  // namespace deep_ep::kernels
