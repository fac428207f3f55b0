// Engram buffer configuration shared by host and kernel (reference: `layout/engram/workspace.hpp:7-37`).
#pragma once

#include "signals.hpp"

namespace deep_ep::layout {

constexpr int kMaxEngramLayers = 64;

struct EngramSignals {
    CommonSignals common;
};

// Per-layer table placement inside each rank's storage shard.
struct EngramLayerTable {
    int num_layers;
    int64_t storage_offset[kMaxEngramLayers];    // byte offset of the layer's `[entries, hidden]` shard
    int64_t sf_offset[kMaxEngramLayers];         // byte offset of the layer's SF shard (`[entries, packs]`)
    int num_entries_per_rank[kMaxEngramLayers];
};

constexpr int64_t kEngramWorkspaceBytes = math::align<int64_t>(sizeof(EngramSignals), kNumAllocationAlignmentBytes);

}  // namespace deep_ep::layout
