// Workspace of the pipeline-parallel buffer (reference: `layout/pp/workspace.hpp:8-14`):
// per direction, counters of sends issued, receives completed, arrivals seen and credits returned.
#pragma once

#include "signals.hpp"

namespace deep_ep::layout {

// Direction index: 0 = peer is my next rank, 1 = peer is my previous rank.
struct PPSignals {
    CommonSignals common;
    // ---- local only ----
    unsigned long long send_count[2];     // messages I have sent towards direction d
    unsigned long long recv_count[2];     // messages I have consumed from direction d
    unsigned long long pad[12];
    // ---- written by peers ----
    alignas(128) unsigned long long arrival[2];   // messages landed in my slots from direction d
    alignas(128) unsigned long long release[2];   // slots the peer in direction d has freed
};

constexpr int64_t kPPWorkspaceBytes = math::align<int64_t>(sizeof(PPSignals), kNumAllocationAlignmentBytes);

}  // namespace deep_ep::layout
