// Bucket list passed by value to the batched all-gather kernel (reference: `comm/bucket.hpp:11-42`,
// `layout/bucket/workspace.hpp:7-13`).
#pragma once

#include "signals.hpp"

namespace deep_ep::layout {

struct Bucket {
    int64_t dst_offset;      // byte offset of the gathered tensor inside the symmetric allocation
    int64_t num_bytes;       // bytes of one rank's shard
    const uint8_t* src;      // this rank's shard (anywhere in device memory)
};

struct BucketList {
    int num_buckets;
    Bucket buckets[kMaxBuckets];
};

struct BucketSignals {
    CommonSignals common;
};

constexpr int64_t kBucketWorkspaceBytes = math::align<int64_t>(sizeof(BucketSignals), kNumAllocationAlignmentBytes);

}  // namespace deep_ep::layout
