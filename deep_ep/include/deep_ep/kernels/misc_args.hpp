// Plain-data argument blocks of the barrier, Engram, bucket all-gather and pipeline kernels
// (usable from g++ and nvcc).
#pragma once

#include "../layout/bucket.hpp"
#include "../layout/engram.hpp"
#include "../layout/pp.hpp"

namespace deep_ep::kernels {

struct BarrierArgs {
    layout::CommonSignals* cs;
    layout::HostStatus* host_status;
    layout::PeerTable peers;
    long long timeout_ns;
    int repeats;              // barriers executed by this launch (1 = a barrier; more = latency measurement)
};

struct EngramFetchArgs {
    layout::PeerTable peers;
    layout::EngramLayerTable table;   // offsets relative to each rank's allocation base
    const int* indices;               // [L, T, P]
    uint8_t* recv;                    // local receive region
    sf_pack_t* sf_out;                // [L][sf_layer_stride] backing, or nullptr
    int64_t sf_token_stride, sf_pack_stride, sf_layer_stride;
    int num_layers, num_tokens, num_entries_per_token, num_max_tokens;
    int hidden_bytes, num_sf_packs;
};

struct AllGatherArgs {
    layout::PeerTable peers;
    layout::BucketList list;
    layout::CommonSignals* cs;
    layout::HostStatus* host_status;
    long long timeout_ns;
    int use_multicast;                // 1: NVLS multimem.st through `peers.mc_base`
    int skip_local;                   // 1: the local shard is already in place
};

// Batched reduce-scatter / all-reduce over tensors that live at the same offset of every rank's symmetric allocation.
// `list.buckets[i] = {offset of the whole tensor, bytes of the whole tensor, unused}`; rank r owns the r-th of
// `num_ranks` equal shards of every tensor.
enum ReduceDtype : int { kReduceBF16 = 0, kReduceFP32 = 1, kReduceFP16 = 2 };
struct BucketReduceArgs {
    layout::PeerTable peers;
    layout::BucketList list;
    layout::CommonSignals* cs;
    layout::HostStatus* host_status;
    long long timeout_ns;
    int dtype[kMaxBuckets];           // ReduceDtype per bucket
    float scale;                      // applied to the fp32 sum before it is rounded to the tensor's dtype
    int all_reduce;                   // 0: the reduced shard stays on its owner; 1: it is also stored to every peer
    int use_multicast;                // 1: `multimem.ld_reduce` / `multimem.st` through `peers.mc_base` (the NVSwitch adds and
                                      //    broadcasts; the order of the additions is the switch's, not rank order)
};

struct PPArgs {
    layout::PeerTable peers;
    layout::PPSignals* ws;
    layout::HostStatus* host_status;
    uint8_t* x;                       // tensor to send from / receive into
    int64_t num_bytes;
    int64_t slot_bytes;               // aligned size of one ring slot
    int64_t storage_offset;           // ring storage offset inside the allocation
    int num_inflight;
    int peer;                         // destination (send) or source (recv) rank
    int direction;                    // 0: peer is my next rank, 1: peer is my previous rank
    long long timeout_ns;
};

constexpr int kMaxLBTensors = 16;

// Expert load balancing over redundant expert slots. `mapping[r * num_redundant + c]` is the global expert id
// that rank r keeps in its redundant slot c (-1 = empty); every rank passes the same mapping.
struct LBArgs {
    layout::PeerTable peers;
    layout::CommonSignals* cs;
    layout::HostStatus* host_status;
    long long timeout_ns;
    const int* mapping;
    int num_redundant, num_local_experts;
    int mode;                                 // 0: push weights into peers' redundant slots, 1: pull and add gradients
    int num_tensors;
    const uint8_t* src[kMaxLBTensors];        // mode 0: local `[num_local_experts, bytes_per_expert]` sources
    int64_t dst_offset[kMaxLBTensors];        // offset of the `[num_redundant, ...]` tensor inside the allocation
    int64_t bytes_per_expert[kMaxLBTensors];
    float* expert_grads;                      // mode 1: `[num_local_experts, hidden]` fp32, accumulated into
    int64_t hidden;
};

}  // namespace deep_ep::kernels
