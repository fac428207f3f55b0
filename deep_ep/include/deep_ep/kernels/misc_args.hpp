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

}  // namespace deep_ep::kernels
