// Compile-time constants and host/device qualifiers shared by the host runtime (g++) and the
// sm_100a kernels (nvcc). Counterpart of the reference's `common/compiled.hpp:33-48`, re-sized for
// one NVSwitch domain of B200s.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define EP_HOST_DEVICE __host__ __device__ __forceinline__
#define EP_DEVICE __device__ __forceinline__
#else
#define EP_HOST_DEVICE inline
#define EP_DEVICE inline
#endif

namespace deep_ep {

constexpr int kMaxRanks = 64;             // peers addressable through one pointer table
constexpr int kMaxExperts = 2048;         // global experts
constexpr int kMaxLocalExperts = 1024;    // experts owned by one rank
constexpr int kMaxTopk = 32;              // one lane per top-k position
constexpr int kMaxCtas = 160;             // persistent CTAs per kernel (B200 has 148 SMs)
constexpr int kMaxContexts = 8;           // groups sharing one allocation
constexpr int kMaxBuckets = 64;           // tensors per batched all-gather

constexpr int64_t kNumAllocationAlignmentBytes = 2ll << 20;   // CUDA VMM granularity
constexpr int kNumRDMAAlignmentBytes = 32;                    // kept for API parity
constexpr int kNumTMAAlignmentBytes = 32;                     // API value; the hardware rule is 16
constexpr int kBulkAlignmentBytes = 16;                       // cp.async.bulk address/size rule

using topk_idx_t = int64_t;
using sf_pack_t = int16_t;                // scale factors travel as opaque 2-byte packs

// Error codes written to the status word by device code (0 = healthy).
enum StatusCode : int {
    kStatusOk = 0,
    kStatusBarrierTimeout = 1,
    kStatusGridSyncTimeout = 2,
    kStatusCountTimeout = 3,
    kStatusArrivalTimeout = 4,
    kStatusCreditTimeout = 5,
    kStatusBadArgument = 6,
    kStatusMbarrierTimeout = 7,
};

}  // namespace deep_ep
