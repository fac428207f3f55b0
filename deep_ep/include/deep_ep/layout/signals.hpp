// Per-context signal block at the start of every symmetric allocation, plus the peer pointer
// table handed to kernels by value. Role of the reference's `layout/common/signals.hpp:9-24`
// (`CommonSignals`, `get_sym_ptr`), laid out for NVLink peer mappings: every process maps every
// peer's allocation at a *different* virtual address, so the table is per process.
#pragma once

#include "../common/compiled.hpp"
#include "../common/math.hpp"

namespace deep_ep::layout {

// Base addresses of each rank's symmetric allocation as mapped in the calling process.
// `mc_base` is the NVLS multicast mapping of the same allocation (nullptr when unavailable).
struct PeerTable {
    uint8_t* base[kMaxRanks];
    uint8_t* mc_base;
    int rank;
    int num_ranks;

    template <typename T>
    EP_HOST_DEVICE T* at(int peer, int64_t byte_offset) const {
        return reinterpret_cast<T*>(base[peer] + byte_offset);
    }
    // Translate a pointer into this rank's allocation to the same offset on `peer`.
    template <typename T>
    EP_HOST_DEVICE T* sym(T* local_ptr, int peer) const {
        return reinterpret_cast<T*>(base[peer] + (reinterpret_cast<uint8_t*>(local_ptr) - base[rank]));
    }
};

// Written by device code when a bounded wait gives up; lives in mapped pinned host memory so the
// host can read it without touching the stream.
struct HostStatus {
    volatile int code;        // StatusCode
    volatile int rank;
    volatile int peer;        // rank waited for, or -1
    volatile int where;       // kernel-specific site id
    volatile long long expected;
    volatile long long observed;
};

struct alignas(128) CommonSignals {
    // ---- local only ----
    unsigned int grid_count;      // arrivals at the current grid-wide sync
    unsigned int grid_gen;        // generation of the grid-wide sync
    int barrier_counter;          // number of rank barriers executed so far (phase/sign source)
    int status;                   // sticky StatusCode; kernels exit early when non-zero
    unsigned int done_ctas;       // CTA completion counter of the running kernel
    unsigned int reserved[27];
    // ---- written by peers ----
    alignas(128) int barrier_signals[2];   // +-1 per rank per phase, never reset
    // One bit per rank and phase, toggled by that rank at every barrier of the phase (never reset either). Only read when a
    // barrier runs out of time: the ranks whose bit has not flipped are the ones that did not arrive.
    unsigned int barrier_arrived[2][kMaxRanks / 32];
    int reserved2[30 - 2 * (kMaxRanks / 32)];
};
static_assert(sizeof(CommonSignals) == 256, "CommonSignals must stay two cache lines");

}  // namespace deep_ep::layout
