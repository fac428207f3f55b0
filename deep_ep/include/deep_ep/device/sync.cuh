// Bounded waits, the sticky status word, the grid-wide sync of persistent kernels and the
// cross-rank barrier. Role of the reference's `comm/barrier.hpp:27-179` and `common/reduction.hpp`,
// with one difference that matters on shared GPUs: a wait that runs out records a status code and
// returns false; nothing traps.
#pragma once

#include "../layout/ep.hpp"
#include "../layout/signals.hpp"
#include "ptx.cuh"

namespace deep_ep::dev {

// Phase stamp for the optional kernel trace (one thread calls it per phase; no-op without a trace buffer).
EP_DEVICE void trace_point(unsigned long long* trace, int slot) {
    if (trace != nullptr) trace[slot] = ptx::globaltimer_ns();
}


struct Deadline {
    unsigned long long end_ns;
    EP_DEVICE explicit Deadline(long long timeout_ns) : end_ns(ptx::globaltimer_ns() + static_cast<unsigned long long>(timeout_ns)) {}
    EP_DEVICE bool expired() const { return ptx::globaltimer_ns() > end_ns; }
};

// Spin on `pred()` until true or the deadline passes; the timer is read every 128 polls.
template <typename Pred>
EP_DEVICE bool spin_until(const Deadline& deadline, Pred pred) {
    while (true) {
        #pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (pred()) return true;
        if (deadline.expired()) return pred();
    }
}

// First failure wins; details go to mapped host memory (may be nullptr).
EP_DEVICE void report_status(layout::CommonSignals* cs, layout::HostStatus* hs, int code, int rank, int peer,
                             int where, long long expected, long long observed) {
    if (atomicCAS(&cs->status, 0, code) == 0 and hs != nullptr) {
        hs->rank = rank, hs->peer = peer, hs->where = where;
        hs->expected = expected, hs->observed = observed;
        __threadfence_system();
        hs->code = code;
    }
}

// Bulk store of a message into the landing area of `peer` at `area_offset` bytes from the area's start. Kernels compiled
// with `-DEP_DEBUG` (the bounds-checked build: `EP_DEBUG=1` for `setup.py`, or for the run-time specialiser) first check
// that the destination lies inside the area and is 16-byte aligned; a store that fails the check is NOT issued, and the
// offending offset is recorded in the status word (`kStatusBadArgument`, `expected` = area size, `observed` = offset).
EP_DEVICE void store_message(layout::CommonSignals* cs, layout::HostStatus* hs, const layout::PeerTable& peers, int peer,
                             int64_t area_start, int64_t area_bytes, int64_t area_offset, const void* smem_src, uint32_t bytes,
                             int where) {
#ifdef EP_DEBUG
    if (peer < 0 or peer >= peers.num_ranks or not layout::landing_range_ok(area_offset, bytes, area_bytes)) {
        report_status(cs, hs, kStatusBadArgument, peers.rank, peer, where, area_bytes, area_offset);
        return;
    }
#else
    (void) cs, (void) hs, (void) area_bytes, (void) where;
#endif
    ptx::bulk_store(peers.base[peer] + area_start + area_offset, smem_src, bytes);
}

EP_DEVICE bool healthy(const layout::CommonSignals* cs) {
    return ptx::ld_relaxed_gpu(&cs->status) == 0;
}

// Grid-wide sync for kernels whose CTAs are all resident (cooperative launch). Returns false on
// timeout or when another CTA has already failed.
EP_DEVICE bool grid_sync(layout::CommonSignals* cs, layout::HostStatus* hs, int num_ctas, long long timeout_ns,
                         int rank, int where) {
    __shared__ int ok_smem;
    __syncthreads();
    if (threadIdx.x == 0) {
        bool ok = true;
        if (num_ctas > 1) {
            const unsigned gen = ptx::ld_acquire_gpu(&cs->grid_gen);
            __threadfence();
            if (atomicAdd(&cs->grid_count, 1u) == static_cast<unsigned>(num_ctas - 1)) {
                cs->grid_count = 0;
                __threadfence();
                ptx::st_release_gpu(&cs->grid_gen, gen + 1);
            } else {
                const Deadline deadline(timeout_ns);
                ok = spin_until(deadline, [&]() { return ptx::ld_acquire_gpu(&cs->grid_gen) != gen or not healthy(cs); });
                if (not ok)
                    report_status(cs, hs, kStatusGridSyncTimeout, rank, -1, where, gen + 1, cs->grid_gen);
            }
        }
        ok_smem = ok and healthy(cs);
    }
    __syncthreads();
    return ok_smem != 0;
}

// Cross-rank barrier executed by one warp of one CTA. Call n uses phase n&1 and sign +1/-1
// alternating every two calls, so the signal swings 0 -> N -> 0 and never needs a reset
// (the scheme of the reference's `comm/barrier.hpp:141-175`). All prior writes of the calling
// thread block that were ordered before this call (e.g. by `__syncthreads`) are released.
EP_DEVICE bool rank_barrier_warp(layout::CommonSignals* cs, layout::HostStatus* hs, const layout::PeerTable& peers,
                                 long long timeout_ns, int where) {
    const int lane = ptx::lane_id();
    int n = 0;
    if (lane == 0) n = cs->barrier_counter;
    n = __shfl_sync(0xffffffffu, n, 0);
    const int phase = n & 1, sign = (n & 2) ? -1 : 1;
    // One system-scope fence releases everything ordered before this call; the arrivals that follow it can then be relaxed
    // (fence + relaxed atomic is a release). A `red.release` per peer would repeat that fence once per lane, and each
    // system-scope fence waits for the acknowledgements of earlier remote writes, a round trip over the links.
    __threadfence_system();
    for (int r = lane; r < peers.num_ranks; r += 32) {
        layout::CommonSignals* peer = peers.sym(cs, r);
        // who arrived (looked at only when the wait below runs out), then the arrival itself
        ptx::red_xor_relaxed_sys(&peer->barrier_arrived[phase][peers.rank / 32], 1u << (peers.rank % 32));
        ptx::red_add_relaxed_sys(&peer->barrier_signals[phase], sign);
    }
    const int target = sign > 0 ? peers.num_ranks : 0;
    bool ok = true;
    if (lane == 0) {
        const Deadline deadline(timeout_ns);
        ok = spin_until(deadline, [&]() { return ptx::ld_acquire_sys(&cs->barrier_signals[phase]) == target; });
        if (not ok) {
            // every rank has toggled its bit (n >> 1) + 1 times once it has arrived at this barrier of the phase: the
            // first rank whose bit still has the old value is named in the report
            const unsigned arrived_value = ((n >> 1) + 1) & 1;
            int absent = -1;
            for (int r = 0; r < peers.num_ranks and absent < 0; ++r)
                if (((ptx::ld_acquire_sys(&cs->barrier_arrived[phase][r / 32]) >> (r % 32)) & 1u) != arrived_value) absent = r;
            report_status(cs, hs, kStatusBarrierTimeout, peers.rank, absent, where, target, cs->barrier_signals[phase]);
        }
        cs->barrier_counter = n + 1;
    }
    // lane 0's acquire load of the completed count orders the peers' released writes before everything after the barrier;
    // the shuffle hands that order to the other lanes, the caller's block-wide sync to the other warps
    ok = __shfl_sync(0xffffffffu, ok, 0);
    ptx::fence_acq_rel_gpu();
    return ok;
}

}  // namespace deep_ep::dev
