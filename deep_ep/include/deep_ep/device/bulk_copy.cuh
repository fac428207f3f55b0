// Warp-level bulk copier: moves a byte range from local or peer memory to one or several destinations through
// a small shared-memory ring with the TMA engine (`cp.async.bulk` load, then one `cp.async.bulk` store per
// destination). A warp keeps `kStages` chunks in flight and spends almost no issue slots, so a handful of CTAs
// saturates an NVLink port. All addresses and sizes must be multiples of 16 bytes.
#pragma once

#include "ptx.cuh"

namespace deep_ep::dev {

constexpr int kCopyChunkBytes = 8192;
constexpr int kCopyStages = 2;

EP_HOST_DEVICE constexpr int64_t bulk_copy_smem_bytes(int num_warps) {
    return int64_t(num_warps) * kCopyStages * kCopyChunkBytes + int64_t(num_warps) * kCopyStages * 8 + 256;
}

struct WarpCopier {
    uint8_t* ring;        // this warp's kCopyStages chunks
    uint64_t* bars;       // this warp's kCopyStages mbarriers
    int issued;           // chunks issued so far by this warp (ring position / phase)
    bool failed;

    // `smem` is the CTA's dynamic shared memory; call from every thread, followed by __syncthreads().
    EP_DEVICE void init(uint8_t* smem, int num_warps, int warp, int lane) {
        uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 127) & ~uintptr_t(127));
        ring = base + int64_t(warp) * kCopyStages * kCopyChunkBytes;
        bars = reinterpret_cast<uint64_t*>(base + int64_t(num_warps) * kCopyStages * kCopyChunkBytes) + warp * kCopyStages;
        issued = 0, failed = false;
        if (lane == 0) {
            for (int s = 0; s < kCopyStages; ++s) ptx::mbarrier_init(&bars[s], 1);
            ptx::fence_mbarrier_init();
        }
        __syncwarp();
    }

    // Copy `bytes` (<= kCopyChunkBytes, multiple of 16) from `src` to `num_dsts` destinations given by `dst_of(i)`.
    template <typename DstOf>
    EP_DEVICE void copy_chunk(const uint8_t* src, int bytes, int num_dsts, DstOf dst_of, int lane) {
        const int s = issued % kCopyStages;
        // the stage was last read by the stores issued kCopyStages chunks ago
        ptx::bulk_wait_read<kCopyStages - 1>();
        __syncwarp();
        if (lane == 0) {
            ptx::mbarrier_arrive_expect_tx(&bars[s], bytes);
            ptx::bulk_load(ring + s * kCopyChunkBytes, src, bytes, &bars[s]);
        }
        if (not ptx::mbarrier_wait(&bars[s], (issued / kCopyStages) & 1)) failed = true;
        for (int d = lane; d < num_dsts; d += 32) ptx::bulk_store(dst_of(d), ring + s * kCopyChunkBytes, bytes);
        ptx::bulk_commit();
        ++issued;
    }

    // All stores of this thread have been performed; call before signalling completion to anyone.
    EP_DEVICE void drain() {
        ptx::bulk_wait<0>();
        ptx::fence_proxy_async();
    }
};

}  // namespace deep_ep::dev
