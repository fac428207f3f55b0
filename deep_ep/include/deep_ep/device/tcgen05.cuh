// Inline-PTX wrappers for the fifth-generation tensor cores of sm_100a: tensor-memory allocation,
// `tcgen05.mma` issued by one thread, commit-to-mbarrier, tensor-memory loads for the epilogue, the
// shared-memory matrix descriptors and the tiled TMA load that feeds them. Every TMA load here is
// CTA-local (no cluster multicast).
#pragma once

#include <cuda.h>

#include "ptx.cuh"

namespace deep_ep::tc {

// ---------------------------------------------------------------- tensor memory
// Executed by one full warp. Writes the base address (lane 0, first column) to `smem_slot`.
EP_DEVICE void tmem_alloc(uint32_t* smem_slot, uint32_t num_columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(ptx::smem_addr(smem_slot)), "r"(num_columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
EP_DEVICE void tmem_dealloc(uint32_t tmem_base, uint32_t num_columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(num_columns) : "memory");
}
EP_DEVICE void fence_before_thread_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
EP_DEVICE void fence_after_thread_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
EP_DEVICE void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives row (lane base + t).
EP_DEVICE void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

// ---------------------------------------------------------------- MMA
// Instruction descriptor of kind::f16 / kind::f8f6f4: fp32 accumulation, dense, no negation.
//   [4,6) D format (1 = F32)   [7,10) A format   [10,13) B format   [15] A major   [16] B major (0 = K, 1 = MN)
//   [17,23) N >> 3             [24,29) M >> 4
constexpr uint32_t kFormatBF16 = 1, kFormatE4M3 = 0;
EP_HOST_DEVICE constexpr uint32_t make_idesc(uint32_t ab_format, int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
           (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle, tile base aligned to 1024 bytes.
//   [0,14) address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version = 1   [61,64) layout = 2 (SWIZZLE_128B)
// K-major tile (rows of 128 bytes along K): 8-row groups are `stride` = 1024 bytes apart; the leading
// offset is unused. MN-major tile (rows of 128 bytes along M/N, one row per K index): 8 K-rows form a
// 1024-byte atom, atoms along K are `stride` bytes apart, 64-element blocks along M/N are `leading` bytes apart.
EP_DEVICE uint64_t make_smem_desc(const void* smem_ptr, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t desc = 0;
    desc |= uint64_t((ptx::smem_addr(smem_ptr) & 0x3ffff) >> 4);
    desc |= uint64_t(leading_bytes >> 4) << 16;
    desc |= uint64_t(stride_bytes >> 4) << 32;
    desc |= uint64_t(1) << 46;
    desc |= uint64_t(2) << 61;
    return desc;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
EP_DEVICE void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
EP_DEVICE void mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
// ---------------------------------------------------------------- block-scaled MMA (kind::mxf8f6f4)
// D[tmem] (+)= (A * SFA) * (B * SFB): one UE8M0 (power of two) scale per row of A and per column of B for the 32
// K elements of the instruction, read from tensor memory. Scale layout in tensor memory, for a tile of 128 rows: lane
// r % 32 (replicated in all four lane quarters), 32-bit column r / 32, and inside the column the byte chosen by the
// instruction descriptor's scale id (0..3); 256 columns of B therefore take eight tensor-memory columns.
// Instruction descriptor: as for kind::f8f6f4 without the D format field, plus
//   [4,6) scale id of B   [23] scale type (1 = UE8M0)   [29,31) scale id of A
EP_HOST_DEVICE constexpr uint32_t make_idesc_block_scaled(uint32_t ab_format, int m, int n, uint32_t sf_id_a, uint32_t sf_id_b) {
    return (sf_id_b << 4) | (ab_format << 7) | (ab_format << 10) | (uint32_t(n >> 3) << 17) | (1u << 23) |
           (uint32_t(m >> 4) << 24) | (sf_id_a << 29);
}
EP_DEVICE void mma_mxf8_block_scaled(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                     uint32_t tmem_sfa, uint32_t tmem_sfb, bool accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(uint32_t(accumulate)), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
// Shared-memory descriptor of an unswizzled K-major matrix of 16-byte rows: 8 consecutive rows form a 128-byte core
// matrix, core matrices follow each other every `stride_bytes`.
EP_DEVICE uint64_t make_smem_desc_noswizzle(const void* smem_ptr, uint32_t stride_bytes) {
    uint64_t desc = 0;
    desc |= uint64_t((ptx::smem_addr(smem_ptr) & 0x3ffff) >> 4);
    desc |= uint64_t(stride_bytes >> 4) << 32;
    desc |= uint64_t(1) << 46;
    return desc;
}
// Copies 32 rows x 16 bytes of shared memory into 4 tensor-memory columns of lanes 0..31 and replicates them into the
// other three lane quarters (the layout scale factors need). Asynchronous; ordered before later MMAs of this thread.
EP_DEVICE void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
EP_DEVICE void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(ptx::smem_addr(bar)) : "memory");
}

// ---------------------------------------------------------------- tiled TMA load (2-D, CTA-local)
// `x` is the innermost coordinate; x * element size must be a multiple of 16 bytes.
EP_DEVICE void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(ptx::smem_addr(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(ptx::smem_addr(bar)) : "memory");
}
// Tiled 2-D store of a shared-memory box to global memory, and the same as an element-wise add into global memory
// (the element type comes from the tensor map). Tracked by the issuing thread's bulk async-group. `x * element size`
// must be a multiple of 16 bytes and no coordinate may be negative.
EP_DEVICE void tma_store_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(ptx::smem_addr(smem_src)) : "memory");
}
EP_DEVICE void tma_reduce_add_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(ptx::smem_addr(smem_src)) : "memory");
}
EP_DEVICE void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2i and 2i + 1) share one MMA: the even CTA issues it, each CTA supplies its half of
// A (128 of the 256 rows) and its half of B (128 of the 256 columns) from its own shared memory at identical offsets,
// and each CTA's tensor memory receives its 128 rows of the accumulator.
EP_DEVICE uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
EP_DEVICE void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_ptr`'s counterpart in CTA `rank` of this cluster
EP_DEVICE uint32_t map_to_cta(const void* local_ptr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(ptx::smem_addr(local_ptr)), "r"(rank));
    return out;
}
EP_DEVICE void mbarrier_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
EP_DEVICE void tmem_alloc_pair(uint32_t* smem_slot, uint32_t num_columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(ptx::smem_addr(smem_slot)), "r"(num_columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
EP_DEVICE void tmem_dealloc_pair(uint32_t tmem_base, uint32_t num_columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(num_columns) : "memory");
}
EP_DEVICE void mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
// One arrival on the mbarrier at the same shared-memory offset in BOTH CTAs of the pair when all MMAs issued so far
// have completed (the commit, not a load, is what is multicast here).
EP_DEVICE void commit_pair(uint64_t* bar) {
    const uint16_t mask = 0x3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(ptx::smem_addr(bar)), "h"(mask) : "memory");
}
// Tiled 2-D load whose completion bytes are counted on the mbarrier of the pair's even CTA (`leader_bar_addr` is a
// shared::cluster address). The data lands in the executing CTA's own shared memory; nothing is multicast.
EP_DEVICE void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(ptx::smem_addr(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(leader_bar_addr) : "memory");
}

}  // namespace deep_ep::tc
