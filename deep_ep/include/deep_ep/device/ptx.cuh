// Thin inline-PTX wrappers for sm_100a: system-scope acquire/release accesses on peer memory,
// mbarriers, and the non-tensor TMA (`cp.async.bulk`) copies in both directions. No load in this
// file carries a cluster-multicast qualifier: every bulk load is CTA-local.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../common/compiled.hpp"

namespace deep_ep::ptx {

// ---------------------------------------------------------------- scoped loads / stores / atomics
EP_DEVICE unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
EP_DEVICE unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
EP_DEVICE int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
EP_DEVICE unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
EP_DEVICE int ld_relaxed_gpu(const int* p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
EP_DEVICE void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
EP_DEVICE void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
EP_DEVICE void st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
EP_DEVICE void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
EP_DEVICE unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
EP_DEVICE void red_add_release_sys(int* p, int v) {
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
EP_DEVICE void red_add_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
EP_DEVICE void red_add_relaxed_sys(int* p, int v) {
    asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
EP_DEVICE void red_xor_relaxed_sys(unsigned int* p, unsigned int v) {
    asm volatile("red.relaxed.sys.global.xor.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
EP_DEVICE void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
EP_DEVICE void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// Orders generic-proxy accesses (ordinary ld/st) against async-proxy accesses (bulk copies).
EP_DEVICE void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
EP_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16-byte vector accesses; `nc` variant only for data that no one writes during the kernel.
EP_DEVICE int4 ld_nc_v4(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
EP_DEVICE int4 ld_v4(const void* p) {
    int4 v;
    asm volatile("ld.global.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
EP_DEVICE void st_v4(void* p, const int4& v) {
    asm volatile("st.global.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Streaming store: written once, not re-read by this kernel.
EP_DEVICE void st_na_v4(void* p, const int4& v) {
    asm volatile("st.global.L1::no_allocate.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

EP_DEVICE unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
EP_DEVICE int lane_id() {
    int l;
    asm("mov.s32 %0, %%laneid;" : "=r"(l));
    return l;
}
EP_DEVICE unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}
EP_DEVICE void named_barrier(int id, int num_threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(num_threads) : "memory");
}

// ---------------------------------------------------------------- mbarrier
EP_DEVICE uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

EP_DEVICE void mbarrier_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
EP_DEVICE void mbarrier_inval(uint64_t* bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
EP_DEVICE void fence_mbarrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
EP_DEVICE void mbarrier_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
EP_DEVICE void mbarrier_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
EP_DEVICE bool mbarrier_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if the phase did not complete within `max_polls` polls or within `max_ns` of wall time,
// whichever comes first (each poll itself blocks for a hardware-defined short interval, so the poll count alone
// does not bound the time).
EP_DEVICE bool mbarrier_wait(uint64_t* bar, uint32_t parity, int max_polls = 1 << 20, unsigned long long max_ns = 10000000000ull) {
    unsigned long long start = 0;
    for (int i = 0; i < max_polls; ++i) {
        if (mbarrier_try_wait(bar, parity)) return true;
        if ((i & 63) == 63) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > max_ns) return false;
        }
    }
    return false;
}

// ---------------------------------------------------------------- bulk (non-tensor TMA) copies
// global -> this CTA's shared memory, completion reported on an mbarrier. Addresses and size must be
// multiples of 16 bytes. The source may be local or a peer's memory.
EP_DEVICE void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// this CTA's shared memory -> global (local or peer), tracked by the thread's bulk async-group.
EP_DEVICE void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gmem_dst), "r"(smem_addr(smem_src)), "r"(bytes) : "memory");
}
EP_DEVICE void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's groups still have to *read* their shared-memory source.
template <int N>
EP_DEVICE void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// Wait until at most N of this thread's groups are not yet complete (writes performed).
template <int N>
EP_DEVICE void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// ---------------------------------------------------------------- small numeric helpers
EP_DEVICE float2 bf16x2_to_float2(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
EP_DEVICE uint32_t float2_to_bf16x2(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
// Smallest power of two >= x (x > 0, finite, normal) as a UE8M0 byte (value 2^(byte - 127)) and its exact reciprocal.
EP_DEVICE void ue8m0_ceil(float x, uint32_t& byte, float& inv) {
    const uint32_t bits = __float_as_uint(x);
    byte = min(max((bits >> 23) + ((bits & 0x7fffffu) != 0), 1u), 253u);
    inv = __uint_as_float((254u - byte) << 23);
}

// two fp32 -> two e4m3 (round-to-nearest-even, saturating), low byte = first argument
EP_DEVICE uint16_t float2_to_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
    return r;
}

}  // namespace deep_ep::ptx
