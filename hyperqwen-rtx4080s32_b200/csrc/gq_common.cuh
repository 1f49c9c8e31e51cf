// Device helpers shared by the kernels: bounded mbarrier waits, bulk (TMA engine) copies, the legacy
// tensor-core MMA used by the small-batch path, and the bit tricks of the in-register dequantisers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>
#include "gq_layout.h"

// status codes returned by the C ABI (negative: rejected on the host before any launch)
#define GQ_OK 0
#define GQ_ERR_TYPE (-1)
#define GQ_ERR_SHAPE (-2)
#define GQ_ERR_ARG (-3)
#define GQ_ERR_WORKSPACE (-4)
#define GQ_ERR_CUDA (-5)
#define GQ_ERR_LIMIT (-6)
// device status word values (positive)
#define GQ_DEV_TIMEOUT 1
#define GQ_DEV_BAD_SHAPE 2

#define GQ_SPIN_LIMIT (1u << 30)   // polls of a try_wait loop before a kernel gives up and reports GQ_DEV_TIMEOUT (the time limit ends it first)

namespace gq {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// one poll (the hardware may park the thread for a short, implementation-defined time before it answers)
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false if the phase did not complete within GQ_WAIT_LIMIT_NS (or GQ_SPIN_LIMIT polls, whichever ends
// first); the caller records the failure in the launch's status word and leaves.  No wait in this library spins
// without a limit.  The limit is wall time, and generous, because under programmatic dependent launch a consumer
// may already be waiting while the kernel in front of this one still runs.
#define GQ_WAIT_LIMIT_NS 4000000000ull
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t i = 0; i < GQ_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && global_timer_ns() - t0 > GQ_WAIT_LIMIT_NS) return false;
    }
    return false;
}

// The same for a thread that expects to wait long and has nothing else to do (the producer of a stage ring waiting
// for a free stage): each poll carries a suspend-time hint, so the hardware parks the thread until the phase completes
// or the hint runs out, and a failed poll is followed by a short sleep — a waiting producer then costs a handful of
// issue slots per k-block instead of one poll every few cycles.
__device__ __forceinline__ bool mbar_wait_parked(uint64_t *bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    uint64_t t0 = 0;
    for (uint32_t i = 0; i < GQ_SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok)
            : "r"(addr), "r"(parity), "r"(20000u)
            : "memory");
        if (ok) return true;
        __nanosleep(64);
        if ((i & 63u) == 63u) {
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > GQ_WAIT_LIMIT_NS) return false;
        }
    }
    return false;
}

// ---- bulk copy global -> shared, completion counted on an mbarrier (bytes a multiple of 16, both
// addresses 16-byte aligned) -------------------------------------------------------------------
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ask the L2 to fetch `bytes` (a multiple of 16) starting at a 16-byte aligned global address; returns at once
__device__ __forceinline__ void prefetch_l2_bulk(const void *gptr, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gptr), "r"(bytes) : "memory");
}

// ---- programmatic dependent launch: a kernel launched with the stream-serialization attribute may start while
// its predecessor in the stream still runs; pdl_wait() returns once the predecessor has completed and its
// writes are visible, pdl_trigger() lets the successor start launching ----------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- thread-block cluster: barrier over all threads of all CTAs of the cluster, and loads from a peer CTA's
// shared memory (distributed shared memory) ----------------------------------------------------------------
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the two halves of a cluster barrier, for a rendezvous that is entered early and only collected when it is needed
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `smem_addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// ---- mma.sync m16n8k16, f16 x f16 -> f32 -----------------------------------------------------
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// d = a . b + z with z a quad the caller keeps at zero for the whole kernel (no per-use clearing of d)
__device__ __forceinline__ void mma16816_z(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const float (&z)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(z[0]), "f"(z[1]), "f"(z[2]), "f"(z[3]));
}

// ---- bit tricks (host fallbacks let the decoders be exercised lane by lane on a CPU) --------------
GQ_HD inline uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#ifdef __CUDA_ARCH__
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
#else
    uint64_t v = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        uint32_t s = (sel >> (4 * i)) & 0xF;
        uint32_t byte = (uint32_t)(v >> (8 * (s & 7))) & 0xFF;
        if (s & 8) byte = (byte & 0x80) ? 0xFF : 0x00;
        r |= byte << (8 * i);
    }
    return r;
#endif
}
template <int LUT>
GQ_HD inline uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
#ifdef __CUDA_ARCH__
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return r;
#else
    uint32_t r = 0;
    for (int i = 0; i < 32; ++i) {
        int idx = (((a >> i) & 1) << 2) | (((b >> i) & 1) << 1) | ((c >> i) & 1);
        r |= (uint32_t)((LUT >> idx) & 1) << i;
    }
    return r;
#endif
}
// (a & b) | c
GQ_HD inline uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) { return lop3<(0xF0 & 0xCC) | 0xAA>(a, b, c); }
// a | (b & c)
GQ_HD inline uint32_t or_and(uint32_t a, uint32_t b, uint32_t c) { return lop3<0xF0 | (0xCC & 0xAA)>(a, b, c); }
// a ^ (b & c)
GQ_HD inline uint32_t xor_and(uint32_t a, uint32_t b, uint32_t c) { return lop3<0xF0 ^ (0xCC & 0xAA)>(a, b, c); }
// shift left by a compile-time amount that may be negative (then a right shift)
template <int S>
GQ_HD inline uint32_t shl_c(uint32_t x) {
    if constexpr (S >= 0) return x << S; else return x >> (-S);
}

GQ_HD inline uint32_t h2_as_u32(__half2 h) { uint32_t u; memcpy(&u, &h, 4); return u; }
GQ_HD inline __half2 u32_as_h2(uint32_t u) { __half2 h; memcpy(&h, &u, 4); return h; }
GQ_HD inline float f16lo(uint32_t u) { return __low2float(u32_as_h2(u)); }
GQ_HD inline float f16hi(uint32_t u) { return __high2float(u32_as_h2(u)); }
GQ_HD inline float f16bits(uint32_t u16) { return f16lo(u16 & 0xFFFFu); }
GQ_HD inline float u32_as_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
// byte `j` (0..3) of `word` as a float, minus `off`: the byte is dropped into the mantissa of 2^23 (one prmt)
// and the constant removed by one add — no integer-to-float conversion instruction
template <int J>
GQ_HD inline float byte_f32(uint32_t word, float off = 0.0f) {
    return u32_as_f32(prmt(word, 0x4B000000u, 0x7440u | J)) - (8388608.0f + off);
}
GQ_HD inline uint32_t hmul2(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
    return h2_as_u32(__hmul2(u32_as_h2(a), u32_as_h2(b)));
#else
    return h2_as_u32(__floats2half2_rn(f16lo(a) * f16lo(b), f16hi(a) * f16hi(b)));
#endif
}
// packed fp16 arithmetic on raw 32-bit registers; every use in the decoders has an exactly representable result
GQ_HD inline uint32_t hsub2(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
    return h2_as_u32(__hsub2(u32_as_h2(a), u32_as_h2(b)));
#else
    return h2_as_u32(__floats2half2_rn(f16lo(a) - f16lo(b), f16hi(a) - f16hi(b)));
#endif
}
GQ_HD inline uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
#ifdef __CUDA_ARCH__
    return h2_as_u32(__hfma2(u32_as_h2(a), u32_as_h2(b), u32_as_h2(c)));
#else
    double lo = (double)f16lo(a) * (double)f16lo(b) + (double)f16lo(c);
    double hi = (double)f16hi(a) * (double)f16hi(b) + (double)f16hi(c);
    return h2_as_u32(__floats2half2_rn((float)lo, (float)hi));
#endif
}
// rotate right by n (0..31), and the number of set bits: device instructions with a host restatement
GQ_HD inline uint32_t rotr32(uint32_t w, int n) {
#ifdef __CUDA_ARCH__
    return __funnelshift_r(w, w, n);
#else
    n &= 31;
    return n ? (w >> n) | (w << (32 - n)) : w;
#endif
}
GQ_HD inline uint32_t popc32(uint32_t w) {
#ifdef __CUDA_ARCH__
    return (uint32_t)__popc(w);
#else
    uint32_t c = 0;
    for (; w; w &= w - 1) ++c;
    return c;
#endif
}
// a 16-bit fp16 constant in both halves
GQ_HD constexpr uint32_t h2c(uint32_t h16) { return h16 | (h16 << 16); }

#define GQ_MAGIC 0x64006400u    // fp16 (1024, 1024): an integer in the low mantissa bits reads as 1024 + it
#define GQ_MAGIC64 0x54005400u  // fp16 (64, 64): an integer in mantissa bits 4.. reads as 64 + it
#define GQ_MAGICB 0x64646464u   // the same high byte in every byte, for prmt (any index 4..7 of the second operand)

}  // namespace gq
