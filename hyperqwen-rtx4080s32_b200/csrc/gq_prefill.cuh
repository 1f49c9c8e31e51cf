// Large-batch (prefill) path: fused dequantise -> shared memory -> tcgen05 MMA with the accumulator in tensor
// memory.  Replaces the reference's wide forms and its dequantise-then-cuBLAS path
// (gguf-plugin/gluon/interface.py:159-188, gguf-plugin/gluon/tiles.py:141-149): the dequantised weights never
// touch HBM.
//
// One CTA computes a 128 (weight rows: two 64-row tiles of the packed run) x NB (batch rows) output tile:
//   warp 0      producer of the activation operand: one bulk copy per 64-wide k-slice of a tile the preparation
//               kernel already stored in the MMA's shared-memory layout (K-major, 128-byte swizzle)
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected thread), commits to the stage barriers
//   warps 2-9   dequantisers: each owns a 16-row slab, reads its lane-ordered chunks straight from global memory,
//               turns them into fp16 weights (exact integer x fp16 scale, minus the fp16 minimum) and stores
//               them into the K-major swizzled A stage; afterwards they drain the accumulator (tcgen05.ld),
//               apply the activation row scale and store bf16.
// Weights sit on the MMA's M side (D rows = output features), batch rows on N, as in the small-batch kernel.
// With a split-K factor S > 1 (grid.z; for launches that would otherwise leave SMs without a CTA) a CTA walks one
// balanced part of the k-blocks and stores fp32 partial outputs, which sum_partials_kernel adds in split order.
// (Streaming the packed tiles through a shared-memory ring with bulk copies instead of loading them straight into
// registers one k-block ahead was measured 8-15 % slower at every batch size: the ring costs an A / B stage at 256
// batch rows, and the loads from it sit at the head of every k-block instead of overlapping the previous one.)
// Every wait is bounded; a wait that runs out sets the status word, and the CTA still frees its tensor memory.
#pragma once
#include "gq_decode.cuh"

// (included after the two __constant__ format tables c_iq3s_grid / c_iq3xxs_grid / c_iq2*_grid / c_iq4_kvalues are declared)
namespace gq {

#define GQ_PF_STAGES 4
#define GQ_PF_A_BYTES (128 * 128)            // 128 rows x 64 fp16
#define GQ_PF_DEQ_WARPS 8
#define GQ_PF_THREADS (32 * (2 + GQ_PF_DEQ_WARPS))

struct PrefillParams {
    const uint8_t *packed;
    const int32_t *desc;      // split-1 descriptor table: one row per 64-row tile
    int n_desc;
    const uint8_t *xp;        // [m_tile][K/64][NB rows][128 B]: fp16 activations in MMA layout
    const float *ex;          // [M] row scales
    __nv_bfloat16 *y;
    int64_t ldy;
    int M, K, nb;
    int *status;
    int split;                // split-K factor (grid.z); > 1: fp32 partials instead of y
    float *partials;          // [split][M][n_total]
    int64_t n_total;
    int cb_mask;              // the codebook types of the run (bit gq_cb_kind): their tables sit side by side in shared memory
};

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

template <int NB>
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    // instruction descriptor: D fp32, A and B fp16, both K-major, N = NB, M = 128
    constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | (8u << 24);
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- one 64-wide k-slice (run pairs 2J, 2J+1) of one slab: decode, scale, store into the A stage ----------
template <int TYPE, int P>
__device__ __forceinline__ void pf_store_pair(const Dec<TYPE> &dec, uint8_t *a_stage, int row0, int g, int t) {
    uint32_t a[2][4];
    dec.template pair<P>(a);
    float d0, d1;
    dec.kscale(d0, d1);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        float s0, s1, m0 = 0.f, m1 = 0.f;
        if constexpr (Dec<TYPE>::GROUP == 32) {
            dec.template scale<P>(s0, s1);
            if constexpr (Dec<TYPE>::HAS_MIN) dec.template minterm<P>(m0, m1);
        } else {
            if (u == 0) { dec.template scale<2 * P>(s0, s1); if constexpr (Dec<TYPE>::HAS_MIN) dec.template minterm<2 * P>(m0, m1); }
            else { dec.template scale<2 * P + 1>(s0, s1); if constexpr (Dec<TYPE>::HAS_MIN) dec.template minterm<2 * P + 1>(m0, m1); }
        }
        const uint32_t sc[2] = {h2_as_u32(__float2half2_rn(s0 * d0)), h2_as_u32(__float2half2_rn(s1 * d1))};
        const uint32_t mn[2] = {h2_as_u32(__float2half2_rn(-m0)), h2_as_u32(__float2half2_rn(-m1))};
        constexpr float off = Dec<TYPE>::template offs<2 * P>();   // both runs of a pair share the field position
        constexpr int chunk0 = 4 * (P & 1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t w01 = a[u][h], w23 = a[u][2 + h];
            if constexpr (off != 0.0f) { w01 = hsub2(w01, h2k(off)); w23 = hsub2(w23, h2k(off)); }
            if constexpr (Dec<TYPE>::HAS_MIN) { w01 = hfma2(w01, sc[h], mn[h]); w23 = hfma2(w23, sc[h], mn[h]); }
            else { w01 = hmul2(w01, sc[h]); w23 = hmul2(w23, sc[h]); }
            // A-tile row of weight row g + 8h of the slab: 2g + h.  Interleaving the two rows a lane owns gives the
            // sixteen lanes of a half-warp (g = 0..3 or 4..7, one h) four different swizzle phases, so their 8-byte
            // stores hit all 32 banks once; with row = g + 8h rows g and g + 8 shared a phase (2-way conflicts)
            const int row = row0 + 2 * g + h;
            const int chunk = chunk0 + 2 * u + (t >> 1);
            uint8_t *dst = a_stage + row * 128 + ((chunk ^ (row & 7)) << 4) + ((t & 1) << 3);
            *reinterpret_cast<uint2 *>(dst) = make_uint2(w01, w23);
        }
    }
}

// the dequantiser loop of one warp for a tile of TYPE: for every k-block, four k-slices through the stage ring
template <int TYPE>
__device__ __forceinline__ bool pf_dequant(const uint8_t *tile_base, int slab, int row0, int nb, uint8_t *smem_a0, int stage_bytes,   // tile_base: first k-block of this CTA's part
                                           uint64_t *a_full, uint64_t *freeb, const DecAux &aux, int lane) {
    const int Bt = gq_type_bytes(TYPE);
    const int g = lane >> 2, t = lane & 3;
    int st = 0, round = 0;
    Dec<TYPE> nxt;
    nxt.load(tile_base + slab * 16 * Bt, lane, aux);
    for (int kb = 0; kb < nb; ++kb) {
        Dec<TYPE> cur = nxt;
        if (kb + 1 < nb) nxt.load(tile_base + (int64_t)(kb + 1) * 64 * Bt + slab * 16 * Bt, lane, aux);
#define GQ_PF_SLICE(J)                                                                                   \
        {                                                                                                \
            if (round > 0 && !mbar_wait(freeb + st, (round - 1) & 1)) return false;                     \
            uint8_t *a_stage = smem_a0 + (size_t)st * stage_bytes;                                       \
            pf_store_pair<TYPE, 2 * (J)>(cur, a_stage, row0, g, t);                                      \
            pf_store_pair<TYPE, 2 * (J) + 1>(cur, a_stage, row0, g, t);                                  \
            fence_proxy_async();                                                                         \
            __syncwarp();                                                                                \
            if (lane == 0) mbar_arrive(a_full + st);                                                     \
            if (++st == GQ_PF_STAGES) { st = 0; ++round; }                                               \
        }
        GQ_PF_SLICE(0) GQ_PF_SLICE(1) GQ_PF_SLICE(2) GQ_PF_SLICE(3)
#undef GQ_PF_SLICE
    }
    return true;
}

// a slab with no tile behind it (odd number of tiles in the run): its rows stay zero; it only keeps the barriers moving
__device__ __forceinline__ bool pf_idle(int nb, uint64_t *a_full, uint64_t *freeb, int lane) {
    int st = 0, round = 0;
    for (int i = 0; i < 4 * nb; ++i) {
        if (round > 0 && !mbar_wait(freeb + st, (round - 1) & 1)) return false;
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full + st);
        if (++st == GQ_PF_STAGES) { st = 0; ++round; }
    }
    return true;
}

template <int NB, bool SPLITK>
__global__ void __launch_bounds__(GQ_PF_THREADS, NB <= 64 ? 2 : 1) gemm_prefill_kernel(const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // layout: [stages x (A 16 KB | B NB*128)] [barriers] [tmem slot] [codebook tables of the run's types]
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int B_BYTES = NB * 128;
    constexpr int STAGE = GQ_PF_A_BYTES + B_BYTES;
    uint64_t *a_full = reinterpret_cast<uint64_t *>(smem + GQ_PF_STAGES * STAGE);
    uint64_t *b_full = a_full + GQ_PF_STAGES;
    uint64_t *freeb = b_full + GQ_PF_STAGES;
    uint64_t *done = freeb + GQ_PF_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(done + 1);
    uint2 *grid_s = reinterpret_cast<uint2 *>(smem + GQ_PF_STAGES * STAGE + 128);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = blockIdx.x, mt = blockIdx.y, z = SPLITK ? (int)blockIdx.z : 0;
    const int kb0 = SPLITK ? (int)(((int64_t)z * p.nb) / p.split) : 0, kb1 = SPLITK ? (int)(((int64_t)(z + 1) * p.nb) / p.split) : p.nb;
    const int nkb = kb1 - kb0, nslices = 4 * nkb;

    // the two 64-row tiles of this CTA
    const int32_t *d0 = p.desc + (int64_t)(2 * pair) * GQ_DESC_WORDS;
    const bool has1 = 2 * pair + 1 < p.n_desc;
    const int32_t *d1 = has1 ? d0 + GQ_DESC_WORDS : d0;

    // a codebook type the call's run_info did not announce has no table space: report and leave (nothing is allocated yet)
    {
        const int k0 = gq_cb_kind(d0[1]), k1 = gq_cb_kind(d1[1]);
        if ((k0 >= 0 && !((p.cb_mask >> k0) & 1)) || (k1 >= 0 && !((p.cb_mask >> k1) & 1))) {
            if (threadIdx.x == 0) { pdl_wait(); report_status(p.status, GQ_DEV_BAD_SHAPE); }      // after the preparation kernel has cleared the word
            return;
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < GQ_PF_STAGES; ++s) {
            mbar_init(a_full + s, GQ_PF_DEQ_WARPS);
            mbar_init(b_full + s, 1);
            mbar_init(freeb + s, 1);
        }
        mbar_init(done, 1);
        fence_barrier_init();
    }
    // the codebook tables of the two tiles' types, each at its place among the tables of the run's types
    for (int which = 0; which < 2; ++which) {
        const int ty = which ? d1[1] : d0[1], kind = gq_cb_kind(ty);
        if (kind < 0 || (which && d1[1] == d0[1])) continue;
        uint8_t *tb = reinterpret_cast<uint8_t *>(grid_s) + gq_cb_offset(p.cb_mask, kind);
        uint32_t *t32 = reinterpret_cast<uint32_t *>(tb);
        uint2 *t64 = reinterpret_cast<uint2 *>(tb);
        switch (ty) {
            case GQ_IQ3_S: for (int i = threadIdx.x; i < 512; i += blockDim.x) t64[i] = iq3s_grid_entry(c_iq3s_grid[i]); break;
            case GQ_IQ3_XXS: for (int i = threadIdx.x; i < 256; i += blockDim.x) t64[i] = iq3s_grid_entry(c_iq3xxs_grid[i]); break;
            case GQ_IQ2_XXS: for (int i = threadIdx.x; i < 512; i += blockDim.x) t32[i] = prmt(c_iq2xxs_grid[i], 0u, 0x3120u); break;
            case GQ_IQ2_XS: for (int i = threadIdx.x; i < 1024; i += blockDim.x) t32[i] = prmt(c_iq2xs_grid[i], 0u, 0x3120u); break;
            case GQ_IQ2_S: for (int i = threadIdx.x; i < 2048; i += blockDim.x) t32[i] = prmt(c_iq2s_grid[i], 0u, 0x3120u); break;
            case GQ_IQ1_M: for (int i = threadIdx.x; i < 4096; i += blockDim.x) t32[i] = prmt(c_iq1_grid[i], 0u, 0x3120u); break;
        }
    }
    if (!has1) {
        // rows 64..127 of every A stage are never written: clear them once
        for (int s = 0; s < GQ_PF_STAGES; ++s)
            for (int i = threadIdx.x; i < 64 * 128 / 16; i += blockDim.x)
                reinterpret_cast<uint4 *>(smem + (size_t)s * STAGE + 64 * 128)[i] = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)NB) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---- activation producer ----
        if (lane == 0) {
            const uint8_t *src = p.xp + ((int64_t)mt * (p.K / 64) + 4 * (int64_t)kb0) * B_BYTES;
            for (int i = 0, st = 0, round = 0; i < nslices; ++i) {
                if (round > 0 && !mbar_wait(freeb + st, (round - 1) & 1)) { ok = false; break; }
                mbar_expect_tx(b_full + st, B_BYTES);
                bulk_g2s(smem + (size_t)st * STAGE + GQ_PF_A_BYTES, src + (int64_t)i * B_BYTES, B_BYTES, b_full + st);
                if (++st == GQ_PF_STAGES) { st = 0; ++round; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            for (int i = 0, st = 0, round = 0; i < nslices; ++i) {
                if (!mbar_wait(a_full + st, round & 1) || !mbar_wait(b_full + st, round & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (size_t)st * STAGE);
                const uint64_t ad = umma_desc(a_addr), bd = umma_desc(a_addr + GQ_PF_A_BYTES);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) umma_f16<NB>(tmem_base, ad + 2 * kk, bd + 2 * kk, (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(freeb + st);          // the stage may be overwritten once these MMAs have read it
                if (++st == GQ_PF_STAGES) { st = 0; ++round; }
            }
            umma_commit(done);
        }
    } else {
        // ---- dequantisers, then epilogue ----
        const int slab = warp - 2;                 // 0..7: rows 16*slab .. 16*slab+15 of the 128
        const int32_t *dd = (slab < 4) ? d0 : d1;
        DecAux aux;
        aux.grid = reinterpret_cast<const uint2 *>(reinterpret_cast<const uint8_t *>(grid_s) + (gq_cb_kind(dd[1]) >= 0 ? gq_cb_offset(p.cb_mask, gq_cb_kind(dd[1])) : 0));
        {
            uint32_t tb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                tb[j] = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) tb[j] |= (uint32_t)(uint8_t)(c_iq4_kvalues[4 * j + i] + 128) << (8 * i);
            }
            aux.iq4 = {tb[0], tb[1], tb[2], tb[3]};
        }
        if (slab >= 4 && !has1) {
            ok = pf_idle(nkb, a_full, freeb, lane);
        } else {
            const uint8_t *tile_base = p.packed + (int64_t)dd[0] * 16 + (int64_t)kb0 * 64 * gq_type_bytes(dd[1]);
            const int sl = slab & 3, row0 = 16 * slab;
#define GQ_PF(T) case T: ok = pf_dequant<T>(tile_base, sl, row0, nkb, smem, STAGE, a_full, freeb, aux, lane); break;
            switch (dd[1]) {
                GQ_PF(GQ_Q4_0) GQ_PF(GQ_Q5_0) GQ_PF(GQ_Q8_0) GQ_PF(GQ_Q2_K) GQ_PF(GQ_Q3_K) GQ_PF(GQ_Q4_K)
                GQ_PF(GQ_Q5_K) GQ_PF(GQ_Q6_K) GQ_PF(GQ_IQ4_NL) GQ_PF(GQ_IQ3_S) GQ_PF(GQ_IQ4_XS) GQ_PF(GQ_IQ3_XXS)
                GQ_PF(GQ_IQ2_XXS) GQ_PF(GQ_IQ2_XS) GQ_PF(GQ_IQ2_S) GQ_PF(GQ_IQ1_M)
            }
#undef GQ_PF
        }
        if (ok && !mbar_wait(done, 0)) ok = false;
        tc_fence_after();
        if (ok) {
            // TMEM lane group of this warp = warp % 4; the two warps of a lane group split the NB columns
            const int lg = warp & 3, half = (warp - 2) >> 2;
            const int feat = 32 * lg + lane;                       // row of the 128-row tile pair
            const int32_t *dt = (feat < 64) ? d0 : d1;
            const int ra = feat & 63;                              // row of the A tile -> weight row of the packed tile
            const int r = (ra & ~15) | ((ra & 15) >> 1) | ((ra & 1) << 3);
            const bool row_ok = (feat < 64 || has1) && r < dt[3];
            const int64_t col = (int64_t)dt[2] + r;
#pragma unroll 1
            for (int c0 = half * (NB / 2); c0 < (half + 1) * (NB / 2); c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * lg) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int n = mt * NB + c0 + j;
                    if (row_ok && n < p.M) {
                        const float val = __uint_as_float(v[j]) * p.ex[n];
                        if constexpr (SPLITK) p.partials[((int64_t)z * p.M + n) * p.n_total + col] = val;
                        else p.y[(int64_t)n * p.ldy + col] = __float2bfloat16_rn(val);
                    }
                }
            }
        }
    }
    if (!ok) {
        // a bounded wait ran out: report it, and give copies and MMAs still in flight a bounded time to land
        if (lane == 0) report_status(p.status, GQ_DEV_TIMEOUT);
        for (int i = 0; i < 100; ++i) __nanosleep(10000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)NB) : "memory");
    }
}

// activation preparation for the prefill path: bf16 row -> fp16 scaled by an exact power of two, stored in the
// MMA's shared-memory layout (tiles of NB rows x 64 k, K-major, 16-byte chunks XOR-swizzled by row % 8) so the
// kernel's producer moves a whole k-slice with one bulk copy
template <int NB>
__global__ void __launch_bounds__(256) prep_x_prefill_kernel(const __nv_bfloat16 *__restrict__ x, int64_t ldx, int K, int M, float *__restrict__ ex,
                                                             uint8_t *__restrict__ xp, int *status) {
    __shared__ float red[8];
    __shared__ float s_scale;
    const int m = blockIdx.x;
    if (m == 0 && threadIdx.x == 0) *status = 0;
    const int mt = m / NB, r = m % NB;
    uint8_t *tile0 = xp + (int64_t)mt * (K / 64) * (NB * 128);
    if (m >= M) {
        // rows past the batch inside the last tile: zeros (their outputs are never stored)
        for (int c = threadIdx.x; c < K / 8; c += 256) {
            const int slice = c >> 3, chunk = c & 7;
            *reinterpret_cast<uint4 *>(tile0 + (int64_t)slice * (NB * 128) + r * 128 + ((chunk ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
        }
        return;
    }
    const __nv_bfloat16 *xr = x + (int64_t)m * ldx;
    float amax = 0.0f;
    for (int c = threadIdx.x; c < K / 8; c += 256) {
        const uint4 v = *reinterpret_cast<const uint4 *>(xr + 8 * c);
        const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(b[j]); amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y))); }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = red[0];
        for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
        int e = 9;
        if (a > 0.0f && a < 3.0e38f) { e = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127; if (e < -100) e = -100; }
        s_scale = __uint_as_float((uint32_t)(127 + 9 - e) << 23);
        ex[m] = __uint_as_float((uint32_t)(127 - 9 + e) << 23);
    }
    __syncthreads();
    const float scale = s_scale;
    for (int c = threadIdx.x; c < K / 8; c += 256) {
        const uint4 v = *reinterpret_cast<const uint4 *>(xr + 8 * c);
        const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&v);
        uint4 o;
        uint32_t *oo = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(b[j]); oo[j] = h2_as_u32(__floats2half2_rn(f.x * scale, f.y * scale)); }
        const int slice = c >> 3, chunk = c & 7;
        *reinterpret_cast<uint4 *>(tile0 + (int64_t)slice * (NB * 128) + r * 128 + ((chunk ^ (r & 7)) << 4)) = o;
    }
}

}  // namespace gq
