// In-register dequantisers of the eleven GGML types, from the lane-ordered slab layout (gq_layout.h) to
// m16n8k16 A-operand fragments.
//
// A slab is 16 output rows x 256 weights.  Lane l = 4*g + t of the warp owns, for rows g and g+8, the four
// weights 16*r + 4*t + {0,1,2,3} of every 16-weight run r.  The MMA of run r takes
//     a[0] = (row g,   k = 4t+0, 4t+1)   a[1] = (row g+8, k = 4t+0, 4t+1)
//     a[2] = (row g,   k = 4t+2, 4t+3)   a[3] = (row g+8, k = 4t+2, 4t+3)
// as packed fp16 pairs, against the B fragment {x[n][16r+4t], x[n][16r+4t+1]}, {x[n][16r+4t+2], x[n][16r+4t+3]}
// (the k order inside an MMA is free as long as A and B agree, so activations stay in natural order).
//
// Every decoder produces the EXACT integer value of the quantised weight (q minus its offset, or the
// codebook / grid entry with its sign) as fp16 — all of them are below 2048 in magnitude — and hands the
// scale out separately: an integer (or fp16 d) per 16- or 32-weight group applied to the fp32 MMA result,
// and the row's fp16 d per k-block.  The minimum term of Q2_K / Q4_K / Q5_K is an extra MMA of the integer
// mins against per-run activation sums.  The value arithmetic follows the formats as the reference states
// them (gguf-plugin/gluon/kq_ref.py:17-79, q2k.py:5-12, q4k.py:5-10, iq3s_int8t.py:4-11, iq4xs.py:5-11);
// Q4_0 / Q5_0 / IQ4_NL, which the reference leaves to the un-vendored plugin, follow gguf-py.
#pragma once
#include "gq_common.cuh"

namespace gq {

// fp16 bit pattern of an exactly representable constant, at compile time
constexpr uint32_t hc(double v) {
    uint32_t s = 0;
    if (v < 0) { s = 0x8000u; v = -v; }
    if (v == 0) return s;
    int e = 0;
    while (v >= 2) { v /= 2; e++; }
    while (v < 1) { v *= 2; e--; }
    return s | ((uint32_t)(e + 15) << 10) | (uint32_t)((v - 1) * 1024 + 0.5);
}
constexpr uint32_t h2k(double v) { return hc(v) | (hc(v) << 16); }

GQ_HD inline uint4 ld16(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }
GQ_HD inline uint2 ld8(const uint8_t *p) { return *reinterpret_cast<const uint2 *>(p); }
GQ_HD inline uint32_t ld4(const uint8_t *p) { return *reinterpret_cast<const uint32_t *>(p); }
GQ_HD inline uint32_t ld2(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
GQ_HD inline uint32_t w4(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
GQ_HD inline float u8f(uint32_t word, int byte) { return (float)((word >> (8 * byte)) & 0xFFu); }
GQ_HD inline float s8f(uint32_t word, int byte) { return (float)(int)(int8_t)((word >> (8 * byte)) & 0xFFu); }

// nibble-pair word (bytes hold weights i0,i2,i1,i3): low nibbles -> `lo`, high nibbles -> `hi`, each as
// {(i0,i1), (i2,i3)} fp16 pairs of (nibble - OFF)
template <int OFF>
GQ_HD inline void nib_word(uint32_t w, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
    const uint32_t w8 = w >> 8;
    lo[0] = hsub2(and_or(w, 0x000f000fu, GQ_MAGIC), h2k(1024 + OFF));
    lo[1] = hsub2(and_or(w8, 0x000f000fu, GQ_MAGIC), h2k(1024 + OFF));
    hi[0] = hfma2(and_or(w, 0x00f000f0u, GQ_MAGIC), h2k(0.0625), h2k(-64 - OFF));
    hi[1] = hfma2(and_or(w8, 0x00f000f0u, GQ_MAGIC), h2k(0.0625), h2k(-64 - OFF));
}

// the IQ4 codebook as unsigned bytes (value + 128) in four registers, filled by the kernel from the
// generated table
struct Iq4Table { uint32_t t0, t1, t2, t3; };

// natural-order nibble word through the 16-entry codebook: lo[] / hi[] as above, exact codebook values
GQ_HD inline void iq4_word(uint32_t w, const Iq4Table &T, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
    const uint32_t s = w & 0x77777777u;
    const uint32_t s2 = and_or(w >> 1, 0x44444444u, 0x32103210u);
    const uint32_t rl = prmt(prmt(T.t0, T.t1, s), prmt(T.t2, T.t3, s), s2);                       // bytes 0,1
    const uint32_t rh = prmt(prmt(T.t0, T.t1, s >> 16), prmt(T.t2, T.t3, s >> 16), s2 >> 16);     // bytes 2,3
    // rl = (b0.lo, b0.hi, b1.lo, b1.hi) as value + 128
    lo[0] = hsub2(prmt(rl, GQ_MAGICB, 0x5250u), h2k(1152));
    lo[1] = hsub2(prmt(rh, GQ_MAGICB, 0x5250u), h2k(1152));
    hi[0] = hsub2(prmt(rl, GQ_MAGICB, 0x5351u), h2k(1152));
    hi[1] = hsub2(prmt(rh, GQ_MAGICB, 0x5351u), h2k(1152));
}

struct DecAux {
    const uint2 *iq3s_grid;   // shared memory: 512 entries, {fp16(m0,m1), fp16(m2,m3)}
    Iq4Table iq4;
};

template <int TYPE>
struct Dec;

// ---- Q4_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q4_K> {
    static constexpr int GROUP = 32;
    static constexpr bool HAS_MIN = true;
    uint4 q[4];
    uint32_t dd[2], sc[2][2], mn[2][2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 hd = ld16(slab + 2048 + 16 * ((lane >> 2) + 8 * h));
            dd[h] = hd.x;
            sc[h][0] = hd.y & 0x3f3f3f3fu;
            mn[h][0] = hd.z & 0x3f3f3f3fu;
            sc[h][1] = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
            mn[h][1] = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
        }
    }
    // run pair P = (2P, 2P+1): qs group c = P>>1, nibble half = P&1, u = run&1
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int c = P >> 1, hi = P & 1;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t lo_[2], hi_[2];
                nib_word<0>(w4(q[c], 2 * h + u), lo_, hi_);
                a[u][h] = hi ? hi_[0] : lo_[0];
                a[u][2 + h] = hi ? hi_[1] : lo_[1];
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = u8f(sc[0][G >> 2], G & 3);
        s1 = u8f(sc[1][G >> 2], G & 3);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    GQ_HD void min_scale(float &m0, float &m1) const { m0 = f16hi(dd[0]); m1 = f16hi(dd[1]); }
    // integer mins of runs 4t..4t+3 (groups 2t, 2t+1) for rows g (a[0], a[2]) and g+8 (a[1], a[3])
    GQ_HD void min_frag(uint32_t (&a)[4]) const {
        const uint32_t j = 2 * (t & 1);
        const uint32_t s0 = 0x5050u | (j * 0x0101u), s1 = 0x5050u | ((j + 1) * 0x0101u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = (t & 2) ? mn[h][1] : mn[h][0];
            a[h] = hsub2(prmt(w, GQ_MAGICB, s0), h2k(1024));
            a[2 + h] = hsub2(prmt(w, GQ_MAGICB, s1), h2k(1024));
        }
    }
};

// ---- Q5_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q5_K> {
    static constexpr int GROUP = 32;
    static constexpr bool HAS_MIN = true;
    uint4 q[5];
    uint32_t dd[2], sc[2][2], mn[2][2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 5; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 hd = ld16(slab + 2560 + 16 * ((lane >> 2) + 8 * h));
            dd[h] = hd.x;
            sc[h][0] = hd.y & 0x3f3f3f3fu;
            mn[h][0] = hd.z & 0x3f3f3f3fu;
            sc[h][1] = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
            mn[h][1] = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
        }
    }
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int c = P >> 1, hi = P & 1, ib = P;   // sub-block index = run pair index
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = w4(q[c], 2 * h + u), H = w4(q[4], 2 * h + u);
                const uint32_t w8 = w >> 8, H8 = H >> 8;
                if constexpr (!hi) {
                    a[u][h] = hsub2(or_and(and_or(w, 0x000f000fu, GQ_MAGIC), shl_c<4 - ib>(H), 0x00100010u), h2k(1024));
                    a[u][2 + h] = hsub2(or_and(and_or(w8, 0x000f000fu, GQ_MAGIC), shl_c<4 - ib>(H8), 0x00100010u), h2k(1024));
                } else {
                    a[u][h] = hfma2(or_and(and_or(w, 0x00f000f0u, GQ_MAGIC), shl_c<8 - ib>(H), 0x01000100u), h2k(0.0625), h2k(-64));
                    a[u][2 + h] = hfma2(or_and(and_or(w8, 0x00f000f0u, GQ_MAGIC), shl_c<8 - ib>(H8), 0x01000100u), h2k(0.0625), h2k(-64));
                }
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = u8f(sc[0][G >> 2], G & 3);
        s1 = u8f(sc[1][G >> 2], G & 3);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    GQ_HD void min_scale(float &m0, float &m1) const { m0 = f16hi(dd[0]); m1 = f16hi(dd[1]); }
    GQ_HD void min_frag(uint32_t (&a)[4]) const {
        const uint32_t j = 2 * (t & 1);
        const uint32_t s0 = 0x5050u | (j * 0x0101u), s1 = 0x5050u | ((j + 1) * 0x0101u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = (t & 2) ? mn[h][1] : mn[h][0];
            a[h] = hsub2(prmt(w, GQ_MAGICB, s0), h2k(1024));
            a[2 + h] = hsub2(prmt(w, GQ_MAGICB, s1), h2k(1024));
        }
    }
};

// ---- Q6_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q6_K> {
    static constexpr int GROUP = 16;
    static constexpr bool HAS_MIN = false;
    uint4 q[6];
    uint4 sc[2];
    uint32_t dd[2];
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
#pragma unroll
        for (int c = 0; c < 6; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            sc[h] = ld16(slab + 3072 + 16 * row);
            dd[h] = ld2(slab + 3072 + 256 + 2 * row);
        }
    }
    // run pair P: half h' = P>>2, t' = P&3 (32-weight quarter of the half), runs u = 0,1
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int hp = P >> 2, tp = P & 3, hi = tp >> 1;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = w4(q[2 * hp + (tp & 1)], 2 * h + u), H = w4(q[4 + hp], 2 * h + u);
                const uint32_t w8 = w >> 8, H8 = H >> 8;
                if constexpr (!hi) {
                    a[u][h] = hsub2(or_and(and_or(w, 0x000f000fu, GQ_MAGIC), shl_c<4 - 2 * tp>(H), 0x00300030u), h2k(1056));
                    a[u][2 + h] = hsub2(or_and(and_or(w8, 0x000f000fu, GQ_MAGIC), shl_c<4 - 2 * tp>(H8), 0x00300030u), h2k(1056));
                } else {
                    a[u][h] = hfma2(or_and(and_or(w, 0x00f000f0u, GQ_MAGIC), shl_c<8 - 2 * tp>(H), 0x03000300u), h2k(0.0625), h2k(-96));
                    a[u][2 + h] = hfma2(or_and(and_or(w8, 0x00f000f0u, GQ_MAGIC), shl_c<8 - 2 * tp>(H8), 0x03000300u), h2k(0.0625), h2k(-96));
                }
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = s8f(w4(sc[0], G >> 2), G & 3);
        s1 = s8f(w4(sc[1], G >> 2), G & 3);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
};

// ---- Q8_0 -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q8_0> {
    static constexpr int GROUP = 32;
    static constexpr bool HAS_MIN = false;
    uint4 q[8];
    uint4 d8[2];
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
#pragma unroll
        for (int c = 0; c < 8; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) d8[h] = ld16(slab + 4096 + 16 * ((lane >> 2) + 8 * h));
    }
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t x = w4(q[P], 2 * h + u) ^ 0x80808080u;
                a[u][h] = hsub2(prmt(x, GQ_MAGICB, 0x5150u), h2k(1152));
                a[u][2 + h] = hsub2(prmt(x, GQ_MAGICB, 0x5352u), h2k(1152));
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        const uint32_t w0 = w4(d8[0], G >> 1), w1 = w4(d8[1], G >> 1);
        s0 = (G & 1) ? f16hi(w0) : f16lo(w0);
        s1 = (G & 1) ? f16hi(w1) : f16lo(w1);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
};

// ---- Q4_0 / IQ4_NL (18-byte blocks: d, 16 nibble bytes) ---------------------------------------------
template <int TYPE>
struct DecLegacy4 {
    static constexpr int GROUP = 32;
    static constexpr bool HAS_MIN = false;
    uint4 q[4];
    uint4 d8[2];
    Iq4Table tab;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        tab = aux.iq4;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) d8[h] = ld16(slab + 2048 + 16 * ((lane >> 2) + 8 * h));
    }
    // run pair P = block P: low nibbles are run 2P, high nibbles run 2P+1
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t lo_[2], hi_[2];
            const uint32_t w = w4(q[P >> 1], 2 * h + (P & 1));
            if constexpr (TYPE == GQ_Q4_0) nib_word<8>(w, lo_, hi_); else iq4_word(w, tab, lo_, hi_);
            a[0][h] = lo_[0]; a[0][2 + h] = lo_[1];
            a[1][h] = hi_[0]; a[1][2 + h] = hi_[1];
        }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        const uint32_t w0 = w4(d8[0], G >> 1), w1 = w4(d8[1], G >> 1);
        s0 = (G & 1) ? f16hi(w0) : f16lo(w0);
        s1 = (G & 1) ? f16hi(w1) : f16lo(w1);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
};
template <> struct Dec<GQ_Q4_0> : DecLegacy4<GQ_Q4_0> {};
template <> struct Dec<GQ_IQ4_NL> : DecLegacy4<GQ_IQ4_NL> {};

// ---- Q5_0 (22-byte blocks: d, qh u32, 16 nibble bytes) ----------------------------------------------
template <>
struct Dec<GQ_Q5_0> {
    static constexpr int GROUP = 32;
    static constexpr bool HAS_MIN = false;
    uint4 q[4];
    uint4 d8[2];
    uint4 qh[2][2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint8_t *p = slab + 2048 + 48 * ((lane >> 2) + 8 * h);
            d8[h] = ld16(p);
            qh[h][0] = ld16(p + 16);
            qh[h][1] = ld16(p + 32);
        }
    }
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = w4(q[P >> 1], 2 * h + (P & 1)), w8 = w >> 8;
            const uint32_t H = w4(qh[h][P >> 2], P & 3);
            // bits 4t..4t+3 belong to the low-nibble run, 16+4t.. to the high-nibble run; spread bit i0 -> 0,
            // i1 -> 16 (and i2, i3 after a shift by 2)
            const uint32_t bl = (H >> (4 * t)) & 0xFu, bh = (H >> (16 + 4 * t)) & 0xFu;
            const uint32_t zl = (bl | (bl << 15)) << 4, zh = (bh | (bh << 15)) << 8;
            a[0][h] = hsub2(or_and(and_or(w, 0x000f000fu, GQ_MAGIC), zl, 0x00100010u), h2k(1040));
            a[0][2 + h] = hsub2(or_and(and_or(w8, 0x000f000fu, GQ_MAGIC), zl >> 2, 0x00100010u), h2k(1040));
            a[1][h] = hfma2(or_and(and_or(w, 0x00f000f0u, GQ_MAGIC), zh, 0x01000100u), h2k(0.0625), h2k(-80));
            a[1][2 + h] = hfma2(or_and(and_or(w8, 0x00f000f0u, GQ_MAGIC), zh >> 2, 0x01000100u), h2k(0.0625), h2k(-80));
        }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        const uint32_t w0 = w4(d8[0], G >> 1), w1 = w4(d8[1], G >> 1);
        s0 = (G & 1) ? f16hi(w0) : f16lo(w0);
        s1 = (G & 1) ? f16hi(w1) : f16lo(w1);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
};

// ---- IQ4_XS ---------------------------------------------------------------------------------------
template <>
struct Dec<GQ_IQ4_XS> {
    static constexpr int GROUP = 32;
    static constexpr bool HAS_MIN = false;
    uint4 q[4];
    uint2 hd[2];
    Iq4Table tab;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        tab = aux.iq4;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) hd[h] = ld8(slab + 2048 + 8 * ((lane >> 2) + 8 * h));
    }
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t lo_[2], hi_[2];
            iq4_word(w4(q[P >> 1], 2 * h + (P & 1)), tab, lo_, hi_);
            a[0][h] = lo_[0]; a[0][2 + h] = lo_[1];
            a[1][h] = hi_[0]; a[1][2 + h] = hi_[1];
        }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t l = (hd[h].y >> (4 * G)) & 0xFu, hh = (hd[h].x >> (16 + 2 * G)) & 3u;
            const float v = (float)((int)(l | (hh << 4)) - 32);
            if (h == 0) s0 = v; else s1 = v;
        }
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(hd[0].x); d1 = f16lo(hd[1].x); }
};

// ---- Q2_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q2_K> {
    static constexpr int GROUP = 16;
    static constexpr bool HAS_MIN = true;
    uint4 q[2];
    uint4 sc[2];
    uint32_t dd[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 2; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            sc[h] = ld16(slab + 1024 + 16 * row);
            dd[h] = ld4(slab + 1024 + 256 + 4 * row);
        }
    }
    // run pair P: n = P>>2 (128-weight half), t' = P&3 (bit pair 2t' of each byte), runs u = 0,1
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int n = P >> 2, tp = P & 3;
        constexpr uint32_t mask = 0x00030003u << (2 * tp);
        constexpr double inv = tp == 0 ? 1.0 : tp == 1 ? 0.25 : tp == 2 ? 0.0625 : 0.015625;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = w4(q[n], 2 * h + u);
                a[u][h] = hfma2(and_or(w, mask, GQ_MAGIC), h2k(inv), h2k(-1024 * inv));
                a[u][2 + h] = hfma2(and_or(w >> 8, mask, GQ_MAGIC), h2k(inv), h2k(-1024 * inv));
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = (float)((w4(sc[0], G >> 2) >> (8 * (G & 3))) & 0xFu);
        s1 = (float)((w4(sc[1], G >> 2) >> (8 * (G & 3))) & 0xFu);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    GQ_HD void min_scale(float &m0, float &m1) const { m0 = f16hi(dd[0]); m1 = f16hi(dd[1]); }
    GQ_HD void min_frag(uint32_t (&a)[4]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = (w4(sc[h], t) >> 4) & 0x0f0f0f0fu;   // mins of runs 4t..4t+3
            a[h] = hsub2(prmt(w, GQ_MAGICB, 0x5150u), h2k(1024));
            a[2 + h] = hsub2(prmt(w, GQ_MAGICB, 0x5352u), h2k(1024));
        }
    }
};

// ---- Q3_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q3_K> {
    static constexpr int GROUP = 16;
    static constexpr bool HAS_MIN = false;
    uint4 q[3];
    uint32_t sv[2][4];   // the sixteen 6-bit scales of a row as bytes (value + 32 ... stored value)
    uint32_t dd[2];
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
#pragma unroll
        for (int c = 0; c < 3; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint8_t *p = slab + 1536 + 12 * row;
            const uint32_t s0 = ld4(p), s1 = ld4(p + 4), s2 = ld4(p + 8);
            sv[h][0] = (s0 & 0x0f0f0f0fu) | ((s2 & 0x03030303u) << 4);
            sv[h][1] = (s1 & 0x0f0f0f0fu) | (((s2 >> 2) & 0x03030303u) << 4);
            sv[h][2] = ((s0 >> 4) & 0x0f0f0f0fu) | (((s2 >> 4) & 0x03030303u) << 4);
            sv[h][3] = ((s1 >> 4) & 0x0f0f0f0fu) | (((s2 >> 6) & 0x03030303u) << 4);
            dd[h] = ld2(slab + 1536 + 192 + 2 * row);
        }
    }
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int n = P >> 2, tp = P & 3;
        constexpr uint32_t mask = 0x00030003u << (2 * tp), hmsk = 0x00040004u << (2 * tp);
        constexpr double inv = tp == 0 ? 1.0 : tp == 1 ? 0.25 : tp == 2 ? 0.0625 : 0.015625;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = w4(q[n], 2 * h + u), H = w4(q[2], 2 * h + u);
                a[u][h] = hfma2(or_and(and_or(w, mask, GQ_MAGIC), shl_c<tp + 2 - 4 * n>(H), hmsk), h2k(inv), h2k(-1024 * inv - 4));
                a[u][2 + h] = hfma2(or_and(and_or(w >> 8, mask, GQ_MAGIC), shl_c<tp + 2 - 4 * n>(H >> 8), hmsk), h2k(inv), h2k(-1024 * inv - 4));
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = u8f(sv[0][G >> 2], G & 3) - 32.0f;
        s1 = u8f(sv[1][G >> 2], G & 3) - 32.0f;
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
};

// ---- IQ3_S ----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_IQ3_S> {
    static constexpr int GROUP = 32;
    static constexpr bool HAS_MIN = false;
    uint4 q[2];      // 16 grid-index bytes per row (byte r = run r)
    uint4 sg[2];     // 16 sign bytes per row, pre-shifted so that the lane's nibble is the low one
    uint2 qh[2];     // the eight qh bytes per row, pre-shifted by t
    uint32_t scw[2], dd[2];
    const uint2 *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        grid = aux.iq3s_grid;
        const int t = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            q[h] = ld16(slab + 512 * h + 16 * lane);
            uint4 s = ld16(slab + 1024 + 32 * row + 16 * (t >> 1));
            const int sh = 4 * (t & 1);
            s.x >>= sh; s.y >>= sh; s.z >>= sh; s.w >>= sh;
            sg[h] = s;
            uint2 hq = ld8(slab + 1536 + 8 * row);
            hq.x >>= t; hq.y >>= t;
            qh[h] = hq;
            scw[h] = ld4(slab + 1664 + 4 * row);
            dd[h] = ld2(slab + 1728 + 2 * row);
        }
    }
    template <int R>
    GQ_HD void run(int h, uint32_t &a01, uint32_t &a23) const {
        constexpr int ib = R >> 1, u = R & 1;
        const uint32_t idxb = (w4(q[h], R >> 2) >> (8 * (R & 3))) & 0xFFu;
        const uint32_t hw = (ib < 4) ? qh[h].x : qh[h].y;
        const uint32_t idx = or_and(idxb, shl_c<8 - (8 * (ib & 3) + 4 * u)>(hw), 0x100u);
        const uint2 e = grid[idx];
        const uint32_t nib = (w4(sg[h], R >> 2) >> (8 * (R & 3))) & 0xFu;
        a01 = xor_and(e.x, nib * 0x40008000u, 0x80008000u);
        a23 = xor_and(e.y, (nib >> 2) * 0x40008000u, 0x80008000u);
    }
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            run<2 * P>(h, a[0][h], a[0][2 + h]);
            run<2 * P + 1>(h, a[1][h], a[1][2 + h]);
        }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = (float)(1 + 2 * ((scw[0] >> (4 * G)) & 0xFu));
        s1 = (float)(1 + 2 * ((scw[1] >> (4 * G)) & 0xFu));
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
};

}  // namespace gq
