// Integer dequantisers of the eleven GGML types for the small-batch kernel (1..16 batch rows): from the
// lane-ordered slab layout (gq_layout.h) straight to int8 A-operand registers of mma.sync m16n8k32 / m16n8k16.
//
// Lane l = 4*g + t owns, for rows g and g+8, the "quad" 16*r + 4*t + {0,1,2,3} of every 16-weight run r.  A quad
// is one 32-bit register of four 8-bit weights, byte z holding weight (0,2,1,3)[z] of the quad (the order in
// which the mask-extracted types already store their bytes); the activation planes use the same byte order, so
// A and B agree.  The k-step S of a k-block (S = 0..7) is the 32-weight sub-block S = runs 2S and 2S+1:
//     a[0] = (row g, run 2S)   a[1] = (row g+8, run 2S)   a[2] = (row g, run 2S+1)   a[3] = (row g+8, run 2S+1)
//
// Four ways a type's group scales reach the result (SCHEME):
//   S32   integer scale per 32 weights (Q4_K, Q5_K, IQ4_XS, IQ3_S): one MMA per sub-block and activation plane,
//         int32 result times the scale into int32 accumulators (one IMAD each)
//   F32   fp16 scale per 32 weights (Q8_0, Q4_0, Q5_0, IQ4_NL): the int32 result goes to fp32 and is scaled there
//   S16   integer scale per 16 weights that cannot be folded (Q6_K): m16n8k16 MMAs, one per run
//   FOLD  the scale is multiplied into the 8-bit weight itself (Q2_K: q*sc <= 45; Q3_K: (q-3)*sc + 128 in 0..252),
//         so the tensor core accumulates the whole k-block and nothing is scaled afterwards
// Whatever is constant over a run — the offset of an unsigned field (q-8, q-16, q-32), the +128 of the Q3_K fold,
// the minimum term of Q2_K / Q4_K / Q5_K — is removed by one fp16 "correction" MMA per k-block of small exact
// per-run integers (or the block's fp16 d) against the per-run activation sums:  acc -= f[row] * sum_run A''[row][run] * Sx[run][n].
// The value arithmetic follows the formats as the reference states them (gguf-plugin/gluon/kq_ref.py:17-79, q2k.py:5-12,
// q4k.py:5-10, iq3s_int8t.py:4-11, iq4xs.py:5-11); Q4_0 / Q5_0 / IQ4_NL follow gguf-py.
#pragma once
#include "gq_decode.cuh"

namespace gq {

enum { GQ_S32 = 0, GQ_F32 = 1, GQ_S16 = 2, GQ_FOLD = 3 };

struct DecAux8 {
    const uint32_t *grid;        // shared memory: the codebook of the CTA's type, four magnitude bytes per entry in quad byte order
                                 // (IQ3_S 512, IQ3_XXS 256 entries; IQ2_*: two words per entry)
    Iq4Table iq4;                // the IQ4 codebook as signed bytes
};

GQ_HD inline uint32_t nib0(uint32_t w) { return w & 0x0f0f0f0fu; }
GQ_HD inline uint32_t nib1(uint32_t w) { return (w >> 4) & 0x0f0f0f0fu; }
template <int HI>
GQ_HD inline uint32_t nibx(uint32_t w) { return HI ? nib1(w) : nib0(w); }
// byte K of w, zero- or sign-extended to 32 bits (one prmt)
template <int K>
GQ_HD inline int ubyte(uint32_t w) { return (int)prmt(w, 0u, 0x4440u | K); }
template <int K>
GQ_HD inline int sbyte(uint32_t w) { return (int)prmt(w, 0u, ((8u | K) * 0x1110u) | K); }
// four unsigned bytes (each below 128) + 96, then the top bit flipped: the bytes of (value - 32) as int8
GQ_HD inline uint32_t minus32_s8(uint32_t w) { return (w + 0x60606060u) ^ 0x80808080u; }

template <int TYPE>
struct Dec8;

// ---- Q4_K -----------------------------------------------------------------------------------------
template <>
struct Dec8<GQ_Q4_K> {
    static constexpr int SCHEME = GQ_S32;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint4 q[4];
    uint32_t dd[2], sc[2][2], mn[2][2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 hd = ld16(slab + 2048 + 16 * ((lane >> 2) + 8 * h));
            dd[h] = hd.x;
            k4_scales(hd, sc[h], mn[h]);
        }
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        constexpr int c = S >> 1, hi = S & 1;
        a[0] = nibx<hi>(q[c].x); a[1] = nibx<hi>(q[c].z); a[2] = nibx<hi>(q[c].y); a[3] = nibx<hi>(q[c].w);
    }
    template <int S>
    GQ_HD void iscale(int &s0, int &s1) const { s0 = ubyte<(S & 3)>(sc[0][S >> 2]); s1 = ubyte<(S & 3)>(sc[1][S >> 2]); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    // the minimum term: A'' = m of sub-blocks 2t (runs 4t, 4t+1) and 2t+1 (runs 4t+2, 4t+3), factor dmin
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
        const uint32_t j = 2 * (t & 1);
        const uint32_t s0 = 0x5050u | (j * 0x0101u), s1 = 0x5050u | ((j + 1) * 0x0101u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t wm = (t & 2) ? mn[h][1] : mn[h][0];
            a[h] = hsub2(bytes_h2(wm, s0), h2k(1024));
            a[2 + h] = hsub2(bytes_h2(wm, s1), h2k(1024));
            f[h] = f16hi(dd[h]);
        }
    }
};

// ---- Q5_K -----------------------------------------------------------------------------------------
template <>
struct Dec8<GQ_Q5_K> {
    static constexpr int SCHEME = GQ_S32;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint4 q[5];
    uint32_t dd[2], sc[2][2], mn[2][2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 5; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 hd = ld16(slab + 2560 + 16 * ((lane >> 2) + 8 * h));
            dd[h] = hd.x;
            k4_scales(hd, sc[h], mn[h]);
        }
    }
    template <int S, int E>
    GQ_HD uint32_t quad() const {
        constexpr int c = S >> 1, hi = S & 1;
        return and_or(shl_c<4 - S>(w4(q[4], E)), 0x10101010u, nibx<hi>(w4(q[c], E)));
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        a[0] = quad<S, 0>(); a[1] = quad<S, 2>(); a[2] = quad<S, 1>(); a[3] = quad<S, 3>();
    }
    template <int S>
    GQ_HD void iscale(int &s0, int &s1) const { s0 = ubyte<(S & 3)>(sc[0][S >> 2]); s1 = ubyte<(S & 3)>(sc[1][S >> 2]); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
        const uint32_t j = 2 * (t & 1);
        const uint32_t s0 = 0x5050u | (j * 0x0101u), s1 = 0x5050u | ((j + 1) * 0x0101u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t wm = (t & 2) ? mn[h][1] : mn[h][0];
            a[h] = hsub2(bytes_h2(wm, s0), h2k(1024));
            a[2 + h] = hsub2(bytes_h2(wm, s1), h2k(1024));
            f[h] = f16hi(dd[h]);
        }
    }
};

// ---- Q6_K: int8 scale per 16 weights, unsigned 6-bit field, the -32 goes to the correction --------------
template <>
struct Dec8<GQ_Q6_K> {
    static constexpr int SCHEME = GQ_S16;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint4 q[6];
    uint4 sc[2];      // the sixteen int8 scales of a row, as stored
    uint32_t dd[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 6; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            sc[h] = ld16(slab + 3072 + 16 * row);
            dd[h] = ld2(slab + 3072 + 256 + 2 * row);
        }
    }
    // run R = 8*hp + 2*tp + u: low-bit nibble in chunk 2*hp + (tp & 1) (high nibble for tp >= 2), bit pair tp of chunk 4 + hp
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        constexpr int P = R >> 1, u = R & 1, hp = P >> 2, tp = P & 3, E = 2 * H + u;
        return and_or(shl_c<4 - 2 * tp>(w4(q[4 + hp], E)), 0x30303030u, nibx<(tp >> 1)>(w4(q[2 * hp + (tp & 1)], E)));
    }
    template <int R>
    GQ_HD void step16(uint32_t (&a)[2]) const { a[0] = quad<R, 0>(); a[1] = quad<R, 1>(); }
    template <int R>
    GQ_HD void iscale16(int &s0, int &s1) const { s0 = sbyte<(R & 3)>(w4(sc[0], R >> 2)); s1 = sbyte<(R & 3)>(w4(sc[1], R >> 2)); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
    // weight = field - 32: A'' = sc of runs 4t..4t+3, factor 32 d
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = w4(sc[h], t) ^ 0x80808080u;
            a[h] = hsub2(bytes_h2(w, 0x5150u), h2k(1152));
            a[2 + h] = hsub2(bytes_h2(w, 0x5352u), h2k(1152));
            f[h] = 32.0f * f16bits(dd[h]);
        }
    }
};

// ---- Q8_0: the stored bytes are the operand ---------------------------------------------------------
template <>
struct Dec8<GQ_Q8_0> {
    static constexpr int SCHEME = GQ_F32;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint4 q[8];
    uint4 d8[2];
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
#pragma unroll
        for (int c = 0; c < 8; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) d8[h] = ld16(slab + 4096 + 16 * ((lane >> 2) + 8 * h));
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const { a[0] = q[S].x; a[1] = q[S].z; a[2] = q[S].y; a[3] = q[S].w; }
    template <int S>
    GQ_HD void fscale(float &s0, float &s1) const { d8_scale<S>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
};

// ---- Q4_0: unsigned nibbles, the -8 goes to the correction (A'' = the block's d, factor 8) ---------------
template <>
struct Dec8<GQ_Q4_0> {
    static constexpr int SCHEME = GQ_F32;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint4 q[4];
    uint4 d8[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) d8[h] = ld16(slab + 2048 + 16 * ((lane >> 2) + 8 * h));
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        const uint32_t w0 = w4(q[S >> 1], S & 1), w1 = w4(q[S >> 1], 2 + (S & 1));
        a[0] = nib0(w0); a[1] = nib0(w1); a[2] = nib1(w0); a[3] = nib1(w1);
    }
    template <int S>
    GQ_HD void fscale(float &s0, float &s1) const { d8_scale<S>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
        uint32_t a1[1][4];
        float f1[1][2];
        d8_corr(t, d8, 8.0f, a1, f1);
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = a1[0][i];
        f[0] = f1[0][0]; f[1] = f1[0][1];
    }
};

// bit i (0..3) of x to bit 4 of byte (0,2,1,3)[i]: the fifth bits of a quad of Q5_0
GQ_HD inline uint32_t spread5(uint32_t x) { return x * ((1u << 4) | (1u << 19) | (1u << 10) | (1u << 25)); }

// ---- Q5_0 ---------------------------------------------------------------------------------------------
template <>
struct Dec8<GQ_Q5_0> {
    static constexpr int SCHEME = GQ_F32;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint4 q[4];
    uint4 d8[2];
    uint4 qh[2][2];   // the eight blocks' fifth-bit words of a row, shifted so that the lane's bits are the low ones
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint8_t *p = slab + 2048 + 48 * ((lane >> 2) + 8 * h);
            d8[h] = ld16(p);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint4 v = ld16(p + 16 + 16 * i);
                v.x >>= 4 * t; v.y >>= 4 * t; v.z >>= 4 * t; v.w >>= 4 * t;
                qh[h][i] = v;
            }
        }
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = w4(q[S >> 1], 2 * h + (S & 1)), H = w4(qh[h][S >> 2], S & 3);
            a[h] = and_or(spread5(H & 0xFu), 0x10101010u, nib0(w));
            a[2 + h] = and_or(spread5((H >> 16) & 0xFu), 0x10101010u, nib1(w));
        }
    }
    template <int S>
    GQ_HD void fscale(float &s0, float &s1) const { d8_scale<S>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
        uint32_t a1[1][4];
        float f1[1][2];
        d8_corr(t, d8, 16.0f, a1, f1);
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = a1[0][i];
        f[0] = f1[0][0]; f[1] = f1[0][1];
    }
};

// natural-order nibble word through the signed 16-entry codebook: lo = the quad of the low nibbles, hi = of the
// high nibbles, both in quad byte order
GQ_HD inline void iq4_word8(uint32_t w, const Iq4Table &T, uint32_t &lo, uint32_t &hi) {
    const uint32_t s = w & 0x77777777u;
    const uint32_t s2 = and_or(w >> 1, 0x44444444u, 0x32103210u);
    const uint32_t rl = prmt(prmt(T.t0, T.t1, s), prmt(T.t2, T.t3, s), s2);                       // nibbles 0..3
    const uint32_t rh = prmt(prmt(T.t0, T.t1, s >> 16), prmt(T.t2, T.t3, s >> 16), s2 >> 16);     // nibbles 4..7
    lo = prmt(rl, rh, 0x6240u);
    hi = prmt(rl, rh, 0x7351u);
}

// ---- IQ4_NL ---------------------------------------------------------------------------------------
template <>
struct Dec8<GQ_IQ4_NL> {
    static constexpr int SCHEME = GQ_F32;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint4 q[4];
    uint4 d8[2];
    Iq4Table tab;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        tab = aux.iq4;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) d8[h] = ld16(slab + 2048 + 16 * ((lane >> 2) + 8 * h));
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        iq4_word8(w4(q[S >> 1], S & 1), tab, a[0], a[2]);
        iq4_word8(w4(q[S >> 1], 2 + (S & 1)), tab, a[1], a[3]);
    }
    template <int S>
    GQ_HD void fscale(float &s0, float &s1) const { d8_scale<S>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
};

// ---- IQ4_XS ---------------------------------------------------------------------------------------
template <>
struct Dec8<GQ_IQ4_XS> {
    static constexpr int SCHEME = GQ_S32;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint4 q[4];
    uint32_t ls[2][2];   // the eight sub-block scales of a row, (6-bit value - 32) as int8 bytes
    uint32_t dd[2];
    Iq4Table tab;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        tab = aux.iq4;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint2 hd = ld8(slab + 2048 + 8 * ((lane >> 2) + 8 * h));
            dd[h] = hd.x;
            const uint32_t e = hd.y & 0x0f0f0f0fu, o = (hd.y >> 4) & 0x0f0f0f0fu;   // groups 0,2,4,6 | 1,3,5,7
            const uint32_t sh = hd.x >> 16;
            uint32_t a0 = (sh | (sh << 12)) & 0x000f000fu;
            a0 = (a0 | (a0 << 6)) & 0x03030303u;
            const uint32_t s8 = sh >> 8;
            uint32_t a1 = (s8 | (s8 << 12)) & 0x000f000fu;
            a1 = (a1 | (a1 << 6)) & 0x03030303u;
            ls[h][0] = minus32_s8(prmt(e, o, 0x5140u) | (a0 << 4));
            ls[h][1] = minus32_s8(prmt(e, o, 0x7362u) | (a1 << 4));
        }
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        iq4_word8(w4(q[S >> 1], S & 1), tab, a[0], a[2]);
        iq4_word8(w4(q[S >> 1], 2 + (S & 1)), tab, a[1], a[3]);
    }
    template <int S>
    GQ_HD void iscale(int &s0, int &s1) const { s0 = sbyte<(S & 3)>(ls[0][S >> 2]); s1 = sbyte<(S & 3)>(ls[1][S >> 2]); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
};

// ---- Q2_K: the 4-bit scale is multiplied into the 2-bit field (at most 45) ----------------------------
template <>
struct Dec8<GQ_Q2_K> {
    static constexpr int SCHEME = GQ_FOLD;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint4 q[2];
    uint4 sc[2], mn[2];   // low / high nibbles of the sixteen scale bytes, one per byte
    uint32_t dd[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 2; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint4 s = ld16(slab + 1024 + 16 * row);
            sc[h] = make_uint4(s.x & 0x0f0f0f0fu, s.y & 0x0f0f0f0fu, s.z & 0x0f0f0f0fu, s.w & 0x0f0f0f0fu);
            mn[h] = make_uint4((s.x >> 4) & 0x0f0f0f0fu, (s.y >> 4) & 0x0f0f0f0fu, (s.z >> 4) & 0x0f0f0f0fu, (s.w >> 4) & 0x0f0f0f0fu);
            dd[h] = ld4(slab + 1024 + 256 + 4 * row);
        }
    }
    // run R = 8n + 2j + u of row half H: bit pair j of word (n, 2H + u), times the run's scale
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        constexpr int n = R >> 3, j = (R >> 1) & 3, u = R & 1;
        const uint32_t f = (w4(q[n], 2 * H + u) >> (2 * j)) & 0x03030303u;
        return f * (uint32_t)ubyte<(R & 3)>(w4(sc[H], R >> 2));
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        a[0] = quad<2 * S, 0>(); a[1] = quad<2 * S, 1>(); a[2] = quad<2 * S + 1, 0>(); a[3] = quad<2 * S + 1, 1>();
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    // the minimum term: A'' = m of runs 4t..4t+3, factor dmin
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t wm = w4(mn[h], t);
            a[h] = hsub2(bytes_h2(wm, 0x5150u), h2k(1024));
            a[2 + h] = hsub2(bytes_h2(wm, 0x5352u), h2k(1024));
            f[h] = f16hi(dd[h]);
        }
    }
};

// ---- Q3_K: weight = (sc - 32) * (w - 4), w the 3-bit field.  With s = sc - 32 in [-32, 31] the byte
// U = s * (w - 3) + 128 lies in [0, 252]; one 32-bit multiply-add makes the four bytes of a quad at once
// (s * w4 + (128 - 3 s) * 0x01010101: no byte of the true result is negative, so none borrows from its neighbour).
// value / d = (U - 128) - s: the correction removes (sc + 96) per run ----------------------------------------
template <>
struct Dec8<GQ_Q3_K> {
    static constexpr int SCHEME = GQ_FOLD;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint4 q[3];
    uint32_t sv[2][4];   // the sixteen 6-bit scales of a row as bytes (raw value, 0..63)
    uint32_t ss[2][4];   // the same minus 32, as int8 bytes
    uint32_t dd[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &) {
        t = lane & 3;
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
#pragma unroll
            for (int i = 0; i < 4; ++i) ss[h][i] = minus32_s8(sv[h][i]);
            dd[h] = ld2(slab + 1536 + 192 + 2 * row);
        }
    }
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        constexpr int n = R >> 3, j = (R >> 1) & 3, u = R & 1, E = 2 * H + u;
        const uint32_t w3 = and_or(shl_c<2 - (4 * n + j)>(w4(q[2], E)), 0x04040404u, (w4(q[n], E) >> (2 * j)) & 0x03030303u);
        const int s = sbyte<(R & 3)>(ss[H][R >> 2]);
        const uint32_t c = (uint32_t)s * 0xFCFCFCFDu + 0x80808080u;      // (128 - 3 s) in every byte
        return w3 * (uint32_t)s + c;
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        a[0] = quad<2 * S, 0>(); a[1] = quad<2 * S, 1>(); a[2] = quad<2 * S + 1, 0>(); a[3] = quad<2 * S + 1, 1>();
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = t == 0 ? sv[h][0] : t == 1 ? sv[h][1] : t == 2 ? sv[h][2] : sv[h][3];
            a[h] = hsub2(bytes_h2(w, 0x5150u), h2k(928));
            a[2 + h] = hsub2(bytes_h2(w, 0x5352u), h2k(928));
            f[h] = f16bits(dd[h]);
        }
    }
};

#define GQ_IQ3S8_SMEM_BYTES 2048
// one entry of the int8 IQ3_S shared-memory grid: the four magnitude bytes in quad byte order (0,2,1,3)
GQ_HD inline uint32_t iq3s_grid_entry8(uint32_t w) { return prmt(w, 0u, 0x3120u); }
// bit i (0..3) of a sign nibble to bit 0 of byte (0,2,1,3)[i]
GQ_HD inline uint32_t spread_sign(uint32_t nib) { return (nib * (1u | (1u << 15) | (1u << 6) | (1u << 21))) & 0x01010101u; }

// ---- IQ3_S ----------------------------------------------------------------------------------------
template <>
struct Dec8<GQ_IQ3_S> {
    static constexpr int SCHEME = GQ_S32;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint4 q[2];      // 16 grid-index bytes per row (byte r = run r)
    uint4 sg[2];     // 16 sign nibbles per row (one per byte: the lane's four signs of run r)
    uint2 qh[2];     // the eight qh bytes per row, pre-shifted by t
    uint32_t sce[2], sco[2], dd[2];   // 1 + 2 s of the even / odd sub-blocks, one per byte
    const uint32_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        grid = aux.grid;
        const int t = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            q[h] = ld16(slab + 512 * h + 16 * lane);
            uint4 s = ld16(slab + 1024 + 32 * row + 16 * (t >> 1));
            const int sh = 4 * (t & 1);
            s.x = (s.x >> sh) & 0x0f0f0f0fu; s.y = (s.y >> sh) & 0x0f0f0f0fu; s.z = (s.z >> sh) & 0x0f0f0f0fu; s.w = (s.w >> sh) & 0x0f0f0f0fu;
            sg[h] = s;
            uint2 hq = ld8(slab + 1536 + 8 * row);
            hq.x >>= t; hq.y >>= t;
            qh[h] = hq;
            const uint32_t scw = ld4(slab + 1664 + 4 * row);
            sce[h] = (scw & 0x0f0f0f0fu) * 2u + 0x01010101u;
            sco[h] = ((scw >> 4) & 0x0f0f0f0fu) * 2u + 0x01010101u;
            dd[h] = ld2(slab + 1728 + 2 * row);
        }
    }
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        constexpr int ib = R >> 1, u = R & 1;
        const uint32_t idxb = (uint32_t)ubyte<(R & 3)>(w4(q[H], R >> 2));
        const uint32_t hw = (ib < 4) ? qh[H].x : qh[H].y;
        const uint32_t idx = or_and(idxb, shl_c<8 - (8 * (ib & 3) + 4 * u)>(hw), 0x100u);
        const uint32_t e = grid[idx];
        const uint32_t one = spread_sign((uint32_t)ubyte<(R & 3)>(w4(sg[H], R >> 2)));
        return (e ^ (one * 0xFFu)) + one;       // negated bytes where the sign bit is set
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        a[0] = quad<2 * S, 0>(); a[1] = quad<2 * S, 1>(); a[2] = quad<2 * S + 1, 0>(); a[3] = quad<2 * S + 1, 1>();
    }
    template <int S>
    GQ_HD void iscale(int &s0, int &s1) const {
        s0 = ubyte<(S >> 1)>((S & 1) ? sco[0] : sce[0]);
        s1 = ubyte<(S >> 1)>((S & 1) ? sco[1] : sce[1]);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
};

// ---- IQ3_XXS ---------------------------------------------------------------------------------------
// Shared memory: the 256 grid words.  The lane's four sign bits come from the stored 7-bit index by arithmetic (the index
// with its parity as bit 7, then the lane's nibble): a 128-entry table of them in shared memory was measured 12-14 %
// slower — with the grid lookups the type is bound by shared-memory gathers, not by the integer pipe.
// `r`: the sign-and-scale word rotated so that the lane's index sits at bits 3..9; shn: 4 x (t & 1).
GQ_HD inline uint32_t sign_index_quad(uint32_t r, int shn) {
    const uint32_t f = (r >> 3) & 0x7Fu;
    const uint32_t mask = f | (popc32(f) << 7);          // bits above 7 fall outside the nibble
    return spread_sign((mask >> shn) & 0xFu);
}

template <>
struct Dec8<GQ_IQ3_XXS> {
    static constexpr int SCHEME = GQ_S32;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint4 q[2];          // 16 grid-index bytes per row (byte r = run r)
    uint32_t sw[2][8];   // the sign-and-scale word of each sub-block
    uint32_t dd[2];
    int rot0, rot1;      // rotate counts that bring the lane's sign index of the first / second run of a sub-block to bits 3..9
    int shn;             // 4 (t & 1): the lane's nibble of an 8-bit sign mask
    const uint32_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        grid = aux.grid;
        const int t = lane & 3;
        shn = 4 * (t & 1);
        rot0 = (7 * (t >> 1) - 3) & 31;
        rot1 = 7 * (2 + (t >> 1)) - 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            q[h] = ld16(slab + 512 * h + 16 * lane);
            const uint4 a = ld16(slab + 1024 + 32 * row), b = ld16(slab + 1040 + 32 * row);
            sw[h][0] = a.x; sw[h][1] = a.y; sw[h][2] = a.z; sw[h][3] = a.w;
            sw[h][4] = b.x; sw[h][5] = b.y; sw[h][6] = b.z; sw[h][7] = b.w;
            dd[h] = ld2(slab + 1536 + 2 * row);
        }
    }
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        const uint32_t e = grid[(uint32_t)ubyte<(R & 3)>(w4(q[H], R >> 2))];
        const uint32_t w = sw[H][R >> 1];
        const uint32_t one = sign_index_quad(rotr32(w, (R & 1) ? rot1 : rot0), shn);
        return (e ^ (one * 0xFFu)) + one;       // negated bytes where the sign bit is set
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        a[0] = quad<2 * S, 0>(); a[1] = quad<2 * S, 1>(); a[2] = quad<2 * S + 1, 0>(); a[3] = quad<2 * S + 1, 1>();
    }
    template <int S>
    GQ_HD void iscale(int &s0, int &s1) const {
        s0 = (int)(2u * (sw[0][S] >> 28) + 1u);
        s1 = (int)(2u * (sw[1][S] >> 28) + 1u);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.25f * f16bits(dd[0]); d1 = 0.25f * f16bits(dd[1]); }
};

// ---- IQ2_XXS / IQ2_XS / IQ2_S --------------------------------------------------------------------------
// A grid entry holds eight magnitudes; the lanes t = 0, 1 (2, 3) of a row share the entry of the first (second) eight
// weights of a run and take its word t & 1.  Shared memory: the grid as two words per entry, each in quad byte order;
// the 7-bit sign indices of IQ2_XXS and IQ2_XS are turned into masks by arithmetic as for IQ3_XXS.
// weight = d (2 s + 1) / 8 x magnitude x sign (gguf-plugin/gluon/iq2.py:6-23).

// bytes tp, 2 + tp of two words -> one word (runtime tp): the even or the odd bytes of eight
GQ_HD inline uint32_t pick_alt_bytes(uint32_t a, uint32_t b, int tp) { return prmt(a, b, 0x6420u + 0x1111u * (uint32_t)tp); }

template <>
struct Dec8<GQ_IQ2_XXS> {
    static constexpr int SCHEME = GQ_S32;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint32_t q[2][4];    // grid-index byte of run r in byte r & 3 of word r >> 2
    uint32_t sw[2][8];   // the sign-and-scale word of each sub-block
    uint32_t dd[2];
    int rot0, rot1, shn;
    const uint8_t *grid;            // offset by the lane's half of an entry
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        const int t = lane & 3, tp = t >> 1;
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
        shn = 4 * (t & 1);
        rot0 = (7 * tp - 3) & 31;
        rot1 = 7 * (2 + tp) - 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint4 ia = ld16(slab + 32 * row), ib = ld16(slab + 32 * row + 16);
            // index word of sub-block ib: bytes l = 0..3; run 2 ib + u takes byte 2 u + tp
            q[h][0] = pick_alt_bytes(ia.x, ia.y, tp); q[h][1] = pick_alt_bytes(ia.z, ia.w, tp);
            q[h][2] = pick_alt_bytes(ib.x, ib.y, tp); q[h][3] = pick_alt_bytes(ib.z, ib.w, tp);
            const uint4 a = ld16(slab + 512 + 32 * row), b = ld16(slab + 528 + 32 * row);
            sw[h][0] = a.x; sw[h][1] = a.y; sw[h][2] = a.z; sw[h][3] = a.w;
            sw[h][4] = b.x; sw[h][5] = b.y; sw[h][6] = b.z; sw[h][7] = b.w;
            dd[h] = ld2(slab + 1024 + 2 * row);
        }
    }
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + 8 * (uint32_t)ubyte<(R & 3)>(q[H][R >> 2]));
        const uint32_t w = sw[H][R >> 1];
        const uint32_t one = sign_index_quad(rotr32(w, (R & 1) ? rot1 : rot0), shn);
        return (e ^ (one * 0xFFu)) + one;
    }
    template <int S>
    GQ_HD void step(uint32_t (&a)[4]) const {
        a[0] = quad<2 * S, 0>(); a[1] = quad<2 * S, 1>(); a[2] = quad<2 * S + 1, 0>(); a[3] = quad<2 * S + 1, 1>();
    }
    template <int S>
    GQ_HD void iscale(int &s0, int &s1) const {
        s0 = (int)(2u * (sw[0][S] >> 28) + 1u);
        s1 = (int)(2u * (sw[1][S] >> 28) + 1u);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
};

// the eight scale bytes of a row (a nibble per run of 16) -> 2 s + 1 of the even runs and of the odd runs, one per byte
GQ_HD inline void iq2_run_scales(uint2 w, uint32_t (&even)[2], uint32_t (&odd)[2]) {
    even[0] = (w.x & 0x0f0f0f0fu) * 2u + 0x01010101u; even[1] = (w.y & 0x0f0f0f0fu) * 2u + 0x01010101u;
    odd[0] = ((w.x >> 4) & 0x0f0f0f0fu) * 2u + 0x01010101u; odd[1] = ((w.y >> 4) & 0x0f0f0f0fu) * 2u + 0x01010101u;
}

template <>
struct Dec8<GQ_IQ2_XS> {
    static constexpr int SCHEME = GQ_S16;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint32_t v[2][8];    // the halfword (9-bit grid index, 7-bit sign index) of run r in half r & 1 of word r >> 1
    uint32_t sce[2][2], sco[2][2], dd[2];
    int shn;
    const uint8_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        const int t = lane & 3, tp = t >> 1;
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
        shn = 4 * (t & 1);
        const uint32_t sel = 0x5410u + 0x2222u * (uint32_t)tp;     // halfword tp of each of two words
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 w = ld16(slab + 64 * row + 16 * c);        // word j of the row = the two halfwords of run j
                v[h][2 * c] = prmt(w.x, w.y, sel);
                v[h][2 * c + 1] = prmt(w.z, w.w, sel);
            }
            iq2_run_scales(ld8(slab + 1024 + 8 * row), sce[h], sco[h]);
            dd[h] = ld2(slab + 1152 + 2 * row);
        }
    }
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        const uint32_t w = v[H][R >> 1];
        const uint32_t goff = (R & 1) ? (w >> 13) & 0xFF8u : (w << 3) & 0xFF8u;
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + goff);
        const uint32_t one = sign_index_quad((R & 1) ? w >> 22 : w >> 6, shn);
        return (e ^ (one * 0xFFu)) + one;
    }
    template <int R>
    GQ_HD void step16(uint32_t (&a)[2]) const { a[0] = quad<R, 0>(); a[1] = quad<R, 1>(); }
    template <int R>
    GQ_HD void iscale16(int &s0, int &s1) const {
        constexpr int ib = R >> 1;
        s0 = ubyte<(ib & 3)>((R & 1) ? sco[0][ib >> 2] : sce[0][ib >> 2]);
        s1 = ubyte<(ib & 3)>((R & 1) ? sco[1][ib >> 2] : sce[1][ib >> 2]);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
};

template <>
struct Dec8<GQ_IQ2_S> {
    static constexpr int SCHEME = GQ_S16;
    static constexpr bool A_SIGNED = true;
    static constexpr int NCORR = 0;
    uint32_t q[2][4];    // low grid-index byte of run r in byte r & 3 of word r >> 2
    uint32_t sg[2][4];   // the lane's sign nibble of run r, same place
    uint2 qh[2];         // the eight qh bytes per row, shifted so that the lane's pair of bits of run 2 ib + u sits at bit 4 u of byte ib
    uint32_t sce[2][2], sco[2][2], dd[2];
    const uint8_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        const int t = lane & 3, tp = t >> 1, sh = 4 * (t & 1);
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint4 ia = ld16(slab + 32 * row), ib = ld16(slab + 32 * row + 16);
            q[h][0] = pick_alt_bytes(ia.x, ia.y, tp); q[h][1] = pick_alt_bytes(ia.z, ia.w, tp);
            q[h][2] = pick_alt_bytes(ib.x, ib.y, tp); q[h][3] = pick_alt_bytes(ib.z, ib.w, tp);
            const uint4 sa = ld16(slab + 512 + 32 * row), sb = ld16(slab + 512 + 32 * row + 16);
            sg[h][0] = (pick_alt_bytes(sa.x, sa.y, tp) >> sh) & 0x0f0f0f0fu; sg[h][1] = (pick_alt_bytes(sa.z, sa.w, tp) >> sh) & 0x0f0f0f0fu;
            sg[h][2] = (pick_alt_bytes(sb.x, sb.y, tp) >> sh) & 0x0f0f0f0fu; sg[h][3] = (pick_alt_bytes(sb.z, sb.w, tp) >> sh) & 0x0f0f0f0fu;
            uint2 hq = ld8(slab + 1024 + 8 * row);
            hq.x >>= 2 * tp; hq.y >>= 2 * tp;
            qh[h] = hq;
            iq2_run_scales(ld8(slab + 1152 + 8 * row), sce[h], sco[h]);
            dd[h] = ld2(slab + 1280 + 2 * row);
        }
    }
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        constexpr int ib = R >> 1, u = R & 1;
        const uint32_t idxb = (uint32_t)ubyte<(R & 3)>(q[H][R >> 2]);
        const uint32_t hw = (ib < 4) ? qh[H].x : qh[H].y;
        const uint32_t idx = or_and(idxb, shl_c<8 - (8 * (ib & 3) + 4 * u)>(hw), 0x300u);
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + 8 * idx);
        const uint32_t one = spread_sign((uint32_t)ubyte<(R & 3)>(sg[H][R >> 2]));
        return (e ^ (one * 0xFFu)) + one;
    }
    template <int R>
    GQ_HD void step16(uint32_t (&a)[2]) const { a[0] = quad<R, 0>(); a[1] = quad<R, 1>(); }
    template <int R>
    GQ_HD void iscale16(int &s0, int &s1) const {
        constexpr int ib = R >> 1;
        s0 = ubyte<(ib & 3)>((R & 1) ? sco[0][ib >> 2] : sce[0][ib >> 2]);
        s1 = ubyte<(ib & 3)>((R & 1) ? sco[1][ib >> 2] : sce[1][ib >> 2]);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
};

// ---- IQ1_M: weight = d (2 s + 1) (g + delta), g in {-1, 0, 1} from a 2048-entry grid of eight, delta = +-1/8 per group of
// eight, a 3-bit scale per 16 weights, the fp16 d spread over the top nibbles of the four scale halfwords (gguf-py
// IQ1_M.dequantize_blocks; the reference has no kernel of its own for this type).  In eighths the weight is 8 g +- 1; the
// grid in shared memory holds 8 g + 16 (bytes 8, 16, 24), so that adding +-1 to all four bytes of a word at once never
// carries, and the constant 16 leaves through the correction MMA (run scales against the run sums). ----
template <>
struct Dec8<GQ_IQ1_M> {
    static constexpr int SCHEME = GQ_S16;
    static constexpr bool A_SIGNED = false;
    static constexpr int NCORR = 1;
    uint32_t q[2][4];    // low grid-index byte of run r in byte r & 3 of word r >> 2
    uint32_t qn[2][4];   // the run's qh nibble, same place: bits 0..2 the index bits 8..10, bit 3 the sign of delta
    uint2 sc[2];         // the four scale halfwords of a row
    uint32_t dd[2];
    int t;
    const uint8_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux8 &aux) {
        t = lane & 3;
        const int tp = t >> 1;
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint4 ia = ld16(slab + 32 * row), ib = ld16(slab + 32 * row + 16);
            q[h][0] = pick_alt_bytes(ia.x, ia.y, tp); q[h][1] = pick_alt_bytes(ia.z, ia.w, tp);
            q[h][2] = pick_alt_bytes(ib.x, ib.y, tp); q[h][3] = pick_alt_bytes(ib.z, ib.w, tp);
            const uint4 hq = ld16(slab + 512 + 16 * row);          // byte r: the nibbles of groups 2 r (low) and 2 r + 1
            qn[h][0] = (hq.x >> (4 * tp)) & 0x0f0f0f0fu; qn[h][1] = (hq.y >> (4 * tp)) & 0x0f0f0f0fu;
            qn[h][2] = (hq.z >> (4 * tp)) & 0x0f0f0f0fu; qn[h][3] = (hq.w >> (4 * tp)) & 0x0f0f0f0fu;
            const uint2 w = ld8(slab + 768 + 8 * row);
            sc[h] = w;
            dd[h] = ((w.x >> 12) & 0xFu) | ((w.x >> 24) & 0xF0u) | ((w.y >> 4) & 0xF00u) | ((w.y >> 16) & 0xF000u);
        }
    }
    template <int R, int H>
    GQ_HD uint32_t quad() const {
        const uint32_t idxb = (uint32_t)ubyte<(R & 3)>(q[H][R >> 2]);
        const uint32_t nb = (uint32_t)ubyte<(R & 3)>(qn[H][R >> 2]);
        const uint32_t idx = or_and(idxb, nb << 8, 0x700u);
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + 8 * idx);
        return e + 0x01010101u - (nb >> 3) * 0x02020202u;
    }
    template <int R>
    GQ_HD void step16(uint32_t (&a)[2]) const { a[0] = quad<R, 0>(); a[1] = quad<R, 1>(); }
    template <int R>
    GQ_HD void iscale16(int &s0, int &s1) const {
        constexpr int hw = R >> 2, sh = 16 * (hw & 1) + 3 * (R & 3);
        s0 = (int)(2u * ((((hw < 2) ? sc[0].x : sc[0].y) >> sh) & 7u) + 1u);
        s1 = (int)(2u * ((((hw < 2) ? sc[1].x : sc[1].y) >> sh) & 7u) + 1u);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
    // weight x 8 = field - 16: A'' = 2 s + 1 of runs 4t..4t+3 (the scale halfword t), factor 16 d / 8
    GQ_HD void corr(uint32_t (&a)[4], float (&f)[2]) const {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = (t & 2) ? sc[h].y : sc[h].x;
            const uint32_t hw = (t & 1) ? w >> 16 : w;
            const uint32_t b = (2u * (hw & 7u) + 1u) | ((2u * ((hw >> 3) & 7u) + 1u) << 8) | ((2u * ((hw >> 6) & 7u) + 1u) << 16) |
                               ((2u * ((hw >> 9) & 7u) + 1u) << 24);
            a[h] = hsub2(bytes_h2(b, 0x5150u), h2k(1024));
            a[2 + h] = hsub2(bytes_h2(b, 0x5352u), h2k(1024));
            f[h] = 2.0f * f16bits(dd[h]);
        }
    }
};

}  // namespace gq
