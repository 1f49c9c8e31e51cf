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
// Every decoder produces an EXACT integer as fp16 — the quantised field plus a power-of-two bias that
// comes for free from dropping the field into the mantissa of a constant (1024 + q for a field at bit 0,
// 64 + q at bit 4, 256 / 16 + q at bits 2 / 6), all below 2048 — and hands the scale out separately: an
// integer (or fp16 d) per 16- or 32-weight group applied to the fp32 MMA result, and the row's fp16 d per
// k-block.  Whatever is constant over a 16-weight run — that bias, the format's offset (q - 8, q - 32, ...)
// and the minimum term of Q2_K / Q4_K / Q5_K — is removed by "correction" MMAs of small exact per-run
// integers against per-run activation sums:  acc -= f[row] * sum_run A''[row][run] * Sx[run][n].
// The value arithmetic follows the formats as the reference states them (gguf-plugin/gluon/kq_ref.py:17-79,
// q2k.py:5-12, q4k.py:5-10, iq3s_int8t.py:4-11, iq4xs.py:5-11); Q4_0 / Q5_0 / IQ4_NL, which the reference
// leaves to the un-vendored plugin, follow gguf-py.
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

// fp16 magic constants: an unsigned field whose lowest bit sits at mantissa bit b reads as 2^(10-b) + field
#define GQ_MAGIC_B0 0x64006400u   // 1024 + field
#define GQ_MAGIC_B2 0x5C005C00u   // 256 + field
#define GQ_MAGIC_B4 0x54005400u   // 64 + field
#define GQ_MAGIC_B6 0x4C004C00u   // 16 + field

// the IQ4 codebook as unsigned bytes (value + 128) in four registers, filled by the kernel from the
// generated table
struct Iq4Table { uint32_t t0, t1, t2, t3; };

// natural-order nibble word through the 16-entry codebook: lo[] = low nibbles {(i0,i1), (i2,i3)}, hi[] = high
// nibbles, each as fp16 pairs of 1024 + (codebook value + 128)
GQ_HD inline void iq4_word(uint32_t w, const Iq4Table &T, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
    const uint32_t s = w & 0x77777777u;
    const uint32_t s2 = and_or(w >> 1, 0x44444444u, 0x32103210u);
    const uint32_t rl = prmt(prmt(T.t0, T.t1, s), prmt(T.t2, T.t3, s), s2);                       // bytes 0,1
    const uint32_t rh = prmt(prmt(T.t0, T.t1, s >> 16), prmt(T.t2, T.t3, s >> 16), s2 >> 16);     // bytes 2,3
    lo[0] = prmt(rl, GQ_MAGICB, 0x5250u);
    lo[1] = prmt(rh, GQ_MAGICB, 0x5250u);
    hi[0] = prmt(rl, GQ_MAGICB, 0x5351u);
    hi[1] = prmt(rh, GQ_MAGICB, 0x5351u);
}

// two bytes j0, j1 of `w` as an fp16 pair of (1024 + byte)
GQ_HD inline uint32_t bytes_h2(uint32_t w, uint32_t sel) { return prmt(w, GQ_MAGICB, sel); }

struct DecAux {
    const uint2 *grid;        // shared memory: the codebook of the type being decoded — IQ3_S (512) / IQ3_XXS (256) entries
                              // {fp16(m0,m1), fp16(m2,m3)}; IQ2_*: 8 magnitude bytes per entry, each word in quad byte order
    Iq4Table iq4;
};

template <int TYPE>
struct Dec;

// the 12 packed scale bytes of Q4_K / Q5_K -> sc[2], mn[2]: eight 6-bit values each, one per byte
GQ_HD inline void k4_scales(const uint4 &hd, uint32_t (&sc)[2], uint32_t (&mn)[2]) {
    sc[0] = hd.y & 0x3f3f3f3fu;
    mn[0] = hd.z & 0x3f3f3f3fu;
    sc[1] = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
    mn[1] = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
}

// Q4_K / Q5_K corrections for lane t (runs 4t..4t+3 = groups 2t (low nibbles, bias 1024) and 2t+1 (high, bias 64)):
// set 0 removes the bias: A'' = 16 sc | sc, factor 64 d;  set 1 is the minimum term: A'' = m, factor dmin
GQ_HD inline void k4_corr(int t, const uint32_t (&sc)[2][2], const uint32_t (&mn)[2][2], const uint32_t (&dd)[2],
                          uint32_t (&a)[2][4], float (&f)[2][2]) {
    const uint32_t j = 2 * (t & 1);
    const uint32_t s0 = 0x5050u | (j * 0x0101u), s1 = 0x5050u | ((j + 1) * 0x0101u);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t ws = (t & 2) ? sc[h][1] : sc[h][0], wm = (t & 2) ? mn[h][1] : mn[h][0];
        a[0][h] = hfma2(bytes_h2(ws, s0), h2k(16), h2k(-16384));
        a[0][2 + h] = hsub2(bytes_h2(ws, s1), h2k(1024));
        a[1][h] = hsub2(bytes_h2(wm, s0), h2k(1024));
        a[1][2 + h] = hsub2(bytes_h2(wm, s1), h2k(1024));
        f[0][h] = 64.0f * f16lo(dd[h]);
        f[1][h] = f16hi(dd[h]);
    }
}

// ---- Q4_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q4_K> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 2;
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
            k4_scales(hd, sc[h], mn[h]);
        }
    }
    // run pair P = (2P, 2P+1): qs group c = P>>1, nibble half = P&1, u = run&1
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int c = P >> 1, hi = P & 1;
        constexpr uint32_t mask = hi ? 0x00f000f0u : 0x000f000fu, magic = hi ? GQ_MAGIC_B4 : GQ_MAGIC_B0;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = w4(q[c], 2 * h + u);
                a[u][h] = and_or(w, mask, magic);
                a[u][2 + h] = and_or(w >> 8, mask, magic);
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = byte_f32<(G & 3)>(sc[0][G >> 2]);
        s1 = byte_f32<(G & 3)>(sc[1][G >> 2]);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    GQ_HD void corr(uint32_t (&a)[2][4], float (&f)[2][2]) const { k4_corr(t, sc, mn, dd, a, f); }
    // for the dequantise-to-fp16 path: integer weight of run R = fragment value - offs<R>();  w = that * (scale * d) - minterm
    static constexpr bool HAS_MIN = true;
    template <int R> static constexpr float offs() { return ((R >> 1) & 1) ? 64.0f : 1024.0f; }
    template <int G>
    GQ_HD void minterm(float &m0, float &m1) const {
        m0 = f16hi(dd[0]) * byte_f32<(G & 3)>(mn[0][G >> 2]);
        m1 = f16hi(dd[1]) * byte_f32<(G & 3)>(mn[1][G >> 2]);
    }
};

// ---- Q5_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q5_K> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 2;
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
            k4_scales(hd, sc[h], mn[h]);
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
                    a[u][h] = or_and(and_or(w, 0x000f000fu, GQ_MAGIC_B0), shl_c<4 - ib>(H), 0x00100010u);
                    a[u][2 + h] = or_and(and_or(w8, 0x000f000fu, GQ_MAGIC_B0), shl_c<4 - ib>(H8), 0x00100010u);
                } else {
                    a[u][h] = or_and(and_or(w, 0x00f000f0u, GQ_MAGIC_B4), shl_c<8 - ib>(H), 0x01000100u);
                    a[u][2 + h] = or_and(and_or(w8, 0x00f000f0u, GQ_MAGIC_B4), shl_c<8 - ib>(H8), 0x01000100u);
                }
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = byte_f32<(G & 3)>(sc[0][G >> 2]);
        s1 = byte_f32<(G & 3)>(sc[1][G >> 2]);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    GQ_HD void corr(uint32_t (&a)[2][4], float (&f)[2][2]) const { k4_corr(t, sc, mn, dd, a, f); }
    // for the dequantise-to-fp16 path: integer weight of run R = fragment value - offs<R>();  w = that * (scale * d) - minterm
    static constexpr bool HAS_MIN = true;
    template <int R> static constexpr float offs() { return ((R >> 1) & 1) ? 64.0f : 1024.0f; }
    template <int G>
    GQ_HD void minterm(float &m0, float &m1) const {
        m0 = f16hi(dd[0]) * byte_f32<(G & 3)>(mn[0][G >> 2]);
        m1 = f16hi(dd[1]) * byte_f32<(G & 3)>(mn[1][G >> 2]);
    }
};

// ---- Q6_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q6_K> {
    static constexpr int GROUP = 16;
    static constexpr int NCORR = 1;
    uint4 q[6];
    uint4 sc[2];      // int8 scales + 128 (unsigned bytes)
    uint32_t dd[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 6; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            uint4 s = ld16(slab + 3072 + 16 * row);
            s.x ^= 0x80808080u; s.y ^= 0x80808080u; s.z ^= 0x80808080u; s.w ^= 0x80808080u;
            sc[h] = s;
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
                    a[u][h] = or_and(and_or(w, 0x000f000fu, GQ_MAGIC_B0), shl_c<4 - 2 * tp>(H), 0x00300030u);
                    a[u][2 + h] = or_and(and_or(w8, 0x000f000fu, GQ_MAGIC_B0), shl_c<4 - 2 * tp>(H8), 0x00300030u);
                } else {
                    a[u][h] = or_and(and_or(w, 0x00f000f0u, GQ_MAGIC_B4), shl_c<8 - 2 * tp>(H), 0x03000300u);
                    a[u][2 + h] = or_and(and_or(w8, 0x00f000f0u, GQ_MAGIC_B4), shl_c<8 - 2 * tp>(H8), 0x03000300u);
                }
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = byte_f32<(G & 3)>(w4(sc[0], G >> 2), 128.0f);
        s1 = byte_f32<(G & 3)>(w4(sc[1], G >> 2), 128.0f);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
    // weight = field - 32 with field biased by 1024 (low-nibble runs: t even) or 64 (high-nibble runs: t odd):
    // A'' = sc * 11 | sc, factor 96 d  (1056 = 96 * 11)
    GQ_HD void corr(uint32_t (&a)[1][4], float (&f)[1][2]) const {
        const uint32_t mult = (t & 1) ? h2k(1) : h2k(11);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = w4(sc[h], t);
            a[0][h] = hmul2(hsub2(bytes_h2(w, 0x5150u), h2k(1152)), mult);
            a[0][2 + h] = hmul2(hsub2(bytes_h2(w, 0x5352u), h2k(1152)), mult);
            f[0][h] = 96.0f * f16bits(dd[h]);
        }
    }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return (((R >> 1) & 3) >> 1) ? 96.0f : 1056.0f; }
};

// scale of 32-weight block G from a row's eight fp16 d's
template <int G>
GQ_HD inline void d8_scale(const uint4 (&d8)[2], float &s0, float &s1) {
    const uint32_t w0 = w4(d8[0], G >> 1), w1 = w4(d8[1], G >> 1);
    s0 = (G & 1) ? f16hi(w0) : f16lo(w0);
    s1 = (G & 1) ? f16hi(w1) : f16lo(w1);
}
// correction operand of the legacy types: the fp16 d of blocks 2t (runs 4t, 4t+1) and 2t+1 (runs 4t+2, 4t+3)
GQ_HD inline void d8_corr(int t, const uint4 (&d8)[2], float bias, uint32_t (&a)[1][4], float (&f)[1][2]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t w = w4(d8[h], t);
        a[0][h] = prmt(w, w, 0x1010u);
        a[0][2 + h] = prmt(w, w, 0x3232u);
        f[0][h] = bias;
    }
}

// ---- Q8_0 -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q8_0> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 1;
    uint4 q[8];
    uint4 d8[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
        t = lane & 3;
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
                const uint32_t x = w4(q[P], 2 * h + u) ^ 0x80808080u;    // int8 + 128, bytes hold weights (0,2,1,3)
                a[u][h] = prmt(x, GQ_MAGICB, 0x5250u);
                a[u][2 + h] = prmt(x, GQ_MAGICB, 0x5351u);
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const { d8_scale<G>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
    GQ_HD void corr(uint32_t (&a)[1][4], float (&f)[1][2]) const { d8_corr(t, d8, 1152.0f, a, f); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 1152.0f; }
};

// ---- Q4_0 (18-byte blocks: d, 16 nibble bytes): exact centring, no correction ------------------------
template <>
struct Dec<GQ_Q4_0> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 0;
    uint4 q[4];
    uint4 d8[2];
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
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
            const uint32_t w = w4(q[P >> 1], 2 * h + (P & 1)), w8 = w >> 8;
            a[0][h] = hsub2(and_or(w, 0x000f000fu, GQ_MAGIC_B0), h2k(1032));
            a[0][2 + h] = hsub2(and_or(w8, 0x000f000fu, GQ_MAGIC_B0), h2k(1032));
            a[1][h] = hsub2(and_or(w, 0x00f000f0u, GQ_MAGIC_B4), h2k(72));
            a[1][2 + h] = hsub2(and_or(w8, 0x00f000f0u, GQ_MAGIC_B4), h2k(72));
        }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const { d8_scale<G>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};

// ---- IQ4_NL (18-byte blocks: d, 16 codebook-index nibble bytes) --------------------------------------
template <>
struct Dec<GQ_IQ4_NL> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 1;
    uint4 q[4];
    uint4 d8[2];
    Iq4Table tab;
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        tab = aux.iq4;
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) d8[h] = ld16(slab + 2048 + 16 * ((lane >> 2) + 8 * h));
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
    GQ_HD void scale(float &s0, float &s1) const { d8_scale<G>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
    GQ_HD void corr(uint32_t (&a)[1][4], float (&f)[1][2]) const { d8_corr(t, d8, 1152.0f, a, f); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 1152.0f; }
};

// ---- Q5_0 (22-byte blocks: d, qh u32, 16 nibble bytes): exact centring, no correction -----------------
template <>
struct Dec<GQ_Q5_0> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 0;
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
            a[0][h] = hsub2(or_and(and_or(w, 0x000f000fu, GQ_MAGIC_B0), zl, 0x00100010u), h2k(1040));
            a[0][2 + h] = hsub2(or_and(and_or(w8, 0x000f000fu, GQ_MAGIC_B0), zl >> 2, 0x00100010u), h2k(1040));
            a[1][h] = hsub2(or_and(and_or(w, 0x00f000f0u, GQ_MAGIC_B4), zh, 0x01000100u), h2k(80));
            a[1][2 + h] = hsub2(or_and(and_or(w8, 0x00f000f0u, GQ_MAGIC_B4), zh >> 2, 0x01000100u), h2k(80));
        }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const { d8_scale<G>(d8, s0, s1); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 1.0f; d1 = 1.0f; }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};

// ---- IQ4_XS ---------------------------------------------------------------------------------------
template <>
struct Dec<GQ_IQ4_XS> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 1;
    uint4 q[4];
    uint32_t ls[2][2];   // the eight 6-bit sub-block scales of a row as bytes (value + 32)
    uint32_t dd[2];
    Iq4Table tab;
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        tab = aux.iq4;
        t = lane & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = ld16(slab + 512 * c + 16 * lane);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint2 hd = ld8(slab + 2048 + 8 * ((lane >> 2) + 8 * h));
            dd[h] = hd.x;
            const uint32_t e = hd.y & 0x0f0f0f0fu, o = (hd.y >> 4) & 0x0f0f0f0fu;   // groups 0,2,4,6 | 1,3,5,7
            const uint32_t sh = hd.x >> 16;
            // the 2-bit high parts: groups 0..3 from bits 0..7, groups 4..7 from bits 8..15, one per byte
            uint32_t a0 = (sh | (sh << 12)) & 0x000f000fu;
            a0 = (a0 | (a0 << 6)) & 0x03030303u;
            const uint32_t s8 = sh >> 8;
            uint32_t a1 = (s8 | (s8 << 12)) & 0x000f000fu;
            a1 = (a1 | (a1 << 6)) & 0x03030303u;
            ls[h][0] = prmt(e, o, 0x5140u) | (a0 << 4);
            ls[h][1] = prmt(e, o, 0x7362u) | (a1 << 4);
        }
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
        s0 = byte_f32<(G & 3)>(ls[0][G >> 2], 32.0f);
        s1 = byte_f32<(G & 3)>(ls[1][G >> 2], 32.0f);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    // value = 1024 + (codebook + 128): A'' = ls of groups 2t, 2t+1, factor 1152 d
    GQ_HD void corr(uint32_t (&a)[1][4], float (&f)[1][2]) const {
        const uint32_t j = 2 * (t & 1);
        const uint32_t s0 = 0x5050u | (j * 0x0101u), s1 = 0x5050u | ((j + 1) * 0x0101u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = (t & 2) ? ls[h][1] : ls[h][0];
            a[0][h] = hsub2(bytes_h2(w, s0), h2k(1056));
            a[0][2 + h] = hsub2(bytes_h2(w, s1), h2k(1056));
            f[0][h] = 1152.0f * f16lo(dd[h]);
        }
    }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 1152.0f; }
};

// multipliers bias/16 of the four runs 4t..4t+3 of the 2-bit types: t even -> bit pairs 0,1 (bias 1024, 256),
// t odd -> bit pairs 2,3 (bias 64, 16)
GQ_HD inline void q23_mult(int t, uint32_t &m01, uint32_t &m23) {
    m01 = (t & 1) ? h2k(4) : h2k(64);
    m23 = (t & 1) ? h2k(1) : h2k(16);
}

// ---- Q2_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q2_K> {
    static constexpr int GROUP = 16;
    static constexpr int NCORR = 2;
    uint4 q[2];
    uint4 sc[2], mn[2];   // low / high nibbles of the sixteen scale bytes, one per byte
    uint32_t dd[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
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
    // run pair P: n = P>>2 (128-weight half), t' = P&3 (bit pair 2t' of each byte), runs u = 0,1
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int n = P >> 2, tp = P & 3;
        constexpr uint32_t mask = 0x00030003u << (2 * tp);
        constexpr uint32_t magic = tp == 0 ? GQ_MAGIC_B0 : tp == 1 ? GQ_MAGIC_B2 : tp == 2 ? GQ_MAGIC_B4 : GQ_MAGIC_B6;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = w4(q[n], 2 * h + u);
                a[u][h] = and_or(w, mask, magic);
                a[u][2 + h] = and_or(w >> 8, mask, magic);
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = byte_f32<(G & 3)>(w4(sc[0], G >> 2));
        s1 = byte_f32<(G & 3)>(w4(sc[1], G >> 2));
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16lo(dd[0]); d1 = f16lo(dd[1]); }
    // set 0 removes the field bias: A'' = sc * bias/16, factor 16 d;  set 1 is the minimum term: A'' = m, factor dmin
    GQ_HD void corr(uint32_t (&a)[2][4], float (&f)[2][2]) const {
        uint32_t m01, m23;
        q23_mult(t, m01, m23);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t ws = w4(sc[h], t), wm = w4(mn[h], t);
            a[0][h] = hmul2(hsub2(bytes_h2(ws, 0x5150u), h2k(1024)), m01);
            a[0][2 + h] = hmul2(hsub2(bytes_h2(ws, 0x5352u), h2k(1024)), m23);
            a[1][h] = hsub2(bytes_h2(wm, 0x5150u), h2k(1024));
            a[1][2 + h] = hsub2(bytes_h2(wm, 0x5352u), h2k(1024));
            f[0][h] = 16.0f * f16lo(dd[h]);
            f[1][h] = f16hi(dd[h]);
        }
    }
    static constexpr bool HAS_MIN = true;
    template <int R> static constexpr float offs() { return float(1024 >> (2 * ((R >> 1) & 3))); }
    template <int G>
    GQ_HD void minterm(float &m0, float &m1) const {
        m0 = f16hi(dd[0]) * byte_f32<(G & 3)>(w4(mn[0], G >> 2));
        m1 = f16hi(dd[1]) * byte_f32<(G & 3)>(w4(mn[1], G >> 2));
    }
};

// ---- Q3_K -----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_Q3_K> {
    static constexpr int GROUP = 16;
    static constexpr int NCORR = 2;
    uint4 q[3];
    uint32_t sv[2][4];   // the sixteen 6-bit scales of a row as bytes (value + 32)
    uint32_t dd[2];
    int t;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &) {
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
            dd[h] = ld2(slab + 1536 + 192 + 2 * row);
        }
    }
    template <int P>
    GQ_HD void pair(uint32_t (&a)[2][4]) const {
        constexpr int n = P >> 2, tp = P & 3;
        constexpr uint32_t mask = 0x00030003u << (2 * tp), hmsk = 0x00040004u << (2 * tp);
        constexpr uint32_t magic = tp == 0 ? GQ_MAGIC_B0 : tp == 1 ? GQ_MAGIC_B2 : tp == 2 ? GQ_MAGIC_B4 : GQ_MAGIC_B6;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = w4(q[n], 2 * h + u), H = w4(q[2], 2 * h + u);
                a[u][h] = or_and(and_or(w, mask, magic), shl_c<tp + 2 - 4 * n>(H), hmsk);
                a[u][2 + h] = or_and(and_or(w >> 8, mask, magic), shl_c<tp + 2 - 4 * n>(H >> 8), hmsk);
            }
    }
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = byte_f32<(G & 3)>(sv[0][G >> 2], 32.0f);
        s1 = byte_f32<(G & 3)>(sv[1][G >> 2], 32.0f);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
    // weight = (q2 + 4 hb) - 4 with the 3-bit field biased by 1024 / 256 / 64 / 16:
    // set 0: A'' = sc * bias/16, factor 16 d;  set 1: A'' = sc, factor 4 d
    GQ_HD void corr(uint32_t (&a)[2][4], float (&f)[2][2]) const {
        uint32_t m01, m23;
        q23_mult(t, m01, m23);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = t == 0 ? sv[h][0] : t == 1 ? sv[h][1] : t == 2 ? sv[h][2] : sv[h][3];
            a[1][h] = hsub2(bytes_h2(w, 0x5150u), h2k(1056));
            a[1][2 + h] = hsub2(bytes_h2(w, 0x5352u), h2k(1056));
            a[0][h] = hmul2(a[1][h], m01);
            a[0][2 + h] = hmul2(a[1][2 + h], m23);
            const float d = f16bits(dd[h]);
            f[0][h] = 16.0f * d;
            f[1][h] = 4.0f * d;
        }
    }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return float((1024 >> (2 * ((R >> 1) & 3))) + 4); }
};


// ---- IQ3_S ----------------------------------------------------------------------------------------
template <>
struct Dec<GQ_IQ3_S> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 0;
    uint4 q[2];      // 16 grid-index bytes per row (byte r = run r)
    uint4 sg[2];     // 16 sign bytes per row, pre-shifted so that the lane's nibble is the low one
    uint2 qh[2];     // the eight qh bytes per row, pre-shifted by t
    uint32_t sce[2], sco[2], dd[2];   // scale nibbles of even / odd sub-blocks, one per byte
    const uint2 *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        grid = aux.grid;
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
            const uint32_t scw = ld4(slab + 1664 + 4 * row);
            sce[h] = scw & 0x0f0f0f0fu;
            sco[h] = (scw >> 4) & 0x0f0f0f0fu;
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
    // 1 + 2 s: the nibble dropped into the mantissa of 2^24 (step 2), minus (2^24 - 1)
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        constexpr uint32_t sel = 0x7640u | (G >> 1);
        s0 = u32_as_f32(prmt((G & 1) ? sco[0] : sce[0], 0x4B800000u, sel)) - 16777215.0f;
        s1 = u32_as_f32(prmt((G & 1) ? sco[1] : sce[1], 0x4B800000u, sel)) - 16777215.0f;
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = f16bits(dd[0]); d1 = f16bits(dd[1]); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};


// ---- IQ3_XXS: d | 64 grid-index bytes | eight words of four 7-bit sign indices and a 4-bit scale ----------------
// weight = d (2 s + 1) / 4 x magnitude x sign; the eighth sign of a group of eight is the parity of the stored seven
// (gguf-plugin/gluon/iq3xxs.py:5-19)
template <>
struct Dec<GQ_IQ3_XXS> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 0;
    uint4 q[2];          // 16 grid-index bytes per row (byte r = run r)
    uint32_t sw[2][8];   // the sign-and-scale word of each sub-block
    uint32_t dd[2];
    int sh0, shn;        // 7 (t >> 1): the lane's sign index inside a half sub-block; 4 (t & 1): its nibble of the mask
    const uint2 *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        grid = aux.grid;
        const int t = lane & 3;
        sh0 = 7 * (t >> 1);
        shn = 4 * (t & 1);
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
    template <int R>
    GQ_HD void run(int h, uint32_t &a01, uint32_t &a23) const {
        const uint32_t idx = (w4(q[h], R >> 2) >> (8 * (R & 3))) & 0xFFu;
        const uint2 e = grid[idx];
        const uint32_t f = (sw[h][R >> 1] >> (14 * (R & 1) + sh0)) & 0x7Fu;
        const uint32_t mask = f | (popc32(f) << 7);          // bit 7: the parity (higher bits fall outside the nibble)
        const uint32_t nib = (mask >> shn) & 0xFu;
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
    // 2 s + 1 dropped into the mantissa of 2^23, minus 2^23
    template <int G>
    GQ_HD void scale(float &s0, float &s1) const {
        s0 = u32_as_f32(0x4B000001u + 2u * (sw[0][G] >> 28)) - 8388608.0f;
        s1 = u32_as_f32(0x4B000001u + 2u * (sw[1][G] >> 28)) - 8388608.0f;
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.25f * f16bits(dd[0]); d1 = 0.25f * f16bits(dd[1]); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};

// ---- IQ2_XXS / IQ2_XS / IQ2_S: eight magnitudes per grid entry, shared by two lanes; weight = d (2 s + 1) / 8 x
// magnitude x sign (gguf-plugin/gluon/iq2.py:6-23).  The shared-memory grid is the integer form's (bytes in quad order
// (0,2,1,3) per word); the bytes become fp16 through the 1024 + byte pattern. ----
GQ_HD inline uint32_t pick_alt_bytes16(uint32_t a, uint32_t b, int tp) { return prmt(a, b, 0x6420u + 0x1111u * (uint32_t)tp); }
// the lane's word e of a grid entry and its four sign bits -> the fp16 pairs (w0, w1), (w2, w3)
GQ_HD inline void iq2_pairs(uint32_t e, uint32_t nib, uint32_t &a01, uint32_t &a23) {
    a01 = xor_and(hsub2(prmt(e, GQ_MAGICB, 0x5250u), h2k(1024)), nib * 0x40008000u, 0x80008000u);
    a23 = xor_and(hsub2(prmt(e, GQ_MAGICB, 0x5351u), h2k(1024)), (nib >> 2) * 0x40008000u, 0x80008000u);
}
GQ_HD inline float odd_scale_f32(uint32_t s) { return u32_as_f32(0x4B000001u + 2u * s) - 8388608.0f; }    // 2 s + 1

template <>
struct Dec<GQ_IQ2_XXS> {
    static constexpr int GROUP = 32;
    static constexpr int NCORR = 0;
    uint32_t q[2][4];    // grid-index byte of run r in byte r & 3 of word r >> 2
    uint32_t sw[2][8];
    uint32_t dd[2];
    int sh0, shn;
    const uint8_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        const int t = lane & 3, tp = t >> 1;
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
        sh0 = 7 * tp;
        shn = 4 * (t & 1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint4 ia = ld16(slab + 32 * row), ib = ld16(slab + 32 * row + 16);
            q[h][0] = pick_alt_bytes16(ia.x, ia.y, tp); q[h][1] = pick_alt_bytes16(ia.z, ia.w, tp);
            q[h][2] = pick_alt_bytes16(ib.x, ib.y, tp); q[h][3] = pick_alt_bytes16(ib.z, ib.w, tp);
            const uint4 a = ld16(slab + 512 + 32 * row), b = ld16(slab + 528 + 32 * row);
            sw[h][0] = a.x; sw[h][1] = a.y; sw[h][2] = a.z; sw[h][3] = a.w;
            sw[h][4] = b.x; sw[h][5] = b.y; sw[h][6] = b.z; sw[h][7] = b.w;
            dd[h] = ld2(slab + 1024 + 2 * row);
        }
    }
    template <int R>
    GQ_HD void run(int h, uint32_t &a01, uint32_t &a23) const {
        const uint32_t idx = (q[h][R >> 2] >> (8 * (R & 3))) & 0xFFu;
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + 8 * idx);
        const uint32_t f = (sw[h][R >> 1] >> (14 * (R & 1) + sh0)) & 0x7Fu;
        const uint32_t mask = f | (popc32(f) << 7);
        iq2_pairs(e, (mask >> shn) & 0xFu, a01, a23);
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
    GQ_HD void scale(float &s0, float &s1) const { s0 = odd_scale_f32(sw[0][G] >> 28); s1 = odd_scale_f32(sw[1][G] >> 28); }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};

template <>
struct Dec<GQ_IQ2_XS> {
    static constexpr int GROUP = 16;
    static constexpr int NCORR = 0;
    uint32_t v[2][8];    // the halfword (9-bit grid index, 7-bit sign index) of run r in half r & 1 of word r >> 1
    uint2 sc[2];         // scales[8] of the row: byte ib = nibbles of runs 2 ib, 2 ib + 1
    uint32_t dd[2];
    int shn;
    const uint8_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        const int t = lane & 3, tp = t >> 1;
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
        shn = 4 * (t & 1);
        const uint32_t sel = 0x5410u + 0x2222u * (uint32_t)tp;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 w = ld16(slab + 64 * row + 16 * c);
                v[h][2 * c] = prmt(w.x, w.y, sel);
                v[h][2 * c + 1] = prmt(w.z, w.w, sel);
            }
            sc[h] = ld8(slab + 1024 + 8 * row);
            dd[h] = ld2(slab + 1152 + 2 * row);
        }
    }
    template <int R>
    GQ_HD void run(int h, uint32_t &a01, uint32_t &a23) const {
        const uint32_t hw = (v[h][R >> 1] >> (16 * (R & 1))) & 0xFFFFu;
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + 8 * (hw & 511u));
        const uint32_t f = hw >> 9;
        const uint32_t mask = f | (popc32(f) << 7);
        iq2_pairs(e, (mask >> shn) & 0xFu, a01, a23);
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
        constexpr int ib = G >> 1, sh = 8 * (ib & 3) + 4 * (G & 1);
        s0 = odd_scale_f32((((ib < 4) ? sc[0].x : sc[0].y) >> sh) & 0xFu);
        s1 = odd_scale_f32((((ib < 4) ? sc[1].x : sc[1].y) >> sh) & 0xFu);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};

template <>
struct Dec<GQ_IQ2_S> {
    static constexpr int GROUP = 16;
    static constexpr int NCORR = 0;
    uint32_t q[2][4], sg[2][4];   // low index byte / the lane's sign nibble of run r in byte r & 3 of word r >> 2
    uint2 qh[2], sc[2];
    uint32_t dd[2];
    const uint8_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        const int t = lane & 3, tp = t >> 1, sh = 4 * (t & 1);
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint4 ia = ld16(slab + 32 * row), ib = ld16(slab + 32 * row + 16);
            q[h][0] = pick_alt_bytes16(ia.x, ia.y, tp); q[h][1] = pick_alt_bytes16(ia.z, ia.w, tp);
            q[h][2] = pick_alt_bytes16(ib.x, ib.y, tp); q[h][3] = pick_alt_bytes16(ib.z, ib.w, tp);
            const uint4 sa = ld16(slab + 512 + 32 * row), sb = ld16(slab + 512 + 32 * row + 16);
            sg[h][0] = (pick_alt_bytes16(sa.x, sa.y, tp) >> sh) & 0x0f0f0f0fu; sg[h][1] = (pick_alt_bytes16(sa.z, sa.w, tp) >> sh) & 0x0f0f0f0fu;
            sg[h][2] = (pick_alt_bytes16(sb.x, sb.y, tp) >> sh) & 0x0f0f0f0fu; sg[h][3] = (pick_alt_bytes16(sb.z, sb.w, tp) >> sh) & 0x0f0f0f0fu;
            uint2 hq = ld8(slab + 1024 + 8 * row);
            hq.x >>= 2 * tp; hq.y >>= 2 * tp;
            qh[h] = hq;
            sc[h] = ld8(slab + 1152 + 8 * row);
            dd[h] = ld2(slab + 1280 + 2 * row);
        }
    }
    template <int R>
    GQ_HD void run(int h, uint32_t &a01, uint32_t &a23) const {
        constexpr int ib = R >> 1, u = R & 1;
        const uint32_t idxb = (q[h][R >> 2] >> (8 * (R & 3))) & 0xFFu;
        const uint32_t hw = (ib < 4) ? qh[h].x : qh[h].y;
        const uint32_t idx = or_and(idxb, shl_c<8 - (8 * (ib & 3) + 4 * u)>(hw), 0x300u);
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + 8 * idx);
        iq2_pairs(e, (sg[h][R >> 2] >> (8 * (R & 3))) & 0xFu, a01, a23);
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
        constexpr int ib = G >> 1, sh = 8 * (ib & 3) + 4 * (G & 1);
        s0 = odd_scale_f32((((ib < 4) ? sc[0].x : sc[0].y) >> sh) & 0xFu);
        s1 = odd_scale_f32((((ib < 4) ? sc[1].x : sc[1].y) >> sh) & 0xFu);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};

// ---- IQ1_M (see gq_decode8.cuh for the format): the shared-memory grid holds 8 g + 16 per weight as bytes; the bytes become
// fp16 through the 1024 + byte pattern and the subtraction takes 1024 + 16 -+ 1 off, leaving 8 g +- 1 exactly ----
template <>
struct Dec<GQ_IQ1_M> {
    static constexpr int GROUP = 16;
    static constexpr int NCORR = 0;
    uint32_t q[2][4], qn[2][4];
    uint2 sc[2];
    uint32_t dd[2];
    const uint8_t *grid;
    GQ_HD void load(const uint8_t *slab, int lane, const DecAux &aux) {
        const int t = lane & 3, tp = t >> 1;
        grid = reinterpret_cast<const uint8_t *>(aux.grid) + 4 * (t & 1);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = (lane >> 2) + 8 * h;
            const uint4 ia = ld16(slab + 32 * row), ib = ld16(slab + 32 * row + 16);
            q[h][0] = pick_alt_bytes16(ia.x, ia.y, tp); q[h][1] = pick_alt_bytes16(ia.z, ia.w, tp);
            q[h][2] = pick_alt_bytes16(ib.x, ib.y, tp); q[h][3] = pick_alt_bytes16(ib.z, ib.w, tp);
            const uint4 hq = ld16(slab + 512 + 16 * row);
            qn[h][0] = (hq.x >> (4 * tp)) & 0x0f0f0f0fu; qn[h][1] = (hq.y >> (4 * tp)) & 0x0f0f0f0fu;
            qn[h][2] = (hq.z >> (4 * tp)) & 0x0f0f0f0fu; qn[h][3] = (hq.w >> (4 * tp)) & 0x0f0f0f0fu;
            const uint2 w = ld8(slab + 768 + 8 * row);
            sc[h] = w;
            dd[h] = ((w.x >> 12) & 0xFu) | ((w.x >> 24) & 0xF0u) | ((w.y >> 4) & 0xF00u) | ((w.y >> 16) & 0xF000u);
        }
    }
    template <int R>
    GQ_HD void run(int h, uint32_t &a01, uint32_t &a23) const {
        const uint32_t idxb = (q[h][R >> 2] >> (8 * (R & 3))) & 0xFFu;
        const uint32_t nb = (qn[h][R >> 2] >> (8 * (R & 3))) & 0xFu;
        const uint32_t e = *reinterpret_cast<const uint32_t *>(grid + 8 * (idxb | ((nb & 7u) << 8)));
        const uint32_t c = h2k(1039) + (nb >> 3) * 0x00020002u;          // fp16 1039 (delta > 0: field - 15) or 1041 (field - 17)
        a01 = hsub2(prmt(e, GQ_MAGICB, 0x5250u), c);
        a23 = hsub2(prmt(e, GQ_MAGICB, 0x5351u), c);
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
        constexpr int hw = G >> 2, sh = 16 * (hw & 1) + 3 * (G & 3);
        s0 = odd_scale_f32((((hw < 2) ? sc[0].x : sc[0].y) >> sh) & 7u);
        s1 = odd_scale_f32((((hw < 2) ? sc[1].x : sc[1].y) >> sh) & 7u);
    }
    GQ_HD void kscale(float &d0, float &d1) const { d0 = 0.125f * f16bits(dd[0]); d1 = 0.125f * f16bits(dd[1]); }
    static constexpr bool HAS_MIN = false;
    template <int R> static constexpr float offs() { return 0.0f; }
};

// one entry of the IQ3_S / IQ3_XXS shared-memory grid: the four magnitude bytes of a grid word as two fp16 pairs
GQ_HD inline uint2 iq3s_grid_entry(uint32_t w) {
    uint2 e;
    e.x = h2_as_u32(__floats2half2_rn((float)(w & 0xFF), (float)((w >> 8) & 0xFF)));
    e.y = h2_as_u32(__floats2half2_rn((float)((w >> 16) & 0xFF), (float)(w >> 24)));
    return e;
}

}  // namespace gq
