/*
 * TEST INFRASTRUCTURE — CPU oracle for the GGUF quantized-linear path.
 *
 * A plain-C restatement of the dequantisation arithmetic of the GGML block types the
 * quantized-linear method handles (Q4_0, Q5_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ3_S,
 * IQ4_XS, and the codebook types IQ3_XXS, IQ2_XXS, IQ2_XS, IQ2_S, IQ1_M) and of the fp32 "dequantise, then
 * multiply" result they are checked against.  Nothing in
 * the shipped library links, loads or calls this file: only the tests, the smoke check and the
 * CPU-baseline leg of the benchmark use it, and only as the checker / the timed CPU figure.
 *
 * The format arithmetic lives in a third-party dependency of the reference (gguf-py, pinned
 * gguf==0.17.1 by gguf-plugin/requirements.txt:1; `gguf.quants.dequantize`).  The reference uses that
 * function as its own format reference (gguf-plugin/gluon/kq_ref.py:1-5,
 * gguf-plugin/test_gguf_rco_cpu.py:345-356, gguf-plugin/test_gluon_kq_gpu.py:123-125).  Each
 * function below states which reference lines describe the same bit mapping.  The operation order
 * reproduces gguf-py bit for bit: (d * sc) rounded to fp32 first, then times q, then minus
 * (dmin * m) (gguf-plugin/gluon/kq_ref.py:83-91); the file must be compiled with
 * -ffp-contract=off so no multiply-add is fused.
 *
 * Parity pinned: tests/test_oracle.py checks every function here against golden vectors made by
 * gguf.quants.dequantize and by the reference's own CPU model (gguf-plugin/gluon/kq_ref.py) — the
 * generating script is tests/golden/make_golden.py.
 *
 * Tables (the IQ3_S, IQ3_XXS and IQ2 grids and the IQ4 16-entry codebook) are not typed in here: the
 * caller loads them from the gguf package at run time (oracle_set_tables, oracle_set_iq_grids), as the
 * reference does (gguf-plugin/gluon/iq3s.py:41-52, gguf-plugin/gluon/iq4xs.py:190-206,
 * gguf-plugin/gluon/iq2.py:8-11, gguf-plugin/gluon/iq3xxs.py:7-8).
 */
#include <stdint.h>
#include <string.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK_K 256

enum {
    T_Q4_0 = 2, T_Q5_0 = 6, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13,
    T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ4_XS = 23,
    T_IQ1_M = 29
};

static uint8_t g_iq3s_grid[512][4];   /* magnitudes, odd 1..15 */
static int8_t g_iq4_kvalues[16];
static int g_tables_set = 0;
static uint8_t g_iq3xxs_grid[256][4], g_iq2xxs_grid[256][8], g_iq2xs_grid[512][8], g_iq2s_grid[1024][8];
static int g_iq_grids_set = 0;
static int8_t g_iq1_grid[2048][8];     /* -1, 0, 1 */
static int g_iq1_grid_set = 0;

void oracle_set_iq1_grid(const int8_t *iq1_2048x8) {
    memcpy(g_iq1_grid, iq1_2048x8, sizeof g_iq1_grid);
    g_iq1_grid_set = 1;
}

void oracle_set_iq_grids(const uint8_t *iq3xxs_256x4, const uint8_t *iq2xxs_256x8, const uint8_t *iq2xs_512x8, const uint8_t *iq2s_1024x8) {
    memcpy(g_iq3xxs_grid, iq3xxs_256x4, sizeof g_iq3xxs_grid);
    memcpy(g_iq2xxs_grid, iq2xxs_256x8, sizeof g_iq2xxs_grid);
    memcpy(g_iq2xs_grid, iq2xs_512x8, sizeof g_iq2xs_grid);
    memcpy(g_iq2s_grid, iq2s_1024x8, sizeof g_iq2s_grid);
    g_iq_grids_set = 1;
}

void oracle_set_tables(const uint8_t *iq3s_grid_512x4, const int8_t *iq4_kvalues_16) {
    memcpy(g_iq3s_grid, iq3s_grid_512x4, sizeof g_iq3s_grid);
    memcpy(g_iq4_kvalues, iq4_kvalues_16, sizeof g_iq4_kvalues);
    g_tables_set = 1;
}

/* bytes of one row segment covering 256 weights; 0 for an unknown type */
int oracle_bytes_per_256(int type) {
    switch (type) {
        case T_Q4_0: return 8 * 18;
        case T_Q5_0: return 8 * 22;
        case T_Q8_0: return 8 * 34;
        case T_Q2_K: return 84;
        case T_Q3_K: return 110;
        case T_Q4_K: return 144;
        case T_Q5_K: return 176;
        case T_Q6_K: return 210;
        case T_IQ4_NL: return 8 * 18;
        case T_IQ3_S: return 110;
        case T_IQ4_XS: return 136;
        case T_IQ3_XXS: return 98;
        case T_IQ2_XXS: return 66;
        case T_IQ2_XS: return 74;
        case T_IQ2_S: return 82;
        case T_IQ1_M: return 56;
        default: return 0;
    }
}

static float f16_to_f32(const uint8_t *p) {
    uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
    uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            man &= 0x3ff;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* ---- 32-weight block types -------------------------------------------------------------- */

/* Q4_0: d | qs[16]; weight j = low nibble of qs[j], weight 16+j = high nibble; w = d * (q - 8).
 * Not described in the reference (falls to the un-vendored plugin, gguf-prefill-dispatch.patch:32-47);
 * bit mapping from gguf-py quants.py Q4_0.dequantize_blocks. */
static void deq_q4_0(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    const uint8_t *qs = b + 2;
    for (int j = 0; j < 16; j++) {
        y[j] = d * (float)((int)(qs[j] & 0xF) - 8);
        y[16 + j] = d * (float)((int)(qs[j] >> 4) - 8);
    }
}

/* Q5_0: d | qh u32 | qs[16]; bit j of qh is bit 4 of weight j; w = d * (q - 16). */
static void deq_q5_0(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
    const uint8_t *qs = b + 6;
    for (int j = 0; j < 16; j++) {
        int lo = (qs[j] & 0xF) | (((qh >> j) & 1) << 4);
        int hi = (qs[j] >> 4) | (((qh >> (16 + j)) & 1) << 4);
        y[j] = d * (float)(lo - 16);
        y[16 + j] = d * (float)(hi - 16);
    }
}

/* Q8_0: d | int8 qs[32]; w = d * qs  (gguf-plugin/gluon/kq_ref.py:35-39). */
static void deq_q8_0(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    const int8_t *qs = (const int8_t *)(b + 2);
    for (int j = 0; j < 32; j++) y[j] = (float)qs[j] * d;
}

/* IQ4_NL: d | qs[16]; as Q4_0 with the nibble indexing the 16-entry signed codebook
 * (gguf-plugin/gluon/iq4xs.py:36,194-199). */
static void deq_iq4_nl(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    const uint8_t *qs = b + 2;
    for (int j = 0; j < 16; j++) {
        y[j] = d * (float)g_iq4_kvalues[qs[j] & 0xF];
        y[16 + j] = d * (float)g_iq4_kvalues[qs[j] >> 4];
    }
}

/* ---- 256-weight superblock types -------------------------------------------------------- */

/* Q2_K: scales[16] (low nibble scale, high nibble min, one byte per 16 weights) | qs[64] | d | dmin
 * weight 128n+32t+l = bits 2t,2t+1 of qs[32n+l]; w = (d*sc)*q - (dmin*m)
 * (gguf-plugin/gluon/q2k.py:5-12). */
static void deq_q2_k(const uint8_t *b, float *y) {
    const uint8_t *scales = b, *qs = b + 16;
    float d = f16_to_f32(b + 80), dmin = f16_to_f32(b + 82);
    for (int w = 0; w < QK_K; w++) {
        int n = w >> 7, t = (w >> 5) & 3, l = w & 31, g = w >> 4;
        float dl = d * (float)(scales[g] & 0xF);
        float ml = dmin * (float)(scales[g] >> 4);
        int q = (qs[32 * n + l] >> (2 * t)) & 3;
        y[w] = dl * (float)q - ml;
    }
}

/* Q3_K: hmask[32] | qs[64] | scales[12] | d   (gguf-plugin/gluon/kq_ref.py:40-56). */
static void deq_q3_k(const uint8_t *b, float *y) {
    const uint8_t *hmask = b, *qs = b + 32, *s = b + 96;
    float d = f16_to_f32(b + 108);
    float dl[16];
    for (int i = 0; i < 16; i++) {
        int lo = (s[i % 8] >> (4 * (i / 8))) & 0xF;
        int hi = (s[8 + i % 4] >> (2 * (i / 4))) & 3;
        int sc = (int)(int8_t)(lo | (hi << 4)) - 32;
        dl[i] = d * (float)sc;
    }
    for (int w = 0; w < QK_K; w++) {
        int nn = w >> 7, j = (w >> 5) & 3, l = w & 31;
        int hb = (hmask[l] >> (4 * nn + j)) & 1;
        int q = (int)((qs[32 * nn + l] >> (2 * j)) & 3) - (hb ? 0 : 4);
        y[w] = dl[w >> 4] * (float)q;
    }
}

/* the 12 scale bytes of Q4_K / Q5_K -> sc[8], m[8]  (gguf-plugin/gluon/kq_ref.py:17-27) */
static void scale_min_k4(const uint8_t *s, int *sc, int *mn) {
    for (int j = 0; j < 4; j++) {
        sc[j] = s[j] & 63;
        mn[j] = s[j + 4] & 63;
        sc[j + 4] = (s[j + 8] & 0xF) | ((s[j] >> 6) << 4);
        mn[j + 4] = (s[j + 8] >> 4) | ((s[j + 4] >> 6) << 4);
    }
}

/* Q4_K: d | dmin | scales[12] | qs[128]  (gguf-plugin/gluon/q4k.py:5-10). */
static void deq_q4_k(const uint8_t *b, float *y) {
    float d = f16_to_f32(b), dmin = f16_to_f32(b + 2);
    int sc[8], mn[8];
    scale_min_k4(b + 4, sc, mn);
    const uint8_t *qs = b + 16;
    for (int ib = 0; ib < 8; ib++) {
        float dl = d * (float)sc[ib], dm = dmin * (float)mn[ib];
        for (int p = 0; p < 32; p++) {
            int q = (qs[32 * (ib >> 1) + p] >> (4 * (ib & 1))) & 0xF;
            y[32 * ib + p] = dl * (float)q - dm;
        }
    }
}

/* Q5_K: d | dmin | scales[12] | qh[32] | qs[128]  (gguf-plugin/gluon/kq_ref.py:57-68). */
static void deq_q5_k(const uint8_t *b, float *y) {
    float d = f16_to_f32(b), dmin = f16_to_f32(b + 2);
    int sc[8], mn[8];
    scale_min_k4(b + 4, sc, mn);
    const uint8_t *qh = b + 16, *qs = b + 48;
    for (int ib = 0; ib < 8; ib++) {
        float dl = d * (float)sc[ib], dm = dmin * (float)mn[ib];
        for (int p = 0; p < 32; p++) {
            int q = ((qs[32 * (ib >> 1) + p] >> (4 * (ib & 1))) & 0xF) | (((qh[p] >> ib) & 1) << 4);
            y[32 * ib + p] = dl * (float)q - dm;
        }
    }
}

/* Q6_K: ql[128] | qh[64] | scales int8[16] | d  (gguf-plugin/gluon/kq_ref.py:69-79). */
static void deq_q6_k(const uint8_t *b, float *y) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    float d = f16_to_f32(b + 208);
    for (int w = 0; w < QK_K; w++) {
        int h = w >> 7, t = (w >> 5) & 3, p = w & 31;
        int q = (int)(int8_t)(((ql[64 * h + 32 * (t & 1) + p] >> (4 * (t >> 1))) & 0xF) |
                              (((qh[32 * h + p] >> (2 * t)) & 3) << 4)) - 32;
        float dl = d * (float)sc[w >> 4];
        y[w] = dl * (float)q;
    }
}

/* IQ3_S: d | qs[64] | qh[8] | signs[32] | scales[4]
 * (gguf-plugin/gluon/iq3s_int8t.py:4-11, gguf-plugin/gluon/iq3s_tile_dequant.py:29-54). */
static void deq_iq3_s(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    const uint8_t *qs = b + 2, *qh = b + 66, *signs = b + 74, *scales = b + 106;
    for (int ib = 0; ib < 8; ib++) {
        int s = (scales[ib >> 1] >> (4 * (ib & 1))) & 0xF;
        float db = d * (float)(1 + 2 * s);
        for (int k = 0; k < 8; k++) {
            int idx = qs[8 * ib + k] | (((qh[ib] >> k) & 1) << 8);
            for (int e = 0; e < 4; e++) {
                int j = 4 * k + e;
                float sg = ((signs[4 * ib + (j >> 3)] >> (j & 7)) & 1) ? -1.0f : 1.0f;
                y[32 * ib + j] = (db * (float)g_iq3s_grid[idx][e]) * sg;
            }
        }
    }
}

/* IQ4_XS: d | scales_h u16 | scales_l[4] | qs[128]  (gguf-plugin/gluon/iq4xs.py:5-11,36). */
static void deq_iq4_xs(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    uint32_t sh = (uint32_t)b[2] | ((uint32_t)b[3] << 8);
    const uint8_t *sl = b + 4, *qs = b + 8;
    for (int ib = 0; ib < 8; ib++) {
        int l = (sl[ib >> 1] >> (4 * (ib & 1))) & 0xF;
        int h = (sh >> (2 * ib)) & 3;
        int ls = (int)(int8_t)(l | (h << 4)) - 32;
        float dl = d * (float)ls;
        for (int j = 0; j < 16; j++) {
            y[32 * ib + j] = dl * (float)g_iq4_kvalues[qs[16 * ib + j] & 0xF];
            y[32 * ib + 16 + j] = dl * (float)g_iq4_kvalues[qs[16 * ib + j] >> 4];
        }
    }
}

/* sign factors, read from memory so that the product stays a multiplication (a negation would flip the sign of a NaN,
 * which the multiplication gguf-py performs leaves alone) */
static const volatile float g_sign[2] = {1.0f, -1.0f};

/* The 8-bit sign mask of a group of 8 weights from its stored 7-bit index: bit 7 is the parity of the seven
 * (llama.cpp's ksigns_iq2xs table, stated as arithmetic: gguf-plugin/gluon/iq2.py:27-28). */
static int sign_mask8(int idx7) {
    int p = idx7 ^ (idx7 >> 4);
    p ^= p >> 2;
    p ^= p >> 1;
    return idx7 | ((p & 1) << 7);
}

/* IQ3_XXS: d | qs[64] | u32[8] (four 7-bit sign indices, scale in bits 28..31); weight = d (2 s + 1) / 4 x
 * magnitude x sign (gguf-plugin/gluon/iq3xxs.py:5-12). */
static void deq_iq3_xxs(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    const uint8_t *qs = b + 2, *sas = b + 66;
    for (int ib = 0; ib < 8; ib++) {
        uint32_t w = (uint32_t)sas[4 * ib] | ((uint32_t)sas[4 * ib + 1] << 8) | ((uint32_t)sas[4 * ib + 2] << 16) | ((uint32_t)sas[4 * ib + 3] << 24);
        float db = d * (0.5f + (float)(w >> 28)) * 0.5f;
        for (int l = 0; l < 4; l++) {
            int sg = sign_mask8((int)((w >> (7 * l)) & 0x7F));
            for (int j = 0; j < 8; j++) {
                int mag = g_iq3xxs_grid[qs[8 * ib + 2 * l + (j >> 2)]][j & 3];
                y[32 * ib + 8 * l + j] = (db * (float)mag) * g_sign[(sg >> j) & 1];
            }
        }
    }
}

/* IQ2_XXS: d | per sub-block two u32: four 8-bit grid indices, then four 7-bit sign indices and the scale in bits
 * 28..31; weight = d (2 s + 1) / 8 x magnitude x sign (gguf-plugin/gluon/iq2.py:12-17). */
static void deq_iq2_xxs(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    for (int ib = 0; ib < 8; ib++) {
        const uint8_t *q = b + 2 + 8 * ib;
        uint32_t w = (uint32_t)q[4] | ((uint32_t)q[5] << 8) | ((uint32_t)q[6] << 16) | ((uint32_t)q[7] << 24);
        float db = d * (0.5f + (float)(w >> 28)) * 0.25f;
        for (int l = 0; l < 4; l++) {
            int sg = sign_mask8((int)((w >> (7 * l)) & 0x7F));
            for (int j = 0; j < 8; j++)
                y[32 * ib + 8 * l + j] = (db * (float)g_iq2xxs_grid[q[l]][j]) * g_sign[(sg >> j) & 1];
        }
    }
}

/* IQ2_XS: d | u16[32]: 9-bit grid index and 7-bit sign index per group of 8 | scales[8]: a nibble per 16 weights
 * (gguf-plugin/gluon/iq2.py:18-20). */
static void deq_iq2_xs(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    const uint8_t *qs = b + 2, *sc = b + 66;
    for (int g = 0; g < 32; g++) {
        int v = qs[2 * g] | (qs[2 * g + 1] << 8);
        int s = (sc[g >> 2] >> (4 * ((g >> 1) & 1))) & 0xF;
        float db = d * (0.5f + (float)s) * 0.25f;
        int sg = sign_mask8(v >> 9);
        for (int j = 0; j < 8; j++)
            y[8 * g + j] = (db * (float)g_iq2xs_grid[v & 511][j]) * g_sign[(sg >> j) & 1];
    }
}

/* IQ2_S: d | qs[32] low index bytes | signs[32] | qh[8]: two high index bits per group | scales[8] as IQ2_XS
 * (gguf-plugin/gluon/iq2.py:21-23). */
static void deq_iq2_s(const uint8_t *b, float *y) {
    float d = f16_to_f32(b);
    const uint8_t *qs = b + 2, *signs = b + 34, *qh = b + 66, *sc = b + 74;
    for (int g = 0; g < 32; g++) {
        int idx = qs[g] | (((qh[g >> 2] >> (2 * (g & 3))) & 3) << 8);
        int s = (sc[g >> 2] >> (4 * ((g >> 1) & 1))) & 0xF;
        float db = d * (0.5f + (float)s) * 0.25f;
        for (int j = 0; j < 8; j++)
            y[8 * g + j] = (db * (float)g_iq2s_grid[idx][j]) * g_sign[(signs[g] >> j) & 1];
    }
}

/* IQ1_M: qs[32] low index bytes | qh[16]: per group of 8 a nibble (three high index bits, bit 3: the sign of delta) |
 * scales[8] = four u16: bits 0..11 four 3-bit scales (one per 16 weights), bits 12..15 a nibble of the fp16 d.
 * weight = d (2 s + 1) (g + delta), g in {-1, 0, 1}, delta = +-1/8 (gguf-py IQ1_M.dequantize_blocks; the reference has no kernel
 * of its own for this type, it leaves it to the plugin's row path). */
static void deq_iq1_m(const uint8_t *b, float *y) {
    const uint8_t *qs = b, *qh = b + 32, *sc = b + 48;
    uint16_t s16[4];
    for (int i = 0; i < 4; i++) s16[i] = (uint16_t)(sc[2 * i] | (sc[2 * i + 1] << 8));
    uint8_t dbits[2];
    uint16_t dv = (uint16_t)((s16[0] >> 12) | ((s16[1] >> 8) & 0x00F0) | ((s16[2] >> 4) & 0x0F00) | (s16[3] & 0xF000));
    dbits[0] = (uint8_t)(dv & 0xFF); dbits[1] = (uint8_t)(dv >> 8);
    float d = f16_to_f32(dbits);
    for (int g = 0; g < 32; g++) {
        int nib = (qh[g >> 1] >> (4 * (g & 1))) & 0xF;
        int idx = qs[g] | ((nib & 7) << 8);
        int s = (s16[g >> 3] >> (3 * ((g >> 1) & 3))) & 7;
        float dl = d * (float)(2 * s + 1);
        float delta = (nib & 8) ? -0.125f : 0.125f;
        for (int j = 0; j < 8; j++) y[8 * g + j] = dl * ((float)g_iq1_grid[idx][j] + delta);
    }
}

/* one row segment of 256 weights -> 256 floats */
static int deq_256(int type, const uint8_t *b, float *y) {
    switch (type) {
        case T_Q4_0: for (int i = 0; i < 8; i++) deq_q4_0(b + 18 * i, y + 32 * i); return 0;
        case T_Q5_0: for (int i = 0; i < 8; i++) deq_q5_0(b + 22 * i, y + 32 * i); return 0;
        case T_Q8_0: for (int i = 0; i < 8; i++) deq_q8_0(b + 34 * i, y + 32 * i); return 0;
        case T_IQ4_NL: for (int i = 0; i < 8; i++) deq_iq4_nl(b + 18 * i, y + 32 * i); return 0;
        case T_Q2_K: deq_q2_k(b, y); return 0;
        case T_Q3_K: deq_q3_k(b, y); return 0;
        case T_Q4_K: deq_q4_k(b, y); return 0;
        case T_Q5_K: deq_q5_k(b, y); return 0;
        case T_Q6_K: deq_q6_k(b, y); return 0;
        case T_IQ3_S: deq_iq3_s(b, y); return 0;
        case T_IQ4_XS: deq_iq4_xs(b, y); return 0;
        case T_IQ3_XXS: deq_iq3_xxs(b, y); return 0;
        case T_IQ2_XXS: deq_iq2_xxs(b, y); return 0;
        case T_IQ2_XS: deq_iq2_xs(b, y); return 0;
        case T_IQ2_S: deq_iq2_s(b, y); return 0;
        case T_IQ1_M: deq_iq1_m(b, y); return 0;
        default: return -1;
    }
}

/* raw uint8 [n_rows, (K/256)*bytes_per_256] -> fp32 [n_rows, K].  Returns 0, or <0 on a bad argument. */
int oracle_dequantize(int type, const uint8_t *raw, int64_t n_rows, int64_t K, float *out) {
    int bb = oracle_bytes_per_256(type);
    if (bb == 0) return -1;
    if (K <= 0 || K % QK_K) return -2;
    if ((type == T_IQ3_S || type == T_IQ4_NL || type == T_IQ4_XS) && !g_tables_set) return -3;
    if ((type == T_IQ3_XXS || type == T_IQ2_XXS || type == T_IQ2_XS || type == T_IQ2_S) && !g_iq_grids_set) return -3;
    if (type == T_IQ1_M && !g_iq1_grid_set) return -3;
    int64_t nb = K / QK_K;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; r++)
        for (int64_t kb = 0; kb < nb; kb++)
            deq_256(type, raw + (r * nb + kb) * bb, out + r * K + kb * QK_K);
    return 0;
}

/* Y[M, n_rows] (fp32, row stride ldy) = X[M, K] (fp32) . dequantize(raw)[n_rows, K]^T, accumulated in
 * fp32 one 256-weight segment at a time: the fused "dequantise then multiply" a CPU would run, every
 * weight byte read once.  All host threads (OpenMP) over the weight rows.  This is the timed CPU
 * baseline; the parity tests use the fp64 product of oracle_dequantize's output instead. */
int oracle_matmul(int type, const uint8_t *raw, int64_t n_rows, int64_t K, const float *X, int64_t M,
                  float *Y, int64_t ldy) {
    int bb = oracle_bytes_per_256(type);
    if (bb == 0) return -1;
    if (K <= 0 || K % QK_K) return -2;
    if ((type == T_IQ3_S || type == T_IQ4_NL || type == T_IQ4_XS) && !g_tables_set) return -3;
    if ((type == T_IQ3_XXS || type == T_IQ2_XXS || type == T_IQ2_XS || type == T_IQ2_S) && !g_iq_grids_set) return -3;
    if (type == T_IQ1_M && !g_iq1_grid_set) return -3;
    int64_t nb = K / QK_K;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; r++) {
        float w[QK_K];
        float acc[64];
        for (int64_t m0 = 0; m0 < M; m0 += 64) {
            int64_t mc = M - m0 < 64 ? M - m0 : 64;
            for (int64_t m = 0; m < mc; m++) acc[m] = 0.0f;
            for (int64_t kb = 0; kb < nb; kb++) {
                deq_256(type, raw + (r * nb + kb) * bb, w);
                for (int64_t m = 0; m < mc; m++) {
                    const float *x = X + (m0 + m) * K + kb * QK_K;
                    float s = 0.0f;
                    for (int k = 0; k < QK_K; k++) s += w[k] * x[k];
                    acc[m] += s;
                }
            }
            for (int64_t m = 0; m < mc; m++) Y[(m0 + m) * ldy + r] = acc[m];
        }
    }
    return 0;
}

/* threads the OpenMP loops use from now on (a launcher may have exported OMP_NUM_THREADS=1 for its workers) */
void oracle_set_num_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
