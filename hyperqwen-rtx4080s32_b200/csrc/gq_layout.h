// Tile-major layout of the packed GGUF weights (the load-time repack target).
//
// A tensor [n_out, K] of one GGML type is cut into tiles of 64 output rows x 256 weights (one k-block).
// Tiles are stored [row_tile][k_block] so that the k-range a CTA walks is one contiguous byte range and
// every pipeline stage is a single bulk copy.  A tile is four slabs of 16 rows; a slab is what one warp
// feeds to m16n8k16 tensor-core instructions.  Inside a slab the quantised bytes are ordered by the lane
// that consumes them: lane l = 4*g + t owns, for rows g and g+8, the weights 16*r + 4*t + {0,1,2,3} of
// every 16-weight run r = 0..15 of the k-block, and reads them as 16-byte chunks (chunk c of lane l sits
// at 512*c + 16*l).  Scales and other fields shared by several lanes follow the chunks, one record per row.
//
// The repack is a pure byte permutation of the raw GGUF block bytes (plus zero rows past n_out): a slab
// holds exactly 16 * bytes_per_256 bytes, so the packed tensor has the raw byte count rounded up to whole
// tiles and can be turned back into the raw rows bit for bit.  It replaces the reference's torch-op repacks
// (gguf-plugin/gluon/tiles.py:24-36,128-130, kq_tiles.py:29-46,76-87, iq3s_int8t.py:64-77,
// iq4xs_int8t.py:161-172, q4k_int8t.py:144-154), whose layouts are tuned for Ada's cp.async stages.
#pragma once
#include <stdint.h>

#define GQ_QK 256
#define GQ_TILE_ROWS 64
#define GQ_SLAB_ROWS 16

enum GqType {
    GQ_Q4_0 = 2, GQ_Q5_0 = 6, GQ_Q8_0 = 8, GQ_Q2_K = 10, GQ_Q3_K = 11, GQ_Q4_K = 12, GQ_Q5_K = 13,
    GQ_Q6_K = 14, GQ_IQ2_XXS = 16, GQ_IQ2_XS = 17, GQ_IQ3_XXS = 18, GQ_IQ4_NL = 20, GQ_IQ3_S = 21, GQ_IQ2_S = 22, GQ_IQ4_XS = 23,
    GQ_IQ1_M = 29
};

#ifdef __CUDACC__
#define GQ_HD __host__ __device__
#else
#define GQ_HD
#endif

// bytes of one row's 256-weight segment (0: unsupported type)
GQ_HD inline int gq_type_bytes(int type) {
    switch (type) {
        case GQ_Q4_0: return 144;
        case GQ_Q5_0: return 176;
        case GQ_Q8_0: return 272;
        case GQ_Q2_K: return 84;
        case GQ_Q3_K: return 110;
        case GQ_Q4_K: return 144;
        case GQ_Q5_K: return 176;
        case GQ_Q6_K: return 210;
        case GQ_IQ4_NL: return 144;
        case GQ_IQ3_S: return 110;
        case GQ_IQ4_XS: return 136;
        case GQ_IQ3_XXS: return 98;
        case GQ_IQ2_XXS: return 66;
        case GQ_IQ2_XS: return 74;
        case GQ_IQ2_S: return 82;
        case GQ_IQ1_M: return 56;
        default: return 0;
    }
}

// number of 512-byte lane-ordered chunks at the head of a slab
GQ_HD inline int gq_type_chunks(int type) {
    switch (type) {
        case GQ_Q4_0: case GQ_IQ4_NL: case GQ_Q4_K: case GQ_IQ4_XS: case GQ_Q5_0: return 4;
        case GQ_Q5_K: return 5;
        case GQ_Q6_K: return 6;
        case GQ_Q8_0: return 8;
        case GQ_Q2_K: return 2;
        case GQ_Q3_K: return 3;
        case GQ_IQ3_S: case GQ_IQ3_XXS: return 2;
        default: return 0;
    }
}

// Codebook types keep a table of grid entries in shared memory while a kernel decodes them.  Kind index of a type
// (-1: not a codebook type), and the table's bytes in the integer form (form 1: magnitudes as bytes) and in the fp16 form (form 0).
GQ_HD inline int gq_cb_kind(int type) {
    switch (type) {
        case GQ_IQ3_S: return 0;
        case GQ_IQ3_XXS: return 1;
        case GQ_IQ2_XXS: return 2;
        case GQ_IQ2_XS: return 3;
        case GQ_IQ2_S: return 4;
        case GQ_IQ1_M: return 5;
        default: return -1;
    }
}
#define GQ_CB_KINDS 6
GQ_HD inline int gq_cb_bytes(int kind, int form) {
    switch (kind) {
        case 0: return form ? 2048 : 4096;     // IQ3_S: 512 entries of 4 bytes / of two fp16 pairs
        case 1: return form ? 1024 : 2048;     // IQ3_XXS: 256 entries of 4 bytes / of two fp16 pairs
        case 2: return 2048;                   // IQ2_XXS: 256 entries of 8 bytes
        case 3: return 4096;                   // IQ2_XS: 512 entries of 8 bytes
        case 4: return 8192;                   // IQ2_S: 1024 entries of 8 bytes
        case 5: return 16384;                  // IQ1_M: 2048 entries of 8 bytes
        default: return 0;
    }
}
// a kernel whose CTAs decode one type each keeps the CTA's table at the start of a region sized for the largest
GQ_HD inline int gq_cb_region_max(int mask, int form) {
    int m = 0;
    for (int k = 0; k < GQ_CB_KINDS; ++k)
        if (((mask >> k) & 1) && gq_cb_bytes(k, form) > m) m = gq_cb_bytes(k, form);
    return m;
}
// a kernel whose CTAs may decode two types keeps the tables of all types of the run side by side (fp16 form)
GQ_HD inline int gq_cb_offset(int mask, int kind) {
    int o = 0;
    for (int k = 0; k < kind; ++k)
        if ((mask >> k) & 1) o += gq_cb_bytes(k, 0);
    return o;
}
GQ_HD inline int gq_cb_region_sum(int mask) { return gq_cb_offset(mask, GQ_CB_KINDS); }

// Source of packed byte p (0 <= p < 16 * bytes_per_256) of a slab: *row in 0..15, *byte = offset inside
// that row's 256-weight segment of raw GGUF bytes.  Returns 0, or -1 for a bad argument.
GQ_HD inline int gq_slab_src(int type, int p, int *row, int *byte) {
    const int B = gq_type_bytes(type);
    const int C = gq_type_chunks(type);
    if (B == 0 || p < 0 || p >= 16 * B) return -1;
    // the byte order inside a 4-byte word of a lane's chunk: types whose stored bytes are read in place (masks,
    // or the int8 weights of Q8_0) put weights (0,2,1,3), so that bytes 0 and 2 (the low bytes of the two 16-bit
    // halves) are k-neighbours and an 8-bit quad has the order the activation planes use; types that go through a
    // byte lookup keep the natural order (the lookup emits whatever order it likes)
    if (p < 512 * C) {
        const int c = p >> 9, l = (p >> 4) & 31, e = (p >> 2) & 3, z = p & 3;
        const int g = l >> 2, t = l & 3;
        const int h = e >> 1, u = e & 1;          // default word meaning: row half h, sub-run u
        const int im = ((z & 1) << 1) | (z >> 1);   // (0,2,1,3): weight index inside the lane's group of four
        switch (type) {
            case GQ_Q4_K:
                *row = g + 8 * h; *byte = 16 + 32 * c + 16 * u + 4 * t + im; return 0;
            case GQ_Q5_K:
                *row = g + 8 * h;
                *byte = c < 4 ? 48 + 32 * c + 16 * u + 4 * t + im : 16 + 16 * u + 4 * t + im;
                return 0;
            case GQ_Q6_K:
                *row = g + 8 * h;
                *byte = c < 4 ? 64 * (c >> 1) + 32 * (c & 1) + 16 * u + 4 * t + im
                              : 128 + 32 * (c - 4) + 16 * u + 4 * t + im;
                return 0;
            case GQ_Q8_0: {
                const int r = 2 * c + u;          // run 0..15
                *row = g + 8 * h; *byte = 34 * (r >> 1) + 2 + 16 * (r & 1) + 4 * t + im; return 0;
            }
            case GQ_Q4_0: { const int b = 2 * c + u; *row = g + 8 * h; *byte = 18 * b + 2 + 4 * t + im; return 0; }
            case GQ_IQ4_NL: { const int b = 2 * c + u; *row = g + 8 * h; *byte = 18 * b + 2 + 4 * t + z; return 0; }
            case GQ_Q5_0: { const int b = 2 * c + u; *row = g + 8 * h; *byte = 22 * b + 6 + 4 * t + im; return 0; }
            case GQ_IQ4_XS: { const int b = 2 * c + u; *row = g + 8 * h; *byte = 8 + 16 * b + 4 * t + z; return 0; }
            case GQ_Q2_K:
                *row = g + 8 * h; *byte = 16 + 32 * c + 16 * u + 4 * t + im; return 0;
            case GQ_Q3_K:
                *row = g + 8 * h;
                *byte = c < 2 ? 32 + 32 * c + 16 * u + 4 * t + im : 16 * u + 4 * t + im;
                return 0;
            case GQ_IQ3_S: case GQ_IQ3_XXS: {
                const int r = 4 * e + z;          // run 0..15: one grid-index byte per run
                *row = g + 8 * c; *byte = 2 + 8 * (r >> 1) + 4 * (r & 1) + t; return 0;
            }
        }
        return -1;
    }
    int q = p - 512 * C;
    switch (type) {
        case GQ_Q4_K: case GQ_Q5_K:               // 16 B per row: d, dmin, scales[12]
            *row = q >> 4; *byte = q & 15; return 0;
        case GQ_Q6_K:                              // scales[16] per row, then d per row
            if (q < 256) { *row = q >> 4; *byte = 192 + (q & 15); } else { q -= 256; *row = q >> 1; *byte = 208 + (q & 1); }
            return 0;
        case GQ_Q8_0:                              // d[8] per row
            *row = q >> 4; *byte = 34 * ((q & 15) >> 1) + (q & 1); return 0;
        case GQ_Q4_0: case GQ_IQ4_NL:
            *row = q >> 4; *byte = 18 * ((q & 15) >> 1) + (q & 1); return 0;
        case GQ_Q5_0: {                            // per row: d[8] (16 B) then qh[8] (32 B)
            const int r = q / 48, o = q % 48;
            *row = r;
            *byte = o < 16 ? 22 * (o >> 1) + (o & 1) : 22 * ((o - 16) >> 2) + 2 + ((o - 16) & 3);
            return 0;
        }
        case GQ_IQ4_XS:                            // 8 B per row: d, scales_h, scales_l[4]
            *row = q >> 3; *byte = q & 7; return 0;
        case GQ_Q2_K:                              // scales[16] per row, then (d, dmin) per row
            if (q < 256) { *row = q >> 4; *byte = q & 15; } else { q -= 256; *row = q >> 2; *byte = 80 + (q & 3); }
            return 0;
        case GQ_Q3_K:                              // scales[12] per row, then d per row
            if (q < 192) { *row = q / 12; *byte = 96 + q % 12; } else { q -= 192; *row = q >> 1; *byte = 108 + (q & 1); }
            return 0;
        case GQ_IQ3_S:                             // signs (32 B per row: even sign bytes, odd sign bytes), qh[8], scales[4], d
            if (q < 512) {
                const int r = q >> 5, a = (q >> 4) & 1, run = q & 15;
                *row = r; *byte = 74 + 4 * (run >> 1) + 2 * (run & 1) + a; return 0;
            }
            q -= 512;
            if (q < 128) { *row = q >> 3; *byte = 66 + (q & 7); return 0; }
            q -= 128;
            if (q < 64) { *row = q >> 2; *byte = 106 + (q & 3); return 0; }
            q -= 64;
            *row = q >> 1; *byte = q & 1; return 0;
        case GQ_IQ2_XXS:                           // no lane-ordered chunks (two lanes share a grid entry): per row the eight
                                                   // index words (32 B), then per row the eight sign-and-scale words, then d
            if (q < 1024) { const int j = q & 31; *row = (q >> 5) & 15; *byte = 2 + 8 * (j >> 2) + 4 * (q >> 9) + (j & 3); return 0; }
            q -= 1024;
            *row = q >> 1; *byte = q & 1; return 0;
        case GQ_IQ2_XS:                            // per row the 32 index-and-sign halfwords (64 B), then scales[8], then d
            if (q < 1024) { *row = q >> 6; *byte = 2 + (q & 63); return 0; }
            q -= 1024;
            if (q < 128) { *row = q >> 3; *byte = 66 + (q & 7); return 0; }
            q -= 128;
            *row = q >> 1; *byte = q & 1; return 0;
        case GQ_IQ1_M:                             // per row the 32 low index bytes, then per row qh[16], then per row the four scale halfwords
            if (q < 512) { *row = q >> 5; *byte = q & 31; return 0; }
            q -= 512;
            if (q < 256) { *row = q >> 4; *byte = 32 + (q & 15); return 0; }
            q -= 256;
            *row = q >> 3; *byte = 48 + (q & 7); return 0;
        case GQ_IQ2_S:                             // per row 32 index bytes, then per row 32 sign bytes, qh[8], scales[8], d
            if (q < 1024) { *row = (q >> 5) & 15; *byte = 2 + 32 * (q >> 9) + (q & 31); return 0; }
            q -= 1024;
            if (q < 256) { *row = (q >> 3) & 15; *byte = 66 + 8 * (q >> 7) + (q & 7); return 0; }
            q -= 256;
            *row = q >> 1; *byte = q & 1; return 0;
        case GQ_IQ3_XXS:                           // the eight sign-and-scale words per row (32 B), then d per row
            if (q < 512) { *row = q >> 5; *byte = 66 + (q & 31); return 0; }
            q -= 512;
            *row = q >> 1; *byte = q & 1; return 0;
    }
    return -1;
}
