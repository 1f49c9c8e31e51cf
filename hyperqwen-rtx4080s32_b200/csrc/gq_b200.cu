// B200 (sm_100a) GGUF quantized-linear path: load-time repack / un-repack / dequantise kernels, the
// activation preparation, the grouped small-batch GEMV/GEMM kernel, the split-K partial sum, and the C ABI
// declared in include/gq_b200.h.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <atomic>
#include <mutex>
#include <unordered_map>
#include "../../include/gq_b200.h"
#include "gq_decode.cuh"
#include "gq_decode8.cuh"
#include <type_traits>
#include "_generated/gq_tables.h"

using namespace gq;

// ---------------------------------------------------------------------------------------------------
// host bookkeeping
// ---------------------------------------------------------------------------------------------------
static thread_local char g_cuda_err[256] = "";
static std::atomic<long long> g_launches{0};

static int cuda_fail(cudaError_t e, const char *what) {
    snprintf(g_cuda_err, sizeof g_cuda_err, "%s: %s", what, cudaGetErrorString(e));
    return GQ_ERR_CUDA;
}
#define GQ_CUDA(call)                                          \
    do {                                                       \
        cudaError_t e_ = (call);                               \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call);    \
    } while (0)
#define GQ_LAUNCHED()                                                    \
    do {                                                                 \
        cudaError_t e_ = cudaGetLastError();                             \
        if (e_ != cudaSuccess) return cuda_fail(e_, "kernel launch");    \
        g_launches.fetch_add(1, std::memory_order_relaxed);              \
    } while (0)

extern "C" const char *gq_last_cuda_error(void) { return g_cuda_err; }
extern "C" int64_t gq_launch_count(void) { return (int64_t)g_launches.load(); }
extern "C" int gq_bytes_per_256(int type) { return gq_type_bytes(type); }

extern "C" int64_t gq_packed_bytes(int type, int64_t n_out, int64_t K) {
    const int B = gq_type_bytes(type);
    if (!B) return GQ_ERR_TYPE;
    if (n_out < 0 || K <= 0 || K % GQ_QK) return GQ_ERR_SHAPE;
    return ((n_out + 63) / 64) * (K / GQ_QK) * 64 * (int64_t)B;
}

extern "C" int gq_slab_map(int type, int32_t *map) {
    const int B = gq_type_bytes(type);
    if (!B) return GQ_ERR_TYPE;
    if (!map) return GQ_ERR_ARG;
    for (int p = 0; p < 16 * B; ++p) {
        int row, byte;
        if (gq_slab_src(type, p, &row, &byte)) return GQ_ERR_TYPE;
        map[p] = row * B + byte;
    }
    return GQ_OK;
}

// ---------------------------------------------------------------------------------------------------
// repack / un-repack: one CTA per (16-row slab, k-block); the slab's raw image goes through shared memory
// ---------------------------------------------------------------------------------------------------
#define GQ_MAX_SLAB (16 * 272)

__global__ void __launch_bounds__(256) repack_kernel(int type, int B, const uint8_t *__restrict__ raw, int64_t n_out, int nb,
                                                     int64_t row_stride, uint8_t *__restrict__ out) {
    __shared__ __align__(16) uint8_t img[GQ_MAX_SLAB];
    const int slab = blockIdx.x, kb = blockIdx.y;
    const int64_t row0 = (int64_t)slab * 16;
    for (int i = threadIdx.x; i < 16 * B; i += 256) {
        const int r = i / B, b = i - r * B;
        img[i] = (row0 + r < n_out) ? raw[(row0 + r) * row_stride + (int64_t)kb * B + b] : (uint8_t)0;
    }
    __syncthreads();
    // packed address: tile = slab / 4, slab-in-tile = slab % 4
    uint8_t *dst = out + (((int64_t)(slab >> 2) * nb + kb) * 4 + (slab & 3)) * (int64_t)(16 * B);
    for (int w = threadIdx.x; w < 4 * B; w += 256) {
        uint32_t v = 0;
#pragma unroll
        for (int z = 0; z < 4; ++z) {
            int row, byte;
            gq_slab_src(type, 4 * w + z, &row, &byte);
            v |= (uint32_t)img[row * B + byte] << (8 * z);
        }
        reinterpret_cast<uint32_t *>(dst)[w] = v;
    }
}

// fills img[16][B] (raw order) from a packed slab
__device__ __forceinline__ void slab_to_raw_image(int type, int B, const uint8_t *__restrict__ src, uint8_t *img) {
    for (int w = threadIdx.x; w < 4 * B; w += blockDim.x) {
        const uint32_t v = reinterpret_cast<const uint32_t *>(src)[w];
#pragma unroll
        for (int z = 0; z < 4; ++z) {
            int row, byte;
            gq_slab_src(type, 4 * w + z, &row, &byte);
            img[row * B + byte] = (uint8_t)(v >> (8 * z));
        }
    }
}

__global__ void __launch_bounds__(256) unrepack_kernel(int type, int B, const uint8_t *__restrict__ tiles, int64_t n_out, int nb,
                                                       uint8_t *__restrict__ raw, int64_t row_stride) {
    __shared__ __align__(16) uint8_t img[GQ_MAX_SLAB];
    const int slab = blockIdx.x, kb = blockIdx.y;
    const uint8_t *src = tiles + (((int64_t)(slab >> 2) * nb + kb) * 4 + (slab & 3)) * (int64_t)(16 * B);
    slab_to_raw_image(type, B, src, img);
    __syncthreads();
    const int64_t row0 = (int64_t)slab * 16;
    for (int i = threadIdx.x; i < 16 * B; i += 256) {
        const int r = i / B, b = i - r * B;
        if (row0 + r < n_out) raw[(row0 + r) * row_stride + (int64_t)kb * B + b] = img[i];
    }
}

// ---------------------------------------------------------------------------------------------------
// bit-exact dequantiser (fp32 in the format reference's operation order: (d*sc) first, then *q, then -(dmin*m);
// explicit round-to-nearest multiplies and subtracts so nothing is fused)
// ---------------------------------------------------------------------------------------------------
// The codebook grids live in global memory, not in constant memory: the kernels copy them into shared memory with one
// index per thread, which the constant cache would serve one address at a time.
__device__ uint32_t c_iq3s_grid[512];
__device__ uint32_t c_iq3xxs_grid[256];
__device__ uint32_t c_iq2xxs_grid[512], c_iq2xs_grid[1024], c_iq2s_grid[2048];    // two words per entry
__device__ uint32_t c_iq1_grid[4096];      // two words per entry, a byte is 8 g + 16
__constant__ int8_t c_iq4_kvalues[16];

// A bounded wait that runs out is reported twice: in the status word of the launch's workspace (gq_read_status) and in
// this per-device word, which keeps the largest code seen since it was last read (gq_device_status) — a caller that
// drops its workspace after every call, or has none to read (the no-allocation entry point), still learns of it.
__device__ int g_sticky_status;
__device__ __forceinline__ void report_status(int *status, int code) {
    atomicExch(status, code);
    atomicMax(&g_sticky_status, code);
}
// time limit of the waits on data from another GPU (the fused and the separate all-reduce), nanoseconds
static std::atomic<unsigned long long> g_peer_wait_ns{GQ_WAIT_LIMIT_NS};

#include "gq_prefill.cuh"

__device__ __forceinline__ float h2f(const uint8_t *p) { return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8)))); }

__device__ __forceinline__ void scale_min_k4(const uint8_t *s, int j, int &sc, int &mn) {
    if (j < 4) { sc = s[j] & 63; mn = s[j + 4] & 63; }
    else { sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4); mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}

// weight w (0..255) of the raw 256-weight segment b
__device__ float deq_one(int type, const uint8_t *b, int w) {
    switch (type) {
        case GQ_Q4_0: { const uint8_t *k = b + 18 * (w >> 5); const int j = w & 31;
            const int q = (j < 16 ? (k[2 + j] & 0xF) : (k[2 + j - 16] >> 4)) - 8; return __fmul_rn(h2f(k), (float)q); }
        case GQ_IQ4_NL: { const uint8_t *k = b + 18 * (w >> 5); const int j = w & 31;
            const int q = c_iq4_kvalues[j < 16 ? (k[2 + j] & 0xF) : (k[2 + j - 16] >> 4)]; return __fmul_rn(h2f(k), (float)q); }
        case GQ_Q5_0: { const uint8_t *k = b + 22 * (w >> 5); const int j = w & 31;
            const uint32_t qh = k[2] | (k[3] << 8) | (k[4] << 16) | ((uint32_t)k[5] << 24);
            const int lo = j < 16 ? (k[6 + j] & 0xF) : (k[6 + j - 16] >> 4);
            const int q = (lo | (((qh >> j) & 1) << 4)) - 16; return __fmul_rn(h2f(k), (float)q); }
        case GQ_Q8_0: { const uint8_t *k = b + 34 * (w >> 5); return __fmul_rn((float)(int8_t)k[2 + (w & 31)], h2f(k)); }
        case GQ_Q2_K: { const int n = w >> 7, t = (w >> 5) & 3, l = w & 31, g = w >> 4;
            const float dl = __fmul_rn(h2f(b + 80), (float)(b[g] & 0xF)), ml = __fmul_rn(h2f(b + 82), (float)(b[g] >> 4));
            const int q = (b[16 + 32 * n + l] >> (2 * t)) & 3; return __fsub_rn(__fmul_rn(dl, (float)q), ml); }
        case GQ_Q3_K: { const int nn = w >> 7, j = (w >> 5) & 3, l = w & 31, i = w >> 4; const uint8_t *s = b + 96;
            const int lo = (s[i % 8] >> (4 * (i / 8))) & 0xF, hi = (s[8 + i % 4] >> (2 * (i / 4))) & 3;
            const float dl = __fmul_rn(h2f(b + 108), (float)((lo | (hi << 4)) - 32));
            const int q = (int)((b[32 + 32 * nn + l] >> (2 * j)) & 3) - (((b[l] >> (4 * nn + j)) & 1) ? 0 : 4);
            return __fmul_rn(dl, (float)q); }
        case GQ_Q4_K: { const int ib = w >> 5, p = w & 31; int sc, mn; scale_min_k4(b + 4, ib, sc, mn);
            const float dl = __fmul_rn(h2f(b), (float)sc), dm = __fmul_rn(h2f(b + 2), (float)mn);
            const int q = (b[16 + 32 * (ib >> 1) + p] >> (4 * (ib & 1))) & 0xF; return __fsub_rn(__fmul_rn(dl, (float)q), dm); }
        case GQ_Q5_K: { const int ib = w >> 5, p = w & 31; int sc, mn; scale_min_k4(b + 4, ib, sc, mn);
            const float dl = __fmul_rn(h2f(b), (float)sc), dm = __fmul_rn(h2f(b + 2), (float)mn);
            const int q = ((b[48 + 32 * (ib >> 1) + p] >> (4 * (ib & 1))) & 0xF) | (((b[16 + p] >> ib) & 1) << 4);
            return __fsub_rn(__fmul_rn(dl, (float)q), dm); }
        case GQ_Q6_K: { const int h = w >> 7, t = (w >> 5) & 3, p = w & 31;
            const int q = (int)(((b[64 * h + 32 * (t & 1) + p] >> (4 * (t >> 1))) & 0xF) | (((b[128 + 32 * h + p] >> (2 * t)) & 3) << 4)) - 32;
            const float dl = __fmul_rn(h2f(b + 208), (float)(int8_t)b[192 + (w >> 4)]); return __fmul_rn(dl, (float)q); }
        case GQ_IQ3_S: { const int ib = w >> 5, j = w & 31, k = j >> 2, e = j & 3;
            const int s = (b[106 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF; const float db = __fmul_rn(h2f(b), (float)(1 + 2 * s));
            const int idx = b[2 + 8 * ib + k] | (((b[66 + ib] >> k) & 1) << 8);
            const float mag = (float)((c_iq3s_grid[idx] >> (8 * e)) & 0xFF);
            const float v = __fmul_rn(db, mag); return ((b[74 + 4 * ib + (j >> 3)] >> (j & 7)) & 1) ? -v : v; }
        case GQ_IQ3_XXS: { const int ib = w >> 5, j = w & 31; const uint8_t *q = b + 66 + 4 * ib;
            const uint32_t sw = q[0] | (q[1] << 8) | (q[2] << 16) | ((uint32_t)q[3] << 24);
            const float db = __fmul_rn(__fmul_rn(h2f(b), 0.5f + (float)(sw >> 28)), 0.5f);
            const uint32_t f = (sw >> (7 * (j >> 3))) & 0x7Fu, mask = f | (((uint32_t)__popc(f) & 1u) << 7);
            const float mag = (float)((c_iq3xxs_grid[b[2 + 8 * ib + (j >> 2)]] >> (8 * (j & 3))) & 0xFF);
            const float v = __fmul_rn(db, mag); return ((mask >> (j & 7)) & 1) ? -v : v; }
        case GQ_IQ2_XXS: { const int ib = w >> 5, j = w & 31, l = j >> 3; const uint8_t *q = b + 2 + 8 * ib;
            const uint32_t sw = q[4] | (q[5] << 8) | (q[6] << 16) | ((uint32_t)q[7] << 24);
            const float db = __fmul_rn(__fmul_rn(h2f(b), 0.5f + (float)(sw >> 28)), 0.25f);
            const uint32_t f = (sw >> (7 * l)) & 0x7Fu, mask = f | (((uint32_t)__popc(f) & 1u) << 7);
            const float mag = (float)((c_iq2xxs_grid[2 * q[l] + ((j >> 2) & 1)] >> (8 * (j & 3))) & 0xFF);
            const float v = __fmul_rn(db, mag); return ((mask >> (j & 7)) & 1) ? -v : v; }
        case GQ_IQ2_XS: { const int g = w >> 3, j = w & 7; const uint32_t hw = b[2 + 2 * g] | (b[3 + 2 * g] << 8);
            const int sc = (b[66 + (g >> 2)] >> (4 * ((g >> 1) & 1))) & 0xF;
            const float db = __fmul_rn(__fmul_rn(h2f(b), 0.5f + (float)sc), 0.25f);
            const uint32_t f = hw >> 9, mask = f | (((uint32_t)__popc(f) & 1u) << 7);
            const float mag = (float)((c_iq2xs_grid[2 * (hw & 511u) + (j >> 2)] >> (8 * (j & 3))) & 0xFF);
            const float v = __fmul_rn(db, mag); return ((mask >> j) & 1) ? -v : v; }
        case GQ_IQ2_S: { const int g = w >> 3, j = w & 7;
            const uint32_t idx = b[2 + g] | (((uint32_t)(b[66 + (g >> 2)] >> (2 * (g & 3))) & 3u) << 8);
            const int sc = (b[74 + (g >> 2)] >> (4 * ((g >> 1) & 1))) & 0xF;
            const float db = __fmul_rn(__fmul_rn(h2f(b), 0.5f + (float)sc), 0.25f);
            const float mag = (float)((c_iq2s_grid[2 * idx + (j >> 2)] >> (8 * (j & 3))) & 0xFF);
            const float v = __fmul_rn(db, mag); return ((b[34 + g] >> j) & 1) ? -v : v; }
        case GQ_IQ1_M: { const int g = w >> 3, j = w & 7;
            const uint32_t s0 = b[48] | (b[49] << 8), s1 = b[50] | (b[51] << 8), s2 = b[52] | (b[53] << 8), s3 = b[54] | (b[55] << 8);
            const uint32_t dv = (s0 >> 12) | ((s1 >> 8) & 0xF0u) | ((s2 >> 4) & 0xF00u) | (s3 & 0xF000u);
            const float d = __half2float(__ushort_as_half((unsigned short)dv));
            const uint32_t nib = (b[32 + (g >> 1)] >> (4 * (g & 1))) & 0xFu, idx = b[g] | ((nib & 7u) << 8);
            const uint32_t sw = (g >> 3) == 0 ? s0 : (g >> 3) == 1 ? s1 : (g >> 3) == 2 ? s2 : s3;
            const float dl = __fmul_rn(d, (float)(2 * ((sw >> (3 * ((g >> 1) & 3))) & 7u) + 1));
            const int byte = (int)((c_iq1_grid[2 * idx + (j >> 2)] >> (8 * (j & 3))) & 0xFF);
            const float gv = (float)(byte - 16) * 0.125f;
            return __fmul_rn(dl, gv + ((nib & 8u) ? -0.125f : 0.125f)); }
        case GQ_IQ4_XS: { const int ib = w >> 5, j = w & 31; const uint32_t sh = b[2] | (b[3] << 8);
            const int ls = (int)(((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
            const float dl = __fmul_rn(h2f(b), (float)ls);
            const int q = c_iq4_kvalues[j < 16 ? (b[8 + 16 * ib + j] & 0xF) : (b[8 + 16 * ib + j - 16] >> 4)];
            return __fmul_rn(dl, (float)q); }
    }
    return 0.0f;
}

__global__ void __launch_bounds__(256) dequant_kernel(int type, int B, const uint8_t *__restrict__ tiles, int64_t n_out, int nb,
                                                      void *__restrict__ out, int out_dtype, int64_t ld) {
    __shared__ __align__(16) uint8_t img[GQ_MAX_SLAB];
    const int slab = blockIdx.x, kb = blockIdx.y;
    const uint8_t *src = tiles + (((int64_t)(slab >> 2) * nb + kb) * 4 + (slab & 3)) * (int64_t)(16 * B);
    slab_to_raw_image(type, B, src, img);
    __syncthreads();
    const int64_t row0 = (int64_t)slab * 16;
    for (int i = threadIdx.x; i < 16 * 256; i += 256) {
        const int r = i >> 8, w = i & 255;
        if (row0 + r >= n_out) continue;
        const float v = deq_one(type, img + r * B, w);
        const int64_t o = (row0 + r) * ld + (int64_t)kb * 256 + w;
        if (out_dtype == 0) reinterpret_cast<float *>(out)[o] = v;
        else reinterpret_cast<__nv_bfloat16 *>(out)[o] = __float2bfloat16_rn(v);
    }
}

// ---------------------------------------------------------------------------------------------------
// activation preparation: bf16 row -> fp16 row scaled by a power of two (so any bf16 magnitude fits fp16
// exactly), the row's inverse scale, and per 16-weight run the fp32 sum split into fp16 hi + lo (the B operand
// of the minimum-term MMA).  One CTA per batch row.  Plays the role of the reference's quantize_activations_256
// (gguf-plugin/gluon/tiles_grouped.py:110-139) without quantising: activations keep all their bf16 bits.
// ---------------------------------------------------------------------------------------------------
struct Workspace {
    int *status;
    float *ex;        // [M]
    uint8_t *xt;      // [nb][M][GQ_XROW_BYTES]: per k-block, per batch row: 256 fp16 | pad | 16 run sums hi | 16 lo
    float *partials;  // [S][M][n_total]
};

// one batch row of one k-block in the staged activation tile: 256 fp16 activations (512 B), 32 B of padding
// (row stride 608 B = 96 mod 128, so the rows an MMA reads together sit in distinct banks), then the sixteen
// 16-weight run sums as fp16 hi parts (32 B) and lo parts (32 B)
#define GQ_XROW_BYTES 608
#define GQ_XROW_SX 544

__host__ __device__ inline int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

// The same row in the integer form used for 1..16 batch rows: per k-block and batch row the activations as 16-bit
// fixed point (x * 2^e, e chosen per row and k-block so that the largest magnitude lands in [2^14, 2^15)), split into
// a signed high-byte plane (256 B) and an unsigned low-byte plane (256 B), then the sixteen 16-weight run sums
// (times 2^-6) as fp16 hi parts (32 B) and lo parts (32 B).  Inside a plane the bytes are ordered for the lane that
// reads them: 16-byte unit 4*i + t holds, for runs 4i..4i+3, the quad 4t..4t+3 with bytes in the order (0,2,1,3).
// 576 = 64 mod 128, so the two rows a quarter-warp reads with one 16-byte load each sit in different banks.
// After the rows of a k-block come their scales 2^-e (fp32, one per batch row, padded to a multiple of 16 bytes).
#define GQ_PRE_NONE 0
#define GQ_PRE_SILU_MUL 1
#define GQ_PRE_ADD_RMSNORM 2
#define GQ_X8_ROW 576
#define GQ_X8_SUMS 512
#ifndef GQ_GEMV8_MAX_ROWS
#define GQ_GEMV8_MAX_ROWS 16      // up to here the integer form runs; above it the fp16 form
#endif

__host__ __device__ inline int gq_x8_tile_bytes(int M) { return M * GQ_X8_ROW + ((4 * M + 15) & ~15); }

static int64_t ws_layout(int64_t M, int64_t K, int64_t n_total, int split, void *base, Workspace *ws) {
    int64_t off = 256;
    const int64_t o_ex = off; off = align256(off + M * 4);
    const int64_t xt_bytes = M <= GQ_GEMV8_MAX_ROWS ? (K / GQ_QK) * gq_x8_tile_bytes((int)M) : (K / GQ_QK) * M * GQ_XROW_BYTES;
    const int64_t o_xt = off; off = align256(off + xt_bytes);
    const int64_t o_p = off; if (split > 1) off = align256(off + (int64_t)split * M * n_total * 4);
    if (ws && base) {
        uint8_t *b = (uint8_t *)base;
        ws->status = (int *)b; ws->ex = (float *)(b + o_ex); ws->xt = b + o_xt; ws->partials = (float *)(b + o_p);
    }
    return off;
}

#define GQ_PREP_THREADS 512
#define GQ_PREP_VECS 5      // 16-byte loads a thread keeps in registers: rows up to 512 * 5 * 8 = 20480 activations are read once

__device__ __forceinline__ float amax8(const uint4 &v) {
    const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&v);
    float a = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        a = fmaxf(a, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    return a;
}

// eight activations (half a 16-weight run) -> fp16 at `scale`, stored into the staged tile; the run's fp32 sum is
// completed with the neighbouring lane, which holds the other half
__device__ __forceinline__ void prep_store8(const uint4 &v, int64_t vec, float scale, int M, int m, uint8_t *__restrict__ xt) {
    const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&v);
    uint4 o;
    __half2 *oh = reinterpret_cast<__half2 *>(&o);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        oh[j] = __floats2half2_rn(f.x * scale, f.y * scale);
        sum += __low2float(oh[j]) + __high2float(oh[j]);
    }
    const int64_t k = vec * 8;                       // first activation of this vector
    const int kb = (int)(k >> 8), rr = (int)((k >> 4) & 15);
    uint8_t *row = xt + ((int64_t)kb * M + m) * GQ_XROW_BYTES;
    *reinterpret_cast<uint4 *>(row + (k & 255) * 2) = o;
    // the two halves of a run sit in lanes 2i and 2i+1: the same order of additions as one pass over the run
    const float other = __shfl_xor_sync(0xffffffffu, sum, 1);
    if (!(vec & 1)) {
        const float tot = sum + other;
        const __half hi = __float2half_rn(tot);
        const __half lo = __float2half_rn(tot - __half2float(hi));
        __half *so = reinterpret_cast<__half *>(row + GQ_XROW_SX);
        so[rr] = hi;
        so[16 + rr] = lo;
    }
}

__global__ void __launch_bounds__(GQ_PREP_THREADS) prep_x_kernel(const __nv_bfloat16 *__restrict__ x, int64_t ldx, int K, int M,
                                                                 float *__restrict__ ex, uint8_t *__restrict__ xt, int *status) {
    __shared__ float red[GQ_PREP_THREADS / 32];
    __shared__ float s_scale;
    const int m = blockIdx.x;
    pdl_trigger();    // the grouped kernel behind this one may start fetching weights
    pdl_wait();       // whatever ran before (possibly still reading this workspace) has finished
    if (m == 0 && threadIdx.x == 0) *status = 0;
    const __nv_bfloat16 *xr = x + (int64_t)m * ldx;
    const int nvec = K >> 3;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);      // 16-byte loads need an aligned row
    uint4 v[GQ_PREP_VECS];
    float amax = 0.0f;
    if (vec_ok) {
#pragma unroll
        for (int i = 0; i < GQ_PREP_VECS; ++i) {
            const int idx = threadIdx.x + i * GQ_PREP_THREADS;
            v[i] = idx < nvec ? __ldg(reinterpret_cast<const uint4 *>(xr) + idx) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int i = 0; i < GQ_PREP_VECS; ++i) amax = fmaxf(amax, amax8(v[i]));
        for (int idx = threadIdx.x + GQ_PREP_VECS * GQ_PREP_THREADS; idx < nvec; idx += GQ_PREP_THREADS)
            amax = fmaxf(amax, amax8(__ldg(reinterpret_cast<const uint4 *>(xr) + idx)));
    } else {
        for (int idx = threadIdx.x; idx < nvec; idx += GQ_PREP_THREADS) {
            uint4 t;
            uint32_t *tw = reinterpret_cast<uint32_t *>(&t);
#pragma unroll
            for (int j = 0; j < 4; ++j) tw[j] = *reinterpret_cast<const uint32_t *>(xr + 8 * idx + 2 * j);
            amax = fmaxf(amax, amax8(t));
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = red[0];
        for (int i = 1; i < GQ_PREP_THREADS / 32; ++i) a = fmaxf(a, red[i]);
        // scale = 2^(9 - e), amax * scale in [512, 1024); identity for a zero, tiny or non-finite row
        int e = 9;
        if (a > 0.0f && a < 3.0e38f) { e = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127; if (e < -100) e = -100; }
        s_scale = __uint_as_float((uint32_t)(127 + 9 - e) << 23);
        ex[m] = __uint_as_float((uint32_t)(127 - 9 + e) << 23);
    }
    __syncthreads();
    const float scale = s_scale;
    // nvec is a multiple of 32 (K of 256), so whole warps run every iteration and the lane-pair exchange is safe
    if (vec_ok) {
#pragma unroll
        for (int i = 0; i < GQ_PREP_VECS; ++i) {
            const int idx = threadIdx.x + i * GQ_PREP_THREADS;
            if (idx < nvec) prep_store8(v[i], idx, scale, M, m, xt);
        }
        for (int idx = threadIdx.x + GQ_PREP_VECS * GQ_PREP_THREADS; idx < nvec; idx += GQ_PREP_THREADS)
            prep_store8(__ldg(reinterpret_cast<const uint4 *>(xr) + idx), idx, scale, M, m, xt);
    } else {
        for (int idx = threadIdx.x; idx < nvec; idx += GQ_PREP_THREADS) {
            uint4 t;
            uint32_t *tw = reinterpret_cast<uint32_t *>(&t);
#pragma unroll
            for (int j = 0; j < 4; ++j) tw[j] = *reinterpret_cast<const uint32_t *>(xr + 8 * idx + 2 * j);
            prep_store8(t, idx, scale, M, m, xt);
        }
    }
}


// ---------------------------------------------------------------------------------------------------
// activation preparation, integer form (1..16 batch rows): one warp per (batch row, k-block).  The 256 activations
// become 16-bit fixed point at a power-of-two scale of their own (exact for every value within 2^-7 of the block's
// largest magnitude, rounded to 2^-16 of it below), stored as the two byte planes, the run sums and the scale
// described at GQ_X8_ROW.  Plays the role of the reference's quantize_activations_256
// (gguf-plugin/gluon/tiles_grouped.py:110-139), which keeps 8 bits per activation; this keeps 16.
// ---------------------------------------------------------------------------------------------------
#define GQ_PREP8_WARPS 8

// The op in front of a linear layer, folded into its activation preparation: what vLLM runs as a kernel of its own
// between two linears reads its input here, on the way into the fixed-point planes, instead of writing a bf16 tensor
// that the preparation reads back.  The arithmetic repeats the unfused kernels' (bf16 wherever they round to bf16).
//   GQ_PRE_SILU_MUL     x = silu(gate) * up with gate = in[:, :K], up = in[:, K:2K]: vLLM's silu_and_mul in front of
//                       down_proj
//   GQ_PRE_ADD_RMSNORM  z = in + residual (stored to residual_out), x = z * rsqrt(mean(z^2) + eps) * weight: vLLM's
//                       fused_add_rms_norm in front of qkv_proj / gate_up_proj; without a residual, plain RMSNorm
// (The reference serves the model with the unfused ops of stock vLLM; its own fusion is the kernel's batching of
// shards, gguf-plugin/gluon/tiles_grouped.py:1204-1313.)
struct PreOp {
    int kind, K;
    const __nv_bfloat16 *weight;          // [K]
    const __nv_bfloat16 *residual;        // [M, ld_res] or null
    __nv_bfloat16 *residual_out;          // [M, ld_res], written when residual is given; never the same memory
    int64_t ld_res;
    float eps;
};

__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(p));
        const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(b[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(p[j]);
    }
}
__device__ __forceinline__ float bf16_round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

// one warp: the 256 activations of batch row m, k-block kb (8 per lane, consecutive) -> planes, run sums, scale
__device__ __forceinline__ void prep8_store(const float (&v)[8], int kb, int m, int M, uint8_t *__restrict__ xt, int lane) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    bool bad = false;
#pragma unroll
    for (int j = 0; j < 8; ++j) bad |= !(fabsf(v[j]) <= 3.0e38f);      // NaN or infinity
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bad = __any_sync(0xffffffffu, bad);
    // scale = 2^(14 - e) with 2^e <= amax < 2^(e+1); a zero block keeps scale 1; a block holding a NaN or an infinity
    // gets a NaN scale, so that every output of that batch row is NaN as it would be in floating point
    int e = 14;
    if (amax > 0.0f) { e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127; if (e < -100) e = -100; }
    const float scale = __uint_as_float((uint32_t)(127 + 14 - e) << 23);
    const float inv = bad ? __uint_as_float(0x7fc00000u) : __uint_as_float((uint32_t)(127 - 14 + e) << 23);
    int xi[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { xi[j] = bad ? 0 : __float2int_rn(v[j] * scale); sum += xi[j]; }
    uint8_t *row = xt + (int64_t)kb * gq_x8_tile_bytes(M) + (int64_t)m * GQ_X8_ROW;
    // this lane holds quads 2*(lane & 1) and 2*(lane & 1) + 1 of run lane >> 1
    const int r = lane >> 1, tq = 2 * (lane & 1);
#pragma unroll
    for (int qd = 0; qd < 2; ++qd) {
        const int *q = xi + 4 * qd;
        const uint32_t hi = ((uint32_t)(q[0] >> 8) & 0xFFu) | (((uint32_t)(q[2] >> 8) & 0xFFu) << 8) | (((uint32_t)(q[1] >> 8) & 0xFFu) << 16) |
                            (((uint32_t)(q[3] >> 8) & 0xFFu) << 24);
        const uint32_t lo = ((uint32_t)q[0] & 0xFFu) | (((uint32_t)q[2] & 0xFFu) << 8) | (((uint32_t)q[1] & 0xFFu) << 16) | (((uint32_t)q[3] & 0xFFu) << 24);
        const int off = 64 * (r >> 2) + 16 * (tq + qd) + 4 * (r & 3);
        *reinterpret_cast<uint32_t *>(row + off) = hi;
        *reinterpret_cast<uint32_t *>(row + 256 + off) = lo;
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if (!(lane & 1)) {
        const float f = (float)sum * 0.015625f;          // exact: |sum| < 2^20
        const __half hi = __float2half_rn(f);
        const __half lo = __float2half_rn(f - __half2float(hi));
        __half *so = reinterpret_cast<__half *>(row + GQ_X8_SUMS);
        so[r] = hi;
        so[16 + r] = lo;
    }
    if (lane == 0) *reinterpret_cast<float *>(xt + (int64_t)kb * gq_x8_tile_bytes(M) + (int64_t)M * GQ_X8_ROW + 4 * m) = inv;
}


template <int PRE>
__global__ void __launch_bounds__(32 * GQ_PREP8_WARPS) prep_x8_kernel(const __nv_bfloat16 *__restrict__ x, int64_t ldx, int M, uint8_t *__restrict__ xt,
                                                                      int *status, const PreOp pre) {
    const int lane = threadIdx.x & 31, kb = blockIdx.x;
    const int m = blockIdx.y * GQ_PREP8_WARPS + (threadIdx.x >> 5);
    pdl_trigger();    // the grouped kernel behind this one may start fetching weights
    pdl_wait();       // whatever ran before (possibly still reading this workspace) has finished
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *status = 0;
    if (m >= M) return;
    const __nv_bfloat16 *xr = x + (int64_t)m * ldx + (int64_t)kb * GQ_QK + 8 * lane;
    float v[8];
    load8(xr, v);
    if constexpr (PRE == GQ_PRE_SILU_MUL) {
        float u[8];
        load8(xr + pre.K, u);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = bf16_round(bf16_round(v[j] / (1.0f + expf(-v[j]))) * u[j]);
    }
    prep8_store(v, kb, m, M, xt, lane);
}

// RMSNorm (with the residual add) in front of the layer: grid (batch rows, k-blocks / 8).  Every CTA sums the squares of
// its whole row (a few KB from L2), then each warp converts one k-block.
__global__ void __launch_bounds__(32 * GQ_PREP8_WARPS) prep_x8_norm_kernel(const __nv_bfloat16 *__restrict__ x, int64_t ldx, int M, uint8_t *__restrict__ xt,
                                                                           int *status, const PreOp pre) {
    __shared__ float red[GQ_PREP8_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, m = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *status = 0;
    const __nv_bfloat16 *row = x + (int64_t)m * ldx;
    const __nv_bfloat16 *res = pre.residual ? pre.residual + (int64_t)m * pre.ld_res : nullptr;
    float ss = 0.0f;
#pragma unroll 4
    for (int c = threadIdx.x; c < pre.K / 8; c += 32 * GQ_PREP8_WARPS) {
        float a[8];
        load8(row + 8 * c, a);
        if (res) {
            float r[8];
            load8(res + 8 * c, r);
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = bf16_round(a[j] + r[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(a[j], a[j], ss);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.0f;
#pragma unroll
    for (int i = 0; i < GQ_PREP8_WARPS; ++i) ss += red[i];
    const float rs = rsqrtf(ss / (float)pre.K + pre.eps);
    const int kb = blockIdx.y * GQ_PREP8_WARPS + warp;
    if (kb < pre.K / GQ_QK) {
        const int64_t col = (int64_t)kb * GQ_QK + 8 * lane;
        float v[8], w[8];
        load8(row + col, v);
        load8(pre.weight + col, w);
        if (res) {
            float r[8];
            load8(res + col, r);
            uint4 z;
            __nv_bfloat162 *zb = reinterpret_cast<__nv_bfloat162 *>(&z);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = bf16_round(v[j] + r[j]);
#pragma unroll
            for (int j = 0; j < 4; ++j) zb[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            __nv_bfloat16 *zo = pre.residual_out + (int64_t)m * pre.ld_res + col;
            if ((reinterpret_cast<uintptr_t>(zo) & 15) == 0) {
                *reinterpret_cast<uint4 *>(zo) = z;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) zo[j] = __float2bfloat16_rn(v[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = bf16_round(bf16_round(v[j] * rs) * w[j]);
        prep8_store(v, kb, m, M, xt, lane);
    }
}

// ---------------------------------------------------------------------------------------------------
// grouped small-batch kernel.  One CTA per descriptor row (64 output columns of one shard x a k-range):
// a producer warp streams the tile's k-blocks (one bulk copy each) plus the matching activation rows through
// an mbarrier ring; four consumer warps each own a 16-row slab, dequantise it in registers and run m16n8k16
// MMAs with the weights on the M side and the batch rows on the N side (8 batch rows per MMA, MT MMAs deep).
// Replaces tiles_grouped_kernel / _run (gguf-plugin/gluon/tiles_grouped.py:343-1201).
// ---------------------------------------------------------------------------------------------------
#define GQ_CONSUMER_WARPS 4
#define GQ_AR_MAX_WORLD 8

// Peer buffers of the fused multiply + all-reduce (row-parallel layers under tensor parallelism).  A rank's buffer:
// [per-unit call counters u32] padded to 4096, then data: 2 sets x world slots of slot_bytes, a slot being an image
// [M][n_total / 2] of 8-byte words {two bf16 values, call number} of one rank's partial output.  A unit is (output
// tile, consumer warp): 16 output columns of all batch rows — the grain at which ranks exchange and sum.
struct ArFused {
    int world, rank, units;          // world == 0: plain output, no exchange
    unsigned long long wait_ns;      // time limit of the wait for the peers' words
    int64_t slot_bytes;
    uint8_t *buf[GQ_AR_MAX_WORLD];
    uint32_t *counters;
};

struct GemvParams {
    const uint8_t *packed;
    const int32_t *desc;
    const uint8_t *xt;
    const float *ex;
    __nv_bfloat16 *y;
    float *partials;
    int *status;
    int M, K, nb, split, stages;
    int64_t ldy, n_total;
    int wbytes_max;      // largest tile bytes in the launch (stage stride of the weight buffers)
    int cb_bytes;                    // shared-memory bytes of the codebook-table region (0: the run has no codebook type)
    int cluster;         // 1: the `split` CTAs of a tile form a thread-block cluster and reduce through shared memory
    int cluster_push;    // 1: the others store their accumulators into slots of the split-0 CTA's shared memory (one cluster barrier)
    const uint8_t *pf_ptr;   // weights the caller will multiply next (or null): prefetched into L2 while this launch computes
    int64_t pf_bytes;
    ArFused ar;
};

template <int TYPE, int MT, int P>
struct PairStep {
    __device__ __forceinline__ static void run(const Dec<TYPE> &dec, const uint8_t *xs, int g, int t, float (&blk)[MT][4], const float (&z)[4]) {
        uint32_t a[2][4];
        dec.template pair<P>(a);
        const uint8_t *xb = xs + g * GQ_XROW_BYTES + 8 * t + 64 * P;   // run 2P at halves 32P + 4t
        if constexpr (Dec<TYPE>::GROUP == 32) {
            float s0, s1;
            dec.template scale<P>(s0, s1);
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                float tmp[4];
                const uint2 b0 = *reinterpret_cast<const uint2 *>(xb + nt * 8 * GQ_XROW_BYTES);
                const uint2 b1 = *reinterpret_cast<const uint2 *>(xb + nt * 8 * GQ_XROW_BYTES + 32);
                mma16816_z(tmp, a[0], b0.x, b0.y, z);
                mma16816(tmp, a[1], b1.x, b1.y);
                blk[nt][0] = fmaf(s0, tmp[0], blk[nt][0]);
                blk[nt][1] = fmaf(s0, tmp[1], blk[nt][1]);
                blk[nt][2] = fmaf(s1, tmp[2], blk[nt][2]);
                blk[nt][3] = fmaf(s1, tmp[3], blk[nt][3]);
            }
        } else {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                float s0, s1;
                if (u == 0) dec.template scale<2 * P>(s0, s1); else dec.template scale<2 * P + 1>(s0, s1);
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    float tmp[4];
                    const uint2 b = *reinterpret_cast<const uint2 *>(xb + nt * 8 * GQ_XROW_BYTES + 32 * u);
                    mma16816_z(tmp, a[u], b.x, b.y, z);
                    blk[nt][0] = fmaf(s0, tmp[0], blk[nt][0]);
                    blk[nt][1] = fmaf(s0, tmp[1], blk[nt][1]);
                    blk[nt][2] = fmaf(s1, tmp[2], blk[nt][2]);
                    blk[nt][3] = fmaf(s1, tmp[3], blk[nt][3]);
                }
            }
        }
        if constexpr (P < 7) PairStep<TYPE, MT, P + 1>::run(dec, xs, g, t, blk, z);
    }
};

// one k-block of one slab: acc += d * sum_groups(scale * (W_int . x)) - sum_sets f * (A'' . run sums)
template <int TYPE, int MT>
__device__ __forceinline__ void slab_kblock(const uint8_t *slab, const uint8_t *xs, const DecAux &aux, int lane, float (&acc)[MT][4],
                                            const float (&z)[4]) {
    Dec<TYPE> dec;
    dec.load(slab, lane, aux);
    const int g = lane >> 2, t = lane & 3;
    float blk[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) blk[nt][0] = blk[nt][1] = blk[nt][2] = blk[nt][3] = 0.f;
    PairStep<TYPE, MT, 0>::run(dec, xs, g, t, blk, z);
    float d0, d1;
    dec.kscale(d0, d1);
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        acc[nt][0] = fmaf(d0, blk[nt][0], acc[nt][0]);
        acc[nt][1] = fmaf(d0, blk[nt][1], acc[nt][1]);
        acc[nt][2] = fmaf(d1, blk[nt][2], acc[nt][2]);
        acc[nt][3] = fmaf(d1, blk[nt][3], acc[nt][3]);
    }
    constexpr int NC = Dec<TYPE>::NCORR;
    if constexpr (NC > 0) {
        uint32_t ac[NC][4];
        float fc[NC][2];
        dec.corr(ac, fc);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            const uint8_t *sb = xs + (nt * 8 + g) * GQ_XROW_BYTES + GQ_XROW_SX + 8 * t;
            const uint2 bh = *reinterpret_cast<const uint2 *>(sb);
            const uint2 bl = *reinterpret_cast<const uint2 *>(sb + 32);
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                float mm[4];
                mma16816_z(mm, ac[j], bh.x, bh.y, z);
                mma16816(mm, ac[j], bl.x, bl.y);
                acc[nt][0] = fmaf(-fc[j][0], mm[0], acc[nt][0]);
                acc[nt][1] = fmaf(-fc[j][0], mm[1], acc[nt][1]);
                acc[nt][2] = fmaf(-fc[j][1], mm[2], acc[nt][2]);
                acc[nt][3] = fmaf(-fc[j][1], mm[3], acc[nt][3]);
            }
        }
    }
}


// The stage ring of one CTA: per stage the weight tile of one k-block and the matching activation tile, filled by two
// bulk copies that complete on the stage's "full" mbarrier; the four consumer warps hand a stage back through its
// "empty" mbarrier, on which the producer warp waits before it refills the stage.  (Letting the last consumer warp to
// finish a stage issue the refill itself — no producer warp, nobody polling — was measured 15 % slower: the arrival
// whose returned state tells a warp that it is the last one, and the copy issue behind it, then sit on the consumer's
// critical path every k-block.)
struct Ring {
    uint8_t *smem;
    uint64_t *full, *empty;
    int stages, stage_bytes, wmax, nk;
    const uint32_t *ar_counter;      // fused all-reduce: this warp's call counter (null: none), read early into ar_prev
};

// Fused all-reduce: lane 0 reads the warp's call counter as soon as the first stage is full — that stage holds
// activations, so every launch in front of this one has finished and the counter is final — and the load's latency
// passes during the multiplication instead of at the start of the exchange.  (The loop below waits on the same phase
// again, which then returns at once.)
__device__ __forceinline__ bool ring_read_counter(const Ring &r, int lane, uint32_t &ar_prev) {
    if (!r.ar_counter) return true;
    if (!mbar_wait(r.full, 0)) return false;
    if (lane == 0) ar_prev = *reinterpret_cast<const volatile uint32_t *>(r.ar_counter);
    return true;
}

// the consumer loop of one warp for a CTA whose shard is of TYPE: waits for each stage, processes its slab,
// releases the stage.  Returns false if a bounded wait ran out.
template <int TYPE, int MT>
__device__ __forceinline__ bool consume(const Ring &r, int slab_off, const DecAux &aux, int lane, float (&acc)[MT][4], uint32_t &ar_prev) {
    float z[4] = {0.f, 0.f, 0.f, 0.f};
    if (!ring_read_counter(r, lane, ar_prev)) return false;
    for (int i = 0, s = 0, round = 0; i < r.nk; ++i) {
        if (!mbar_wait(r.full + s, round & 1)) return false;
        const uint8_t *st = r.smem + (size_t)s * r.stage_bytes;
        slab_kblock<TYPE, MT>(st + slab_off, st + r.wmax, aux, lane, acc, z);
        __syncwarp();
        if (lane == 0) mbar_arrive(r.empty + s);
        if (++s == r.stages) { s = 0; ++round; }
    }
    return true;
}


// ---- integer form (1..16 batch rows): mma.sync m16n8k32 / m16n8k16 on 8-bit operands ----------------------
// D (int32, 16 x 8) = A (16 weight rows x 32 k, 8-bit) . B (32 k x 8 batch rows, 8-bit) [+ C].  AS / BS: operand is signed.
template <bool AS, bool BS>
__device__ __forceinline__ void imma32(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int c0, int c1, int c2, int c3) {
    if constexpr (AS && BS)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
    else if constexpr (AS && !BS)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
    else if constexpr (!AS && BS)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}
template <bool AS, bool BS>
__device__ __forceinline__ void imma16(int (&d)[4], const uint32_t (&a)[2], uint32_t b0) {
    if constexpr (AS && BS)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(b0), "r"(0));
    else if constexpr (AS && !BS)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(b0), "r"(0));
    else if constexpr (!AS && BS)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(b0), "r"(0));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(b0), "r"(0));
}

template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F &&f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

// one k-block of one slab in the integer form.  `xs` is the staged activation tile of the k-block (rows of GQ_X8_ROW
// bytes, then the batch rows' scales at xs_off).  Per MMA the weights are 8-bit integers and the activations one of the
// two byte planes (x = 256 hi + lo with hi signed, lo unsigned); int32 sums per plane are exact.  At the end of the
// k-block:  acc += 2^-e[n] * ( d[row] * (256 sumH + sumL) - f[row] * 64 * sum_run A''[row][run] * Sx[run][n] ).
template <int TYPE, int MT>
__device__ __forceinline__ void slab_kblock8(const uint8_t *slab, const uint8_t *xs, int xs_off, const DecAux8 &aux, int lane, float (&acc)[MT][4]) {
    using D = Dec8<TYPE>;
    constexpr bool AS = D::A_SIGNED;
    D dec;
    dec.load(slab, lane, aux);
    const int g = lane >> 2, t = lane & 3;
    const uint8_t *xb = xs + g * GQ_X8_ROW + 16 * t;     // unit (i, t) of batch row g; + 8 nt rows, + 256 for the low plane
    int aH[MT][4], aL[MT][4], bH[MT][4], bL[MT][4];
    float bf[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) { aH[nt][j] = 0; aL[nt][j] = 0; bH[nt][j] = 0; bL[nt][j] = 0; bf[nt][j] = 0.f; }
    static_for<0, 4>([&](auto i_) {
        constexpr int I = decltype(i_)::value;
        uint4 xh[MT], xl[MT];
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            xh[nt] = ld16(xb + nt * 8 * GQ_X8_ROW + 64 * I);
            xl[nt] = ld16(xb + nt * 8 * GQ_X8_ROW + 64 * I + 256);
        }
        if constexpr (D::SCHEME == GQ_S16) {
            static_for<0, 4>([&](auto r_) {
                constexpr int RR = decltype(r_)::value, R = 4 * I + RR;
                uint32_t a[2];
                dec.template step16<R>(a);
                int s0, s1;
                dec.template iscale16<R>(s0, s1);
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    int th[4], tl[4];
                    imma16<AS, true>(th, a, w4(xh[nt], RR));
                    imma16<AS, false>(tl, a, w4(xl[nt], RR));
                    aH[nt][0] += s0 * th[0]; aH[nt][1] += s0 * th[1]; aH[nt][2] += s1 * th[2]; aH[nt][3] += s1 * th[3];
                    aL[nt][0] += s0 * tl[0]; aL[nt][1] += s0 * tl[1]; aL[nt][2] += s1 * tl[2]; aL[nt][3] += s1 * tl[3];
                }
            });
        } else {
            static_for<0, 2>([&](auto v_) {
                constexpr int V = decltype(v_)::value, S = 2 * I + V;
                uint32_t a[4];
                dec.template step<S>(a);
                int s0 = 1, s1 = 1;
                float f0 = 1.f, f1 = 1.f;
                if constexpr (D::SCHEME == GQ_S32) dec.template iscale<S>(s0, s1);
                if constexpr (D::SCHEME == GQ_F32) dec.template fscale<S>(f0, f1);
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const uint32_t bh0 = V ? xh[nt].z : xh[nt].x, bh1 = V ? xh[nt].w : xh[nt].y;
                    const uint32_t bl0 = V ? xl[nt].z : xl[nt].x, bl1 = V ? xl[nt].w : xl[nt].y;
                    if constexpr (D::SCHEME == GQ_FOLD) {
                        // two accumulator chains per plane (even / odd k-steps): half the dependent MMAs in a row
                        if constexpr (V == 0) {
                            imma32<AS, true>(aH[nt], a, bh0, bh1, aH[nt][0], aH[nt][1], aH[nt][2], aH[nt][3]);
                            imma32<AS, false>(aL[nt], a, bl0, bl1, aL[nt][0], aL[nt][1], aL[nt][2], aL[nt][3]);
                        } else {
                            imma32<AS, true>(bH[nt], a, bh0, bh1, bH[nt][0], bH[nt][1], bH[nt][2], bH[nt][3]);
                            imma32<AS, false>(bL[nt], a, bl0, bl1, bL[nt][0], bL[nt][1], bL[nt][2], bL[nt][3]);
                        }
                    } else {
                        int th[4], tl[4];
                        imma32<AS, true>(th, a, bh0, bh1, 0, 0, 0, 0);
                        imma32<AS, false>(tl, a, bl0, bl1, 0, 0, 0, 0);
                        if constexpr (D::SCHEME == GQ_S32) {
                            aH[nt][0] += s0 * th[0]; aH[nt][1] += s0 * th[1]; aH[nt][2] += s1 * th[2]; aH[nt][3] += s1 * th[3];
                            aL[nt][0] += s0 * tl[0]; aL[nt][1] += s0 * tl[1]; aL[nt][2] += s1 * tl[2]; aL[nt][3] += s1 * tl[3];
                        } else {
                            bf[nt][0] = fmaf(f0, (float)(th[0] * 256 + tl[0]), bf[nt][0]);
                            bf[nt][1] = fmaf(f0, (float)(th[1] * 256 + tl[1]), bf[nt][1]);
                            bf[nt][2] = fmaf(f1, (float)(th[2] * 256 + tl[2]), bf[nt][2]);
                            bf[nt][3] = fmaf(f1, (float)(th[3] * 256 + tl[3]), bf[nt][3]);
                        }
                    }
                }
            });
        }
    });
    float d0, d1;
    dec.kscale(d0, d1);
    uint32_t ac[4] = {0u, 0u, 0u, 0u};
    float fc[2] = {0.f, 0.f};
    if constexpr (D::NCORR > 0) {
        dec.corr(ac, fc);
        fc[0] *= -64.0f; fc[1] *= -64.0f;
    }
    const float z[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        float tot[4];
        if constexpr (D::SCHEME == GQ_F32) {
#pragma unroll
            for (int j = 0; j < 4; ++j) tot[j] = bf[nt][j];
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) tot[j] = (j < 2 ? d0 : d1) * fmaf((float)(aH[nt][j] + bH[nt][j]), 256.0f, (float)(aL[nt][j] + bL[nt][j]));
        }
        if constexpr (D::NCORR > 0) {
            const uint8_t *sb = xs + (nt * 8 + g) * GQ_X8_ROW + GQ_X8_SUMS + 8 * t;
            const uint2 bh = *reinterpret_cast<const uint2 *>(sb);
            const uint2 bl = *reinterpret_cast<const uint2 *>(sb + 32);
            float mm[4];
            mma16816_z(mm, ac, bh.x, bh.y, z);
            mma16816(mm, ac, bl.x, bl.y);
#pragma unroll
            for (int j = 0; j < 4; ++j) tot[j] = fmaf(fc[j >> 1], mm[j], tot[j]);
        }
        const float2 sx = *reinterpret_cast<const float2 *>(xs + xs_off + (nt * 8 + 2 * t) * 4);
        acc[nt][0] = fmaf(sx.x, tot[0], acc[nt][0]);
        acc[nt][1] = fmaf(sx.y, tot[1], acc[nt][1]);
        acc[nt][2] = fmaf(sx.x, tot[2], acc[nt][2]);
        acc[nt][3] = fmaf(sx.y, tot[3], acc[nt][3]);
    }
}


template <int TYPE, int MT>
__device__ __forceinline__ bool consume8(const Ring &r, int xs_off, int slab_off, const DecAux8 &aux, int lane, float (&acc)[MT][4], uint32_t &ar_prev) {
    if (!ring_read_counter(r, lane, ar_prev)) return false;
    for (int i = 0, s = 0, round = 0; i < r.nk; ++i) {
        if (!mbar_wait(r.full + s, round & 1)) return false;
        const uint8_t *st = r.smem + (size_t)s * r.stage_bytes;
        slab_kblock8<TYPE, MT>(st + slab_off, st + r.wmax, xs_off, aux, lane, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(r.empty + s);
        if (++s == r.stages) { s = 0; ++round; }
    }
    return true;
}

// One warp's share of the fused all-reduce.  `blk` (shared memory) holds the warp's bf16 block [M][16] of this
// rank's partial output (columns col .. col + ncols - 1 of every batch row; col and ncols even).  Push based, one
// shot, and free of fences: every pair of bf16 values travels as one 8-byte word {values, call number}, stored
// whole (an aligned 64-bit store is single-copy atomic) into this rank's slot of every rank's buffer — plain stores
// through peer pointers, own buffer included.  The receiver polls the words of its OWN memory until their call
// number is this call's (with a time limit), adds the ranks' values in rank order in fp32 and rounds once into y:
// the data is its own flag, so no release / acquire at system scope is needed (on a busy SM those cost several
// microseconds per warp).  No loads from remote memory, no multicast.  The call number lives in device memory per
// (tile, warp) and selects one of two slot sets; a stale word of the same set carries an older number, and a rank
// cannot run two calls ahead of a peer because each call needs every peer's words of that call.
__device__ __noinline__ void fused_allreduce_block(const GemvParams &p, const uint32_t *blk, int unit, int col, int ncols, int lane, uint32_t prev) {
    const ArFused &a = p.ar;
    // the call number: one more than the counter, which lane 0 read while the first k-block was being multiplied
    const uint32_t seq = __shfl_sync(0xffffffffu, prev, 0) + 1;
    const uint32_t set = seq & 1u;
    const int M = p.M, half = ncols >> 1;
    const int64_t row_words = p.n_total >> 1, slot_words = a.slot_bytes >> 3;
    const int64_t first = (int64_t)(col >> 1);
    const int n_el = M * half;
    for (int pr = 0; pr < a.world; ++pr) {
        unsigned long long *dst = reinterpret_cast<unsigned long long *>(a.buf[pr]) + ((int64_t)set * a.world + a.rank) * slot_words + first;
        for (int e = lane; e < n_el; e += 32) {
            const int n = e / half, c2 = e - n * half;
            const unsigned long long w = (unsigned long long)blk[n * 8 + c2] | ((unsigned long long)seq << 32);
            asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(dst + n * row_words + c2), "l"(w) : "memory");
        }
    }
    const unsigned long long *src = reinterpret_cast<const unsigned long long *>(a.buf[a.rank]) + (int64_t)set * a.world * slot_words + first;
    bool fail = false;
    uint64_t t0 = 0;
    // Two elements per lane and pass; the words of all ranks for both are requested before any is looked at, so a pass
    // costs one trip to the L2 whatever the number of ranks (polled one after the other, the 2 x 8 dependent loads of an
    // 8-rank exchange took longer than the kernel in front of them).
    for (int e0 = lane; e0 < n_el; e0 += 64) {
        const int e1 = e0 + 32;
        const bool has1 = e1 < n_el;
        const int n0 = e0 / half, c0 = e0 - n0 * half, n1 = has1 ? e1 / half : n0, c1 = has1 ? e1 - n1 * half : c0;
        const unsigned long long *q0 = src + n0 * row_words + c0, *q1 = src + n1 * row_words + c1;
        unsigned long long w0[GQ_AR_MAX_WORLD], w1[GQ_AR_MAX_WORLD];
        const uint32_t all = (1u << a.world) - 1u;
        uint32_t pending = all | (has1 ? all << 8 : 0u);
        for (uint32_t it = 0; pending; ++it) {
#pragma unroll
            for (int r = 0; r < GQ_AR_MAX_WORLD; ++r) {
                if ((pending >> r) & 1u) asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w0[r]) : "l"(q0 + (int64_t)r * slot_words) : "memory");
                if ((pending >> (8 + r)) & 1u) asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w1[r]) : "l"(q1 + (int64_t)r * slot_words) : "memory");
            }
#pragma unroll
            for (int r = 0; r < GQ_AR_MAX_WORLD; ++r) {
                if (((pending >> r) & 1u) && (uint32_t)(w0[r] >> 32) == seq) pending &= ~(1u << r);
                if (((pending >> (8 + r)) & 1u) && (uint32_t)(w1[r] >> 32) == seq) pending &= ~(1u << (8 + r));
            }
            if (pending && (it & 255u) == 255u) {      // the clock is read only once a wait has become long
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > a.wait_ns) { fail = true; break; }
            }
        }
        if (fail) break;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (k == 1 && !has1) break;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int r = 0; r < GQ_AR_MAX_WORLD; ++r) {
                if (r < a.world) {
                    const uint32_t v = (uint32_t)(k ? w1[r] : w0[r]);
                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v));
                    s0 += f.x; s1 += f.y;
                }
            }
            __nv_bfloat16 *yp = p.y + (int64_t)(k ? n1 : n0) * p.ldy + col + 2 * (k ? c1 : c0);
            if (!(reinterpret_cast<uintptr_t>(yp) & 3)) *reinterpret_cast<__nv_bfloat162 *>(yp) = __floats2bfloat162_rn(s0, s1);
            else { yp[0] = __float2bfloat16_rn(s0); yp[1] = __float2bfloat16_rn(s1); }
        }
    }
    fail = __any_sync(0xffffffffu, fail);
    if (lane == 0) {
        if (fail) report_status(p.status, GQ_DEV_TIMEOUT);
        a.counters[unit] = seq;
    }
}

// MINB = CTAs per SM the compiler must leave room for (0: its own choice).  For the M <= 8 form 4 gives it 96
// registers, which it turns into more loads and MMAs in flight per warp: measured 14 % faster than the 72-register
// build when a CTA walks ten or more k-blocks, a little slower on launches of many short CTAs, 2 % faster on the
// mixed stack.  (Compiling both and choosing per call was slower than either alone: alternating between two large
// kernels costs more in instruction-cache misses at every launch than the better fit gains.)  The 17..32-row form
// is about 10 % faster with room for two CTAs (168 registers) than with the compiler's own 144; the 16- and 64-row
// forms were best left alone.
//
// FORM 0: fp16 form (activations as fp16, weights decoded to fp16 pairs, m16n8k16 f16 MMAs), used for 17..64 batch rows.
// FORM 1: integer form (activations as two byte planes, weights decoded to 8-bit quads, m16n8k32 / m16n8k16 integer
// MMAs), used for 1..16 batch rows: about half the instructions per weight.
// ONLY: 0 compiles the decoders of all eleven types (the branch is per CTA); a GGML type id compiles that type alone,
// for launches whose shards all share it (a smaller kernel; most launches of a real model are such).
template <int MT, int FORM>
__host__ __device__ constexpr int gq_stage_xbytes() { return FORM ? 8 * MT * GQ_X8_ROW + 32 * MT : 8 * MT * GQ_XROW_BYTES; }

template <int MT, int MINB, int FORM, int ONLY>
__global__ void __launch_bounds__(32 * (GQ_CONSUMER_WARPS + 1), MINB) gemv_grouped_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: [stages x (weights wbytes_max | activation tile)] [full barriers] [empty barriers] [IQ3_S grid] [reduction scratch]
    const int stages = p.stages, wmax = p.wbytes_max, M = p.M;
    constexpr int xbytes = gq_stage_xbytes<MT, FORM>();
    const int stage_bytes = wmax + xbytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + (size_t)stages * stage_bytes);
    uint64_t *empty = full + stages;
    uint2 *grid_s = reinterpret_cast<uint2 *>(empty + stages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int32_t *d = p.desc + (int64_t)blockIdx.x * GQ_DESC_WORDS;
    const int64_t off = (int64_t)d[0] * 16;
    const int type = ONLY ? ONLY : d[1];
    const int col0 = d[2], nvalid = d[3], kb0 = d[4], kb1 = d[5], split_idx = d[6];
    const int B = gq_type_bytes(type);
    const int tile_bytes = 64 * B;
    const int nk = kb1 - kb0;

    // a tile whose type contradicts the call's run_info (not the single type it named, or a codebook type it did not
    // announce, which has no table space): report and leave (every CTA of a cluster works on the same tile, so a cluster
    // leaves as one)
    if ((ONLY != 0 && d[1] != ONLY) || (gq_cb_kind(type) >= 0 && gq_cb_bytes(gq_cb_kind(type), FORM) > p.cb_bytes)) {
        if (threadIdx.x == 0) { pdl_wait(); report_status(p.status, GQ_DEV_BAD_SHAPE); }      // after the preparation kernel has cleared the word
        return;
    }
    Ring ring;
    ring.smem = smem; ring.full = full; ring.empty = empty;
    ring.stages = stages; ring.stage_bytes = stage_bytes; ring.wmax = wmax; ring.nk = nk;
    ring.ar_counter = (p.ar.world > 0 && (p.split == 1 || p.cluster) && split_idx == 0 && warp < GQ_CONSUMER_WARPS)
                          ? p.ar.counters + (int64_t)(blockIdx.x / (unsigned)p.split) * GQ_CONSUMER_WARPS + warp : nullptr;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, GQ_CONSUMER_WARPS); }
        fence_barrier_init();
    }
    __syncthreads();
    // the codebook table of this CTA's type, at the start of the table region: filled by the consumer warps while the
    // producer's first copies are already on their way, closed by a barrier among the consumers only
    if (p.cb_bytes && warp < GQ_CONSUMER_WARPS) {
        uint32_t *g32 = reinterpret_cast<uint32_t *>(grid_s);
        if ((ONLY == 0 || ONLY == GQ_IQ3_S) && type == GQ_IQ3_S) {
            if constexpr (FORM) { for (int i = threadIdx.x; i < 512; i += 32 * GQ_CONSUMER_WARPS) g32[i] = iq3s_grid_entry8(c_iq3s_grid[i]); }
            else { for (int i = threadIdx.x; i < 512; i += 32 * GQ_CONSUMER_WARPS) grid_s[i] = iq3s_grid_entry(c_iq3s_grid[i]); }
        }
        if ((ONLY == 0 || ONLY == GQ_IQ3_XXS) && type == GQ_IQ3_XXS) {
            if constexpr (FORM) { for (int i = threadIdx.x; i < 256; i += 32 * GQ_CONSUMER_WARPS) g32[i] = iq3s_grid_entry8(c_iq3xxs_grid[i]); }
            else { for (int i = threadIdx.x; i < 256; i += 32 * GQ_CONSUMER_WARPS) grid_s[i] = iq3s_grid_entry(c_iq3xxs_grid[i]); }
        }
        if ((ONLY == 0 || ONLY == GQ_IQ2_XXS) && type == GQ_IQ2_XXS) {
            for (int i = threadIdx.x; i < 512; i += 32 * GQ_CONSUMER_WARPS) g32[i] = iq3s_grid_entry8(c_iq2xxs_grid[i]);
        }
        if ((ONLY == 0 || ONLY == GQ_IQ2_XS) && type == GQ_IQ2_XS) {
            for (int i = threadIdx.x; i < 1024; i += 32 * GQ_CONSUMER_WARPS) g32[i] = iq3s_grid_entry8(c_iq2xs_grid[i]);
        }
        if ((ONLY == 0 || ONLY == GQ_IQ2_S) && type == GQ_IQ2_S) {
            for (int i = threadIdx.x; i < 2048; i += 32 * GQ_CONSUMER_WARPS) g32[i] = iq3s_grid_entry8(c_iq2s_grid[i]);
        }
        if ((ONLY == 0 || ONLY == GQ_IQ1_M) && type == GQ_IQ1_M) {
            for (int i = threadIdx.x; i < 4096; i += 32 * GQ_CONSUMER_WARPS) g32[i] = iq3s_grid_entry8(c_iq1_grid[i]);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * GQ_CONSUMER_WARPS) : "memory");
    }
    // push-form split-K: a CTA may store into the split-0 CTA's shared memory only once that CTA is known to run;
    // every thread enters this rendezvous here and collects it just before its first remote store (or before the
    // closing barrier), long after everyone has arrived
    const bool push = p.cluster && p.cluster_push;
    if (push) cluster_arrive_relaxed();

    if (warp == GQ_CONSUMER_WARPS) {
        // ---- producer: one thread; per k-block one bulk copy of the weight tile and one of the activation tile.
        // The weights do not depend on the kernel in front of this one, so the first stages' weight copies go out
        // before the dependency wait; the activation tiles (written by the preparation kernel) follow it.  The
        // kernel behind this one is allowed to start launching when this CTA has two k-blocks left. ----
        if (lane == 0) {
            const uint8_t *src = p.packed + off + (int64_t)kb0 * tile_bytes;
            const uint32_t abytes = FORM ? (uint32_t)gq_x8_tile_bytes(M) : (uint32_t)M * GQ_XROW_BYTES;
            const uint8_t *xsrc = p.xt + (int64_t)kb0 * abytes;
            const int pre = nk < stages ? nk : stages;
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(full + i, (uint32_t)tile_bytes + abytes);
                bulk_g2s(smem + (size_t)i * stage_bytes, src + (int64_t)i * tile_bytes, (uint32_t)tile_bytes, full + i);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) bulk_g2s(smem + (size_t)i * stage_bytes + wmax, xsrc + (int64_t)i * abytes, abytes, full + i);
            if (nk - pre <= 2) pdl_trigger();
            for (int i = pre, s = 0, round = 1; i < nk; ++i) {
                if (!mbar_wait_parked(empty + s, (round - 1) & 1)) { report_status(p.status, GQ_DEV_TIMEOUT); break; }
                uint8_t *st = smem + (size_t)s * stage_bytes;
                mbar_expect_tx(full + s, (uint32_t)tile_bytes + abytes);
                bulk_g2s(st, src + (int64_t)i * tile_bytes, (uint32_t)tile_bytes, full + s);
                bulk_g2s(st + wmax, xsrc + (int64_t)i * abytes, abytes, full + s);
                if (i == nk - 3) pdl_trigger();
                if (++s == stages) { s = 0; ++round; }
            }
        }
        else if (p.pf_ptr) {
            // the producer warp's other lanes: this CTA's share of the next layer's weights, 16 KB per request
            const int64_t chunk = 16384;
            const int64_t n_chunks = (p.pf_bytes + chunk - 1) / chunk;
            for (int64_t c = (int64_t)blockIdx.x * 31 + (lane - 1); c < n_chunks; c += (int64_t)gridDim.x * 31) {
                const int64_t o = c * chunk;
                const int64_t sz = (p.pf_bytes - o < chunk ? p.pf_bytes - o : chunk) & ~(int64_t)15;
                if (sz > 0) prefetch_l2_bulk(p.pf_ptr + o, (uint32_t)sz);
            }
        }
        if (!p.cluster) return;
        if (push) cluster_wait();
        cluster_sync_all();     // the reduction's cluster barriers need every thread of every CTA
        if (!push) cluster_sync_all();
        return;
    }

    // ---- consumers ----
    float acc[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    bool ok = true;
    uint32_t ar_prev = 0;
    const int slab_off = warp * 16 * B;
    // the IQ4 codebook in four registers: signed bytes for the integer form, + 128 for the fp16 form
    Iq4Table iq4;
    {
        uint32_t tb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            tb[j] = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) tb[j] |= (uint32_t)(uint8_t)(c_iq4_kvalues[4 * j + i] + (FORM ? 0 : 128)) << (8 * i);
        }
        iq4 = {tb[0], tb[1], tb[2], tb[3]};
    }
    if constexpr (FORM) {
        DecAux8 aux;
        aux.grid = reinterpret_cast<const uint32_t *>(grid_s);
        aux.iq4 = iq4;
        const int xs_off = M * GQ_X8_ROW;
#define GQ_CONSUME(T) case T: ok = consume8<T, MT>(ring, xs_off, slab_off, aux, lane, acc, ar_prev); break;
        if constexpr (ONLY != 0) {
            ok = consume8<(ONLY ? ONLY : GQ_Q4_K), MT>(ring, xs_off, slab_off, aux, lane, acc, ar_prev);
        } else {
            switch (type) {
                GQ_CONSUME(GQ_Q4_0) GQ_CONSUME(GQ_Q5_0) GQ_CONSUME(GQ_Q8_0) GQ_CONSUME(GQ_Q2_K) GQ_CONSUME(GQ_Q3_K) GQ_CONSUME(GQ_Q4_K)
                GQ_CONSUME(GQ_Q5_K) GQ_CONSUME(GQ_Q6_K) GQ_CONSUME(GQ_IQ4_NL) GQ_CONSUME(GQ_IQ3_S) GQ_CONSUME(GQ_IQ4_XS) GQ_CONSUME(GQ_IQ3_XXS)
                GQ_CONSUME(GQ_IQ2_XXS) GQ_CONSUME(GQ_IQ2_XS) GQ_CONSUME(GQ_IQ2_S) GQ_CONSUME(GQ_IQ1_M)
            }
        }
#undef GQ_CONSUME
    } else {
        DecAux aux;
        aux.grid = grid_s;
        aux.iq4 = iq4;
#define GQ_CONSUME(T) case T: ok = consume<T, MT>(ring, slab_off, aux, lane, acc, ar_prev); break;
        switch (type) {
            GQ_CONSUME(GQ_Q4_0) GQ_CONSUME(GQ_Q5_0) GQ_CONSUME(GQ_Q8_0) GQ_CONSUME(GQ_Q2_K) GQ_CONSUME(GQ_Q3_K) GQ_CONSUME(GQ_Q4_K)
            GQ_CONSUME(GQ_Q5_K) GQ_CONSUME(GQ_Q6_K) GQ_CONSUME(GQ_IQ4_NL) GQ_CONSUME(GQ_IQ3_S) GQ_CONSUME(GQ_IQ4_XS) GQ_CONSUME(GQ_IQ3_XXS)
                GQ_CONSUME(GQ_IQ2_XXS) GQ_CONSUME(GQ_IQ2_XS) GQ_CONSUME(GQ_IQ2_S) GQ_CONSUME(GQ_IQ1_M)
        }
#undef GQ_CONSUME
    }
    if (!ok && lane == 0) report_status(p.status, GQ_DEV_TIMEOUT);   // the result is then incomplete; the status word says so

    // ---- epilogue: rows of the MMA are output columns, columns of the MMA are batch rows ----
    const int g = lane >> 2, t = lane & 3;
    // scratch of its own behind the ring (a slower warp may still read the ring): GQ_CONSUMER_WARPS x MT x 512 bytes
    float4 *red = reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(grid_s) + p.cb_bytes);
    if (push) {
        cluster_wait();         // the rendezvous entered at the start: every CTA of the cluster is running
        // split-K inside a cluster, push form: the CTAs of splits 1.. store their accumulators into their slot of the
        // split-0 CTA's scratch through distributed shared memory; one cluster barrier (release / acquire) later that
        // CTA adds the slots from its own shared memory, in split order, and writes bf16 once.  No partial sums in
        // HBM, no second kernel, fixed order of the additions.
        if (split_idx != 0) {
            const uint32_t dst = map_to_rank(smem_u32(red), 0u) + (uint32_t)((split_idx - 1) * GQ_CONSUMER_WARPS * MT * 512);
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
                st_cluster_f4(dst + (uint32_t)(((warp * MT + nt) * 32 + lane) * 16), acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
        }
        cluster_sync_all();
        if (split_idx != 0) return;
        for (int s = 1; s < p.split; ++s) {
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                const float4 v = red[((s - 1) * GQ_CONSUMER_WARPS * MT + warp * MT + nt) * 32 + lane];
                acc[nt][0] += v.x; acc[nt][1] += v.y; acc[nt][2] += v.z; acc[nt][3] += v.w;
            }
        }
        __syncwarp();       // the warp's part of slot 0 becomes its scratch again below
    } else if (p.cluster) {
        // pull form (when the slots do not fit without costing a resident CTA): every CTA parks its accumulators in
        // its own shared memory, the CTA of split 0 adds the others' in split order through distributed shared
        // memory between two cluster barriers
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) red[(warp * MT + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
        cluster_sync_all();
        if (split_idx == 0) {
            const uint32_t my = smem_u32(red);
            for (int s = 1; s < p.split; ++s) {
                const uint32_t peer = map_to_rank(my, (uint32_t)s);
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    const float4 v = ld_cluster_f4(peer + (uint32_t)(((warp * MT + nt) * 32 + lane) * 16));
                    acc[nt][0] += v.x; acc[nt][1] += v.y; acc[nt][2] += v.z; acc[nt][3] += v.w;
                }
            }
        }
        cluster_sync_all();      // peers stay resident until their shared memory has been read
        if (split_idx != 0) return;
    }
    if (p.ar.world > 0 && (p.split == 1 || p.cluster)) {
        // tensor parallel, row-parallel layer: this rank's partial output does not go to y but, as bf16, through
        // the warp's scratch to every rank; y receives the sum over ranks (fused_allreduce_tile)
        __nv_bfloat16 *blk = reinterpret_cast<__nv_bfloat16 *>(reinterpret_cast<uint8_t *>(red) + warp * MT * 512);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int rl = g + 8 * (j >> 1), n = nt * 8 + 2 * t + (j & 1);
                const bool valid = ok && warp * 16 + rl < nvalid && n < p.M;
                blk[n * 16 + rl] = __float2bfloat16_rn(valid ? (FORM ? acc[nt][j] : acc[nt][j] * p.ex[n]) : 0.0f);
            }
        __syncwarp();
        const int ncols = nvalid - warp * 16 < 16 ? nvalid - warp * 16 : 16;
        if (ncols > 0) {
            if (((col0 | ncols | (int)p.n_total) & 1) && lane == 0) report_status(p.status, GQ_DEV_BAD_SHAPE);    // pairs of columns travel together
            else fused_allreduce_block(p, reinterpret_cast<const uint32_t *>(blk), (int)(blockIdx.x / (unsigned)p.split) * GQ_CONSUMER_WARPS + warp,
                                       col0 + warp * 16, ncols, lane, ar_prev);
        }
        return;
    }
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = warp * 16 + g + 8 * (j >> 1);      // row inside the 64-row tile
            const int n = nt * 8 + 2 * t + (j & 1);          // batch row
            if (ok && r < nvalid && n < p.M) {
                const float v = FORM ? acc[nt][j] : acc[nt][j] * p.ex[n];    // the integer form scales per k-block
                if (p.split == 1 || p.cluster) p.y[(int64_t)n * p.ldy + col0 + r] = __float2bfloat16_rn(v);
                else p.partials[((int64_t)split_idx * p.M + n) * p.n_total + col0 + r] = v;
            }
        }
}

// Y = sum over splits of the fp32 partials, rounded once to bf16 (reference: sum_partials,
// gguf-plugin/gluon/tiles_grouped.py:142-162)
__global__ void __launch_bounds__(256) sum_partials_kernel(const float *__restrict__ P, int S, int64_t M, int64_t n_total,
                                                           __nv_bfloat16 *__restrict__ y, int64_t ldy) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= M * n_total) return;
    float a = 0.f;
    for (int s = 0; s < S; ++s) a += P[(int64_t)s * M * n_total + i];
    const int64_t m = i / n_total, c = i - m * n_total;
    y[m * ldy + c] = __float2bfloat16_rn(a);
}

// ---------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------
static int ensure_tables() {
    // per-device one-time upload of the format tables
    static std::atomic<unsigned long long> done_mask{0};
    int dev = 0;
    GQ_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && (done_mask.load() >> dev) & 1ull) return GQ_OK;
    GQ_CUDA(cudaMemcpyToSymbol(c_iq3s_grid, GQ_IQ3S_GRID, sizeof GQ_IQ3S_GRID));
    GQ_CUDA(cudaMemcpyToSymbol(c_iq3xxs_grid, GQ_IQ3XXS_GRID, sizeof GQ_IQ3XXS_GRID));
    GQ_CUDA(cudaMemcpyToSymbol(c_iq2xxs_grid, GQ_IQ2XXS_GRID, sizeof GQ_IQ2XXS_GRID));
    GQ_CUDA(cudaMemcpyToSymbol(c_iq2xs_grid, GQ_IQ2XS_GRID, sizeof GQ_IQ2XS_GRID));
    GQ_CUDA(cudaMemcpyToSymbol(c_iq2s_grid, GQ_IQ2S_GRID, sizeof GQ_IQ2S_GRID));
    GQ_CUDA(cudaMemcpyToSymbol(c_iq1_grid, GQ_IQ1_GRID, sizeof GQ_IQ1_GRID));
    GQ_CUDA(cudaMemcpyToSymbol(c_iq4_kvalues, GQ_IQ4_KVALUES, sizeof GQ_IQ4_KVALUES));
    if (dev < 64) done_mask.fetch_or(1ull << dev);
    return GQ_OK;
}

static int check_tensor_args(int type, int64_t n_out, int64_t K) {
    if (!gq_type_bytes(type)) return GQ_ERR_TYPE;
    if (n_out < 0 || K <= 0 || K % GQ_QK || K / GQ_QK > 65535) return GQ_ERR_SHAPE;
    return GQ_OK;
}

extern "C" int gq_repack(int type, const void *raw_dev, int64_t n_out, int64_t K, int64_t raw_row_stride, void *out_dev, void *stream) {
    if (int rc = check_tensor_args(type, n_out, K)) return rc;
    const int B = gq_type_bytes(type);
    const int nb = (int)(K / GQ_QK);
    if (n_out == 0) return GQ_OK;
    if (!raw_dev || !out_dev || ((uintptr_t)out_dev & 15) || raw_row_stride < (int64_t)nb * B) return GQ_ERR_ARG;
    const int64_t slabs = ((n_out + 63) / 64) * 4;
    if (slabs > 0x7fffffff) return GQ_ERR_LIMIT;
    repack_kernel<<<dim3((unsigned)slabs, (unsigned)nb), 256, 0, (cudaStream_t)stream>>>(type, B, (const uint8_t *)raw_dev, n_out, nb,
                                                                                     raw_row_stride, (uint8_t *)out_dev);
    GQ_LAUNCHED();
    return GQ_OK;
}

extern "C" int gq_unrepack(int type, const void *tiles_dev, int64_t n_out, int64_t K, void *raw_dev, int64_t raw_row_stride, void *stream) {
    if (int rc = check_tensor_args(type, n_out, K)) return rc;
    const int B = gq_type_bytes(type);
    const int nb = (int)(K / GQ_QK);
    if (n_out == 0) return GQ_OK;
    if (!raw_dev || !tiles_dev || ((uintptr_t)tiles_dev & 15) || raw_row_stride < (int64_t)nb * B) return GQ_ERR_ARG;
    const int64_t slabs = ((n_out + 63) / 64) * 4;
    if (slabs > 0x7fffffff) return GQ_ERR_LIMIT;
    unrepack_kernel<<<dim3((unsigned)slabs, (unsigned)nb), 256, 0, (cudaStream_t)stream>>>(type, B, (const uint8_t *)tiles_dev, n_out, nb,
                                                                                       (uint8_t *)raw_dev, raw_row_stride);
    GQ_LAUNCHED();
    return GQ_OK;
}

extern "C" int gq_dequant(int type, const void *tiles_dev, int64_t n_out, int64_t K, void *out_dev, int out_dtype, int64_t ld, void *stream) {
    if (int rc = check_tensor_args(type, n_out, K)) return rc;
    const int B = gq_type_bytes(type);
    const int nb = (int)(K / GQ_QK);
    if (n_out == 0) return GQ_OK;
    if (!out_dev || !tiles_dev || ((uintptr_t)tiles_dev & 15) || ld < K || (out_dtype != 0 && out_dtype != 1)) return GQ_ERR_ARG;
    if (int rc = ensure_tables()) return rc;
    const int64_t slabs = ((n_out + 63) / 64) * 4;
    if (slabs > 0x7fffffff) return GQ_ERR_LIMIT;
    dequant_kernel<<<dim3((unsigned)slabs, (unsigned)nb), 256, 0, (cudaStream_t)stream>>>(type, B, (const uint8_t *)tiles_dev, n_out, nb, out_dev,
                                                                                      out_dtype, ld);
    GQ_LAUNCHED();
    return GQ_OK;
}

extern "C" int64_t gq_desc_rows(int n_shards, const int64_t *n_outs, int split) {
    if (n_shards <= 0 || !n_outs || split < 1) return GQ_ERR_ARG;
    int64_t tiles = 0;
    for (int i = 0; i < n_shards; ++i) { if (n_outs[i] < 0) return GQ_ERR_SHAPE; tiles += (n_outs[i] + 63) / 64; }
    return tiles * split;
}

extern "C" int64_t gq_build_descs(int n_shards, const int32_t *types, const int64_t *n_outs, int64_t K, int split, int32_t *desc_host) {
    if (n_shards <= 0 || !types || !n_outs || !desc_host) return GQ_ERR_ARG;
    if (K <= 0 || K % GQ_QK) return GQ_ERR_SHAPE;
    const int64_t nb = K / GQ_QK;
    if (split < 1 || split > nb) return GQ_ERR_ARG;
    int64_t base = 0, col0 = 0, row = 0;
    for (int i = 0; i < n_shards; ++i) {
        const int B = gq_type_bytes(types[i]);
        if (!B) return GQ_ERR_TYPE;
        if (n_outs[i] < 0) return GQ_ERR_SHAPE;
        const int64_t n_tiles = (n_outs[i] + 63) / 64, tile_kb_bytes = 64 * (int64_t)B;
        for (int64_t ti = 0; ti < n_tiles; ++ti)
            for (int s = 0; s < split; ++s) {
                const int64_t o = base + ti * nb * tile_kb_bytes;
                if ((o >> 4) > 0x7fffffff || col0 + ti * 64 > 0x7fffffff) return GQ_ERR_LIMIT;
                int32_t *r = desc_host + row * GQ_DESC_WORDS;
                r[0] = (int32_t)(o >> 4);
                r[1] = types[i];
                r[2] = (int32_t)(col0 + ti * 64);
                r[3] = (int32_t)(n_outs[i] - ti * 64 < 64 ? n_outs[i] - ti * 64 : 64);
                r[4] = (int32_t)((s * nb) / split);
                r[5] = (int32_t)(((s + 1) * nb) / split);
                r[6] = s;
                r[7] = 0;
                ++row;
            }
        base += n_tiles * nb * tile_kb_bytes;
        col0 += n_outs[i];
    }
    return row;
}

extern "C" int gq_split_for(int64_t n_tiles, int64_t nb, int64_t M, int avg_bytes_per_256, int sm_count) {
    (void)M; (void)avg_bytes_per_256;
    if (n_tiles <= 0 || nb <= 0) return 1;
    if (sm_count <= 0) sm_count = 148;
    // from sweeps on B200 (Q4_K / Q2_K / IQ3_S / IQ4_XS; 80-, 112-, 272- and 544-tile layers at K 5120 and 17408): the
    // largest split that (a) leaves a CTA at least three k-blocks, (b) stays inside one thread-block cluster (8), and
    // (c) keeps the launch in one wave of four CTAs per SM — counting that clusters cannot use every slot: a launch
    // of clusters of S fills at most about 1 - 0.03 (S - 1) of them before a second wave starts
    const int64_t slots = 4 * (int64_t)sm_count;
    int64_t s_max = nb / 3;
    if (s_max > 8) s_max = 8;
    int64_t s = 1;
    for (int64_t c = 2; c <= s_max; ++c)
        if (c * n_tiles * 100 <= slots * (100 - 3 * (c - 1))) s = c;
    if (s > nb) s = nb;
    return (int)s;
}

extern "C" int64_t gq_workspace_bytes(int64_t M, int64_t K, int64_t n_total, int split) {
    if (M < 0 || K <= 0 || K % GQ_QK || n_total < 0 || split < 1) return GQ_ERR_SHAPE;
    return ws_layout(M, K, n_total, split, nullptr, nullptr);
}

template <int MT, int MINB, int FORM, int ONLY>
static int launch_gemv(const GemvParams &p, int64_t n_desc, cudaStream_t stream) {
    constexpr int xbytes = gq_stage_xbytes<MT, FORM>();
    const int stage_bytes = p.wbytes_max + xbytes;
    const size_t smem = (size_t)p.stages * stage_bytes + (size_t)p.stages * 16 + (size_t)p.cb_bytes +
                        (size_t)GQ_CONSUMER_WARPS * MT * 512 * (p.cluster_push ? p.split - 1 : 1);
    if (smem > 232448) return GQ_ERR_LIMIT;
    // opt in once per device to the largest dynamic shared memory a CTA can have
    static std::atomic<unsigned long long> done_mask{0};
    int dev = 0;
    GQ_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !((done_mask.load() >> dev) & 1ull)) {
        GQ_CUDA(cudaFuncSetAttribute(gemv_grouped_kernel<MT, MINB, FORM, ONLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
        if (dev < 64) done_mask.fetch_or(1ull << dev);
    }
    {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[2];
        int na = 0;
        if (p.cluster) {
            attr[na].id = cudaLaunchAttributeClusterDimension;
            attr[na].val.clusterDim.x = (unsigned)p.split; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
            ++na;
        }
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
        cfg.gridDim = dim3((unsigned)n_desc); cfg.blockDim = dim3(32 * (GQ_CONSUMER_WARPS + 1)); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
        cfg.attrs = attr; cfg.numAttrs = na;
        GQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_grouped_kernel<MT, MINB, FORM, ONLY>, p));
    }
    GQ_LAUNCHED();
    return GQ_OK;
}

// integer form, M <= 8: one instantiation per type for runs of a single type, the all-types one otherwise
static int launch_gemv8_m8(const GemvParams &p, int64_t n_desc, cudaStream_t st, int only) {
    switch (only) {
#define GQ_ONE(T) case T: return launch_gemv<1, 4, 1, T>(p, n_desc, st);
        GQ_ONE(GQ_Q4_0) GQ_ONE(GQ_Q5_0) GQ_ONE(GQ_Q8_0) GQ_ONE(GQ_Q2_K) GQ_ONE(GQ_Q3_K) GQ_ONE(GQ_Q4_K)
        GQ_ONE(GQ_Q5_K) GQ_ONE(GQ_Q6_K) GQ_ONE(GQ_IQ4_NL) GQ_ONE(GQ_IQ3_S) GQ_ONE(GQ_IQ4_XS) GQ_ONE(GQ_IQ3_XXS) GQ_ONE(GQ_IQ2_XXS) GQ_ONE(GQ_IQ2_XS) GQ_ONE(GQ_IQ2_S) GQ_ONE(GQ_IQ1_M)
#undef GQ_ONE
        default: return launch_gemv<1, 4, 1, 0>(p, n_desc, st);
    }
}

extern "C" int gq_run_info(int n_shards, const int32_t *types) {
    if (n_shards <= 0 || !types) return GQ_ERR_ARG;
    int maxb = 0, cb = 0, single = types[0];
    for (int i = 0; i < n_shards; ++i) {
        const int B = gq_type_bytes(types[i]);
        if (!B) return GQ_ERR_TYPE;
        if (B > maxb) maxb = B;
        if (gq_cb_kind(types[i]) >= 0) cb |= 1 << gq_cb_kind(types[i]);     // a codebook type: the kernels keep its grid in shared memory
        if (types[i] != single) single = 0;
    }
    return maxb | ((cb ? 1 : 0) << 16) | (single << 17) | (cb << 22);
}

static int gemv_grouped_impl(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                             int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *workspace_dev,
                             int64_t workspace_bytes, void *stream, int phases, const void *next_packed_dev, int64_t next_bytes,
                             const ArFused *ar = nullptr, const PreOp *pre = nullptr) {
    if (M < 0 || M > GQ_MAX_GEMV_ROWS || K <= 0 || K % GQ_QK || n_total < 0 || n_desc < 0 || split < 1) return GQ_ERR_SHAPE;
    if (M == 0 || n_total == 0 || n_desc == 0) return GQ_OK;
    if (!x_dev || !packed_dev || !desc_dev || !y_dev || !workspace_dev) return GQ_ERR_ARG;
    if (((uintptr_t)packed_dev & 15) || ((uintptr_t)workspace_dev & 255) || ((uintptr_t)x_dev & 3) || ldx < K || ldy < n_total) return GQ_ERR_ARG;
    if (n_desc > 0x7fffffff) return GQ_ERR_LIMIT;
    Workspace ws;
    const int64_t need = ws_layout(M, K, n_total, split, workspace_dev, &ws);
    if (workspace_bytes < need) return GQ_ERR_WORKSPACE;
    if (int rc = ensure_tables()) return rc;
    cudaStream_t st = (cudaStream_t)stream;

    const int form = M <= GQ_GEMV8_MAX_ROWS ? 1 : 0;
    if (phases & 1) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.dynamicSmemBytes = 0; cfg.stream = st; cfg.attrs = attr; cfg.numAttrs = 1;
        if (form) {
            cfg.gridDim = dim3((unsigned)(K / GQ_QK), (unsigned)((M + GQ_PREP8_WARPS - 1) / GQ_PREP8_WARPS)); cfg.blockDim = dim3(32 * GQ_PREP8_WARPS);
            const PreOp po = pre ? *pre : PreOp{};
            if (po.kind == GQ_PRE_ADD_RMSNORM) {
                cfg.gridDim = dim3((unsigned)M, (unsigned)((K / GQ_QK + GQ_PREP8_WARPS - 1) / GQ_PREP8_WARPS));
                GQ_CUDA(cudaLaunchKernelEx(&cfg, prep_x8_norm_kernel, (const __nv_bfloat16 *)x_dev, ldx, (int)M, ws.xt, ws.status, po));
            } else {
                auto *kern = po.kind == GQ_PRE_SILU_MUL ? prep_x8_kernel<GQ_PRE_SILU_MUL> : prep_x8_kernel<GQ_PRE_NONE>;
                GQ_CUDA(cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16 *)x_dev, ldx, (int)M, ws.xt, ws.status, po));
            }
        } else {
            if (pre && pre->kind) return GQ_ERR_SHAPE;      // the folded ops exist in the integer form's preparation only
            cfg.gridDim = dim3((unsigned)M); cfg.blockDim = dim3(GQ_PREP_THREADS);
            GQ_CUDA(cudaLaunchKernelEx(&cfg, prep_x_kernel, (const __nv_bfloat16 *)x_dev, ldx, (int)K, (int)M, ws.ex, ws.xt, ws.status));
        }
        GQ_LAUNCHED();
    }
    if (!(phases & 6)) return GQ_OK;

    GemvParams p;
    p.packed = (const uint8_t *)packed_dev; p.desc = desc_dev; p.xt = ws.xt; p.ex = ws.ex;
    p.y = (__nv_bfloat16 *)y_dev; p.partials = ws.partials; p.status = ws.status;
    p.M = (int)M; p.K = (int)K; p.nb = (int)(K / GQ_QK); p.split = split; p.ldy = ldy; p.n_total = n_total;
    const int maxb = run_info & 0xFFFF;
    if (maxb < 56 || maxb > 272 || (maxb & 1)) return GQ_ERR_ARG;
    p.wbytes_max = 64 * maxb;   // every stage can hold a tile of any shard of the run
    p.cb_bytes = gq_cb_region_max((run_info >> 22) & 63, form);
    // split-K up to 8 reduces inside a thread-block cluster (portable cluster size); larger splits keep the fp32
    // partials and the separate sum
    p.cluster = (split > 1 && split <= 8 && n_desc % split == 0) ? 1 : 0;
    p.cluster_push = 0;
    p.pf_ptr = (next_packed_dev && next_bytes > 0 && !((uintptr_t)next_packed_dev & 15)) ? (const uint8_t *)next_packed_dev : nullptr;
    p.pf_bytes = next_bytes;
    if (ar) {
        if (split > 1 && !p.cluster) return GQ_ERR_ARG;        // the exchange needs the whole tile sum in one CTA
        if (n_desc / split * GQ_CONSUMER_WARPS > ar->units) return GQ_ERR_LIMIT;
        p.ar = *ar;
    } else {
        p.ar = ArFused{};
    }
    const int mt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
    {
        // ring depth: four stages when four CTAs of them still fit an SM's shared memory, else three (swept on the
        // 64-layer stack: deeper rings with fewer resident CTAs were slower overall)
        const int xb = !form ? 8 * mt * GQ_XROW_BYTES : mt == 1 ? gq_stage_xbytes<1, 1>() : mt == 2 ? gq_stage_xbytes<2, 1>() : gq_stage_xbytes<4, 1>();
        const int stage_bytes = p.wbytes_max + xb;
        // (an SM has 228 KB of shared memory and the system keeps 1 KB of it per resident CTA)
        const int fixed = 64 + p.cb_bytes + 1024, red1 = GQ_CONSUMER_WARPS * mt * 512;
        // split-K in a cluster: the push form of the reduction needs a scratch slot per other split in every CTA; it
        // is used when that costs no resident CTA (the ring then has three stages; its depth does not matter)
        if (p.cluster) {
            const int pull = (228 * 1024) / (3 * stage_bytes + fixed + red1), push = (228 * 1024) / (3 * stage_bytes + fixed + red1 * (split - 1));
            const int cap = mt == 1 ? 4 : 8;     // resident CTAs the register budget allows anyway
            p.cluster_push = (push > cap ? cap : push) >= (pull > cap ? cap : pull) ? 1 : 0;
        }
        const int red = p.cluster_push ? red1 * (split - 1) : red1;
        p.stages = (4 * (4 * stage_bytes + fixed + red) <= 228 * 1024) ? 4 : 3;
    }
    int rc = GQ_OK;
    if (phases & 2) {
        switch (mt) {
            case 1: rc = launch_gemv8_m8(p, n_desc, st, (run_info >> 17) & 31); break;
            case 2: rc = launch_gemv<2, 3, 1, 0>(p, n_desc, st); break;
            case 4: rc = form ? launch_gemv<4, 2, 1, 0>(p, n_desc, st) : launch_gemv<4, 2, 0, 0>(p, n_desc, st); break;
            default: rc = launch_gemv<8, 0, 0, 0>(p, n_desc, st); break;
        }
    }
    if (rc) return rc;
    if (split > 1 && !p.cluster && (phases & 4)) {
        const int64_t n = M * n_total;
        sum_partials_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ws.partials, split, M, n_total, (__nv_bfloat16 *)y_dev, ldy);
        GQ_LAUNCHED();
    }
    return GQ_OK;
}

extern "C" int gq_gemv_grouped_phases(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                                      int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                                      void *workspace_dev, int64_t workspace_bytes, void *stream, int phases) {
    return gemv_grouped_impl(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, workspace_dev,
                             workspace_bytes, stream, phases, nullptr, 0);
}

extern "C" int gq_gemv_grouped_prefetch(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                                        int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                                        void *workspace_dev, int64_t workspace_bytes, void *stream, const void *next_packed_dev,
                                        int64_t next_bytes) {
    return gemv_grouped_impl(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, workspace_dev,
                             workspace_bytes, stream, 7, next_packed_dev, next_bytes);
}

extern "C" int gq_gemv_grouped(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                               int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *workspace_dev,
                               int64_t workspace_bytes, void *stream) {
    return gq_gemv_grouped_phases(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, workspace_dev,
                                  workspace_bytes, stream, 7);
}

// ---- the same call with the op in front of the layer folded into the activation preparation -----------------
// pre_op GQ_PRE_SILU_MUL: x_dev is the [M, 2K] output of gate_up_proj (ldx >= 2K), the layer multiplies
// silu(x[:, :K]) * x[:, K:].  GQ_PRE_ADD_RMSNORM: x_dev is [M, K]; norm_weight [K]; residual_in / residual_out [M, ld_res]
// both or neither (distinct memory: every warp of a row reads the whole old residual).  1..GQ_GEMV8_MAX_ROWS rows.
extern "C" int gq_gemv_grouped_pre(const void *x_dev, int64_t M, int64_t K, int64_t ldx, int pre_op, const void *norm_weight_dev,
                                   const void *residual_in_dev, void *residual_out_dev, int64_t ld_res, float eps, const void *packed_dev,
                                   const int32_t *desc_dev, int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy,
                                   int64_t n_total, void *workspace_dev, int64_t workspace_bytes, void *stream) {
    if (M < 0 || M > GQ_GEMV8_MAX_ROWS) return GQ_ERR_SHAPE;
    PreOp po{};
    po.kind = pre_op; po.K = (int)K; po.eps = eps;
    if (pre_op == GQ_PRE_SILU_MUL) {
        if (ldx < 2 * K) return GQ_ERR_ARG;
    } else if (pre_op == GQ_PRE_ADD_RMSNORM) {
        if (!norm_weight_dev || ((uintptr_t)norm_weight_dev & 1)) return GQ_ERR_ARG;
        if ((residual_in_dev == nullptr) != (residual_out_dev == nullptr)) return GQ_ERR_ARG;
        if (residual_in_dev && (residual_in_dev == residual_out_dev || ld_res < K)) return GQ_ERR_ARG;
        po.weight = (const __nv_bfloat16 *)norm_weight_dev;
        po.residual = (const __nv_bfloat16 *)residual_in_dev; po.residual_out = (__nv_bfloat16 *)residual_out_dev; po.ld_res = ld_res;
    } else if (pre_op != GQ_PRE_NONE) {
        return GQ_ERR_ARG;
    }
    return gemv_grouped_impl(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, workspace_dev,
                             workspace_bytes, stream, 7, nullptr, 0, nullptr, &po);
}

// ---- the same call for callers that cannot allocate device memory -------------------------------------
// Scratch lives in this fixed array, part of the library's device image: every GPU that loads the library
// holds it until the process exits.  All calls of gq_gemv_grouped_static on a device share it.
#define GQ_STATIC_WS_BYTES (8ll << 20)
static __device__ __align__(256) unsigned char g_static_ws[GQ_STATIC_WS_BYTES];

extern "C" int64_t gq_static_workspace_limit(void) { return GQ_STATIC_WS_BYTES; }

extern "C" int gq_gemv_grouped_static(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                                      int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *stream) {
    if (M < 0 || M > GQ_MAX_GEMV_ROWS || K <= 0 || K % GQ_QK || n_total < 0 || n_desc < 0 || split < 1) return GQ_ERR_SHAPE;
    const int64_t need = ws_layout(M, K, n_total, split, nullptr, nullptr);
    if (need > GQ_STATIC_WS_BYTES) {
        snprintf(g_cuda_err, sizeof g_cuda_err, "gq_gemv_grouped_static: this call needs %lld bytes of scratch, the built-in buffer holds %lld",
                 (long long)need, (long long)GQ_STATIC_WS_BYTES);
        return GQ_ERR_LIMIT;
    }
    // In host code `g_static_ws` is only a handle for the symbol; the address the kernels may use is looked up
    // once per device, with that device current.
    static void *dev_ptr[64] = {nullptr};
    int dev = 0;
    GQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return GQ_ERR_LIMIT;
    void *ws = dev_ptr[dev];
    if (!ws) {
        GQ_CUDA(cudaGetSymbolAddress(&ws, g_static_ws));
        if (!ws) return GQ_ERR_CUDA;
        dev_ptr[dev] = ws;
    }
    return gq_gemv_grouped_phases(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, ws,
                                  GQ_STATIC_WS_BYTES, stream, 7);
}

// ---- the same call fused with the all-reduce of a row-parallel layer ---------------------------------------
// Every rank multiplies its K shard; the kernel's epilogue exchanges the bf16 partial outputs through peer memory
// and leaves the sum over ranks in y on every rank (fused_allreduce_tile).  Same arithmetic as the grouped call
// followed by gq_allreduce_push, without the second launch and its latency.
static int64_t fused_ar_units(int64_t max_n_total) { return (max_n_total / 64 + 64) * GQ_CONSUMER_WARPS; }
static int64_t fused_ar_header(int64_t max_n_total) { return (4 * fused_ar_units(max_n_total) + 4095) & ~(int64_t)4095; }

extern "C" int64_t gq_fused_allreduce_buffer_bytes(int world, int64_t max_m, int64_t max_n_total) {
    if (world < 1 || world > GQ_AR_MAX_WORLD || max_m < 1 || max_m > GQ_MAX_GEMV_ROWS || max_n_total < 1) return GQ_ERR_ARG;
    return fused_ar_header(max_n_total) + 2 * (int64_t)world * align256(max_m * max_n_total * 4);
}

static int gemv_grouped_allreduce_impl(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                                       int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                                       void *workspace_dev, int64_t workspace_bytes, int rank, int world, const uint64_t *peer_buffers,
                                       int64_t max_m, int64_t max_n_total, void *stream, const PreOp *pre) {
    if (world < 1 || world > GQ_AR_MAX_WORLD || rank < 0 || rank >= world || !peer_buffers) return GQ_ERR_ARG;
    if (max_m < 1 || max_m > GQ_MAX_GEMV_ROWS || M > max_m || n_total > max_n_total) return GQ_ERR_SHAPE;
    ArFused ar = {};
    ar.world = world; ar.rank = rank; ar.units = (int)fused_ar_units(max_n_total);
    ar.wait_ns = g_peer_wait_ns.load();
    if (n_total & 1) return GQ_ERR_SHAPE;
    if (world > 1 && M > 0 && n_total > 0 && n_desc > 0) {
        // a buffer serves one output width: the words' positions depend on n_total while the call numbers are kept per
        // (tile, warp), so a second width on the same buffer could meet a stale word that carries a current number
        static std::mutex mu;
        static std::unordered_map<uint64_t, int64_t> bound;
        std::lock_guard<std::mutex> lock(mu);
        auto it = bound.find(peer_buffers[rank]);
        if (it == bound.end()) bound.emplace(peer_buffers[rank], n_total);
        else if (it->second != n_total) {
            snprintf(g_cuda_err, sizeof g_cuda_err, "gq_gemv_grouped_allreduce: this buffer exchanges outputs of %lld columns, the call has %lld",
                     (long long)it->second, (long long)n_total);
            return GQ_ERR_ARG;
        }
    }
    ar.slot_bytes = align256(max_m * max_n_total * 4);
    const int64_t header = fused_ar_header(max_n_total);
    for (int p = 0; p < world; ++p) {
        if (!peer_buffers[p] || (peer_buffers[p] & 255)) return GQ_ERR_ARG;
        uint8_t *b = reinterpret_cast<uint8_t *>(peer_buffers[p]);
        ar.buf[p] = b + header;
    }
    ar.counters = reinterpret_cast<uint32_t *>(peer_buffers[rank]);
    return gemv_grouped_impl(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, workspace_dev,
                             workspace_bytes, stream, 7, nullptr, 0, &ar, pre);
}

extern "C" int gq_gemv_grouped_allreduce(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                                         int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                                         void *workspace_dev, int64_t workspace_bytes, int rank, int world, const uint64_t *peer_buffers,
                                         int64_t max_m, int64_t max_n_total, void *stream) {
    return gemv_grouped_allreduce_impl(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, workspace_dev,
                                       workspace_bytes, rank, world, peer_buffers, max_m, max_n_total, stream, nullptr);
}

// the fused multiply + all-reduce of a row-parallel down_proj with silu_and_mul folded into its activation preparation:
// x_dev is this rank's [M, 2K] slice pair (gate | up of its K columns, ldx >= 2K), 1..GQ_GEMV8_MAX_ROWS rows
extern "C" int gq_gemv_grouped_allreduce_silu_mul(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev,
                                                  const int32_t *desc_dev, int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy,
                                                  int64_t n_total, void *workspace_dev, int64_t workspace_bytes, int rank, int world,
                                                  const uint64_t *peer_buffers, int64_t max_m, int64_t max_n_total, void *stream) {
    if (M < 0 || M > GQ_GEMV8_MAX_ROWS) return GQ_ERR_SHAPE;
    if (ldx < 2 * K) return GQ_ERR_ARG;
    PreOp po{};
    po.kind = GQ_PRE_SILU_MUL; po.K = (int)K;
    return gemv_grouped_allreduce_impl(x_dev, M, K, ldx, packed_dev, desc_dev, n_desc, split, run_info, y_dev, ldy, n_total, workspace_dev,
                                       workspace_bytes, rank, world, peer_buffers, max_m, max_n_total, stream, &po);
}

// ---- small-message all-reduce over peer memory (tensor-parallel row-parallel layers) ---------------------
// One-shot, push based: every rank stores its bf16 vector into its slot of every peer's buffer (plain stores
// over NVLink into memory the peers mapped for each other), publishes a per-CTA flag, waits — with a limit —
// for the peers' flags, and sums the slots from its OWN memory in rank order (deterministic, fp32, one bf16
// rounding).  No loads from remote memory, no multicast.  Two slot sets alternate by call parity; the call
// number lives in device memory (one counter per CTA) so a captured CUDA graph replays correctly.
// The reference has no collective of its own on this path (docs/multi-gpu.md:8-13 leaves it to vLLM's NCCL).
#define GQ_AR_CTAS 32

struct ArPeers {
    uint8_t *buf[GQ_AR_MAX_WORLD];      // data area of each rank's buffer: [2 sets][world][slot_bytes]
    uint32_t *flags[GQ_AR_MAX_WORLD];   // flag area of each rank's buffer: [2 sets][world][GQ_AR_CTAS]
};

__global__ void __launch_bounds__(256) allreduce_push_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, int64_t n_vec, int rank,
                                                             int world, ArPeers peers, int64_t slot_bytes, uint32_t *counters, int *status,
                                                             unsigned long long wait_ns) {
    __shared__ uint32_t s_seq;
    __shared__ int s_fail;
    const int c = blockIdx.x, G = gridDim.x;
    if (threadIdx.x == 0) { s_seq = counters[c] + 1; s_fail = 0; }
    __syncthreads();
    const uint32_t seq = s_seq, set = seq & 1u;
    const int64_t per = (n_vec + G - 1) / G, v0 = (int64_t)c * per, v1 = v0 + per < n_vec ? v0 + per : n_vec;
    // push this CTA's share of the vector into slot `rank` of every rank's buffer (own included)
    for (int p = 0; p < world; ++p) {
        uint4 *dst = reinterpret_cast<uint4 *>(peers.buf[p] + ((int64_t)set * world + rank) * slot_bytes);
        for (int64_t i = v0 + threadIdx.x; i < v1; i += 256) dst[i] = in[i];
    }
    __syncthreads();
    if ((int)threadIdx.x < world) {
        // release at system scope: the stores of this CTA (ordered before by the barrier) are visible to the peer
        // before the flag is; the matching acquire load on the peer's side orders its reads of the slot after it
        uint32_t *f = peers.flags[threadIdx.x] + ((int64_t)set * world + rank) * G + c;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
        const uint32_t *mine = peers.flags[rank] + ((int64_t)set * world + threadIdx.x) * G + c;
        uint32_t v;
        uint64_t t0 = 0;
        for (uint32_t it = 0;; ++it) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v == seq) break;
            if ((it & 255u) == 255u) {      // the clock is read only once a wait has become long
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > wait_ns || it > GQ_SPIN_LIMIT) { s_fail = 1; break; }
            }
        }
    }
    __syncthreads();
    if (s_fail) {
        if (threadIdx.x == 0) { report_status(status, GQ_DEV_TIMEOUT); counters[c] = seq; }
        return;
    }
    const uint8_t *base = peers.buf[rank] + (int64_t)set * world * slot_bytes;
    for (int64_t i = v0 + threadIdx.x; i < v1; i += 256) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // all ranks' vectors are requested before any is added (one trip to the L2 instead of one per rank)
        uint4 v[GQ_AR_MAX_WORLD];
#pragma unroll
        for (int r = 0; r < GQ_AR_MAX_WORLD; ++r)
            if (r < world) v[r] = __ldcg(reinterpret_cast<const uint4 *>(base + (int64_t)r * slot_bytes) + i);
#pragma unroll
        for (int r = 0; r < GQ_AR_MAX_WORLD; ++r) {
            if (r < world) {
                const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&v[r]);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(b[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
            }
        }
        uint4 o;
        __nv_bfloat162 *ob = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        out[i] = o;
    }
    if (threadIdx.x == 0) counters[c] = seq;
}

extern "C" int64_t gq_allreduce_buffer_bytes(int world, int64_t max_bytes) {
    if (world < 1 || world > GQ_AR_MAX_WORLD || max_bytes <= 0) return GQ_ERR_ARG;
    const int64_t slot = align256(max_bytes);
    // [flags 2*world*CTAS u32 | counters CTAS u32 | status] padded to 4096, then data 2 * world * slot
    return 4096 + 2 * (int64_t)world * slot;
}

extern "C" int gq_allreduce_push(const void *in_dev, void *out_dev, int64_t n_bytes, int rank, int world, const uint64_t *peer_buffers,
                                 int64_t max_bytes, void *stream) {
    if (world < 1 || world > GQ_AR_MAX_WORLD || rank < 0 || rank >= world) return GQ_ERR_ARG;
    if (n_bytes < 0 || n_bytes > max_bytes || (n_bytes & 15)) return GQ_ERR_SHAPE;
    if (n_bytes == 0) return GQ_OK;
    if (!in_dev || !out_dev || !peer_buffers || ((uintptr_t)in_dev & 15) || ((uintptr_t)out_dev & 15)) return GQ_ERR_ARG;
    ArPeers peers;
    for (int p = 0; p < GQ_AR_MAX_WORLD; ++p) { peers.buf[p] = nullptr; peers.flags[p] = nullptr; }
    for (int p = 0; p < world; ++p) {
        if (!peer_buffers[p] || (peer_buffers[p] & 255)) return GQ_ERR_ARG;
        peers.flags[p] = reinterpret_cast<uint32_t *>(peer_buffers[p]);
        peers.buf[p] = reinterpret_cast<uint8_t *>(peer_buffers[p]) + 4096;
    }
    uint8_t *own = reinterpret_cast<uint8_t *>(peer_buffers[rank]);
    uint32_t *counters = reinterpret_cast<uint32_t *>(own + 2 * GQ_AR_MAX_WORLD * GQ_AR_CTAS * 4);
    int *status = reinterpret_cast<int *>(own + 2 * GQ_AR_MAX_WORLD * GQ_AR_CTAS * 4 + GQ_AR_CTAS * 4);
    allreduce_push_kernel<<<GQ_AR_CTAS, 256, 0, (cudaStream_t)stream>>>((const uint4 *)in_dev, (uint4 *)out_dev, n_bytes / 16, rank, world, peers,
                                                                     align256(max_bytes), counters, status, g_peer_wait_ns.load());
    GQ_LAUNCHED();
    return GQ_OK;
}

// ---- prefill ----------------------------------------------------------------------------------------
static int prefill_nb(int64_t M) { return M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// Split-K of a prefill launch: one CTA per (pair of 64-row tiles, NB batch rows) is resident per SM, so a launch of
// few CTAs (o / down / qkv at a few hundred rows) leaves SMs idle; its k-blocks are then cut into S balanced parts
// (grid.z), S chosen to minimise waves x (k-blocks per CTA + a fixed cost per wave).  Larger launches keep S = 1.
static int prefill_split(int64_t n_desc, int64_t M, int64_t nb, int nbt, int sms) {
    const int64_t ctas = ((n_desc + 1) / 2) * ((M + nbt - 1) / nbt);
    if (sms <= 0) sms = 148;
    if (nbt <= 64) sms *= 2;       // the 64-row variant is built for two CTAs per SM
    int best = 1;
    double best_cost = 1e300;
    // the fp32 partials cost a write and a read of S x M x n_total x 4 bytes: worth it only while a launch fills less than
    // half of the GPU (measured: down at 512 rows, 80 CTAs on 148 SMs, gains nothing from a split; at 64 rows it halves)
    if (ctas * 2 > sms) return 1;
    for (int S = 1; S <= 8 && (int64_t)S * 4 <= nb; ++S) {
        const int64_t waves = (ctas * S + sms - 1) / sms;
        const double cost = (double)waves * ((double)nb / S + 6.0) + (S > 1 ? 2.0 : 0.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = S; }
    }
    return best;
}

static int device_sms() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cached[dev].load();
    if (v <= 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev].store(v);
    }
    return v;
}

static int64_t pf_ws_layout(int64_t M, int64_t K, int nbt, int split, int64_t n_total, void *base, int **status, float **ex, uint8_t **xp,
                            float **partials) {
    const int64_t mt = (M + nbt - 1) / nbt;
    int64_t off = 256;
    const int64_t o_ex = off; off = align256(off + M * 4);
    off = (off + 1023) & ~(int64_t)1023;
    const int64_t o_xp = off; off += mt * nbt * K * 2;
    const int64_t o_p = off; if (split > 1) off = align256(off + (int64_t)split * M * n_total * 4);
    if (base) { uint8_t *b = (uint8_t *)base; *status = (int *)b; *ex = (float *)(b + o_ex); *xp = b + o_xp; *partials = (float *)(b + o_p); }
    return off;
}

extern "C" int64_t gq_prefill_workspace_bytes(int64_t M, int64_t K, int64_t n_total, int64_t n_desc) {
    if (M < 0 || K <= 0 || K % GQ_QK || n_total < 0 || n_desc < 0) return GQ_ERR_SHAPE;
    const int nbt = prefill_nb(M);
    return pf_ws_layout(M, K, nbt, prefill_split(n_desc, M, K / GQ_QK, nbt, device_sms()), n_total, nullptr, nullptr, nullptr, nullptr, nullptr);
}

template <int NB>
static int launch_prefill(PrefillParams &p, const __nv_bfloat16 *x, int64_t ldx, float *ex, uint8_t *xp, cudaStream_t st) {
    const int mt = (p.M + NB - 1) / NB;
    const size_t smem_base = 1024 + (size_t)GQ_PF_STAGES * (GQ_PF_A_BYTES + NB * 128) + 128;
    // the tables of the run's codebook types sit side by side; the opt-in covers every combination that fits a CTA at all
    const size_t smem = smem_base + (size_t)gq_cb_region_sum(p.cb_mask);
    const size_t smem_all = smem_base + (size_t)gq_cb_region_sum(63), smem_max = smem_all < 232448 ? smem_all : 232448;
    if (smem > smem_max) return GQ_ERR_LIMIT;
    static std::atomic<unsigned long long> done_mask{0};
    int dev = 0;
    GQ_CUDA(cudaGetDevice(&dev));
    if (dev >= 64 || !((done_mask.load() >> dev) & 1ull)) {
        GQ_CUDA(cudaFuncSetAttribute(gemm_prefill_kernel<NB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        GQ_CUDA(cudaFuncSetAttribute(gemm_prefill_kernel<NB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
        if (dev < 64) done_mask.fetch_or(1ull << dev);
    }
    prep_x_prefill_kernel<NB><<<(unsigned)(mt * NB), 256, 0, st>>>(x, ldx, p.K, p.M, ex, xp, p.status);
    GQ_LAUNCHED();
    if (p.split > 1) gemm_prefill_kernel<NB, true><<<dim3((unsigned)((p.n_desc + 1) / 2), (unsigned)mt, (unsigned)p.split), GQ_PF_THREADS, smem, st>>>(p);
    else gemm_prefill_kernel<NB, false><<<dim3((unsigned)((p.n_desc + 1) / 2), (unsigned)mt), GQ_PF_THREADS, smem, st>>>(p);
    GQ_LAUNCHED();
    if (p.split > 1) {
        const int64_t n = (int64_t)p.M * p.n_total;
        sum_partials_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(p.partials, p.split, p.M, p.n_total, p.y, p.ldy);
        GQ_LAUNCHED();
    }
    return GQ_OK;
}

extern "C" int gq_gemm_prefill(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                               int64_t n_desc, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *workspace_dev,
                               int64_t workspace_bytes, void *stream) {
    if (M < 0 || K <= 0 || K % GQ_QK || n_total < 0 || n_desc < 0) return GQ_ERR_SHAPE;
    if (M == 0 || n_total == 0 || n_desc == 0) return GQ_OK;
    if (!x_dev || !packed_dev || !desc_dev || !y_dev || !workspace_dev) return GQ_ERR_ARG;
    if (((uintptr_t)packed_dev & 15) || ((uintptr_t)workspace_dev & 1023) || ((uintptr_t)x_dev & 15) || (ldx & 7) || ldx < K || ldy < n_total)
        return GQ_ERR_ARG;
    if (n_desc > 0x7ffffffe || M > (int64_t)65535 * 64) return GQ_ERR_LIMIT;
    const int maxb = run_info & 0xFFFF;
    if (maxb < 56 || maxb > 272 || (maxb & 1)) return GQ_ERR_ARG;
    const int nbt = prefill_nb(M);
    const int split = prefill_split(n_desc, M, K / GQ_QK, nbt, device_sms());
    int *status; float *ex; uint8_t *xp; float *partials;
    const int64_t need = pf_ws_layout(M, K, nbt, split, n_total, workspace_dev, &status, &ex, &xp, &partials);
    if (workspace_bytes < need) return GQ_ERR_WORKSPACE;
    if (int rc = ensure_tables()) return rc;
    PrefillParams p;
    p.packed = (const uint8_t *)packed_dev; p.desc = desc_dev; p.n_desc = (int)n_desc; p.xp = xp; p.ex = ex;
    p.y = (__nv_bfloat16 *)y_dev; p.ldy = ldy; p.M = (int)M; p.K = (int)K; p.nb = (int)(K / GQ_QK); p.status = status;
    p.split = split; p.partials = partials; p.n_total = n_total; p.cb_mask = (run_info >> 22) & 63;
    cudaStream_t st = (cudaStream_t)stream;
    switch (nbt) {
        case 64: return launch_prefill<64>(p, (const __nv_bfloat16 *)x_dev, ldx, ex, xp, st);
        case 128: return launch_prefill<128>(p, (const __nv_bfloat16 *)x_dev, ldx, ex, xp, st);
        default: return launch_prefill<256>(p, (const __nv_bfloat16 *)x_dev, ldx, ex, xp, st);
    }
}

extern "C" int gq_device_status(int clear, void *stream) {
    int v = 0;
    GQ_CUDA(cudaMemcpyFromSymbolAsync(&v, g_sticky_status, sizeof v, 0, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    GQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (clear && v != 0) {
        const int zero = 0;
        GQ_CUDA(cudaMemcpyToSymbolAsync(g_sticky_status, &zero, sizeof zero, 0, cudaMemcpyHostToDevice, (cudaStream_t)stream));
        GQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    }
    return v;
}

extern "C" int gq_set_peer_wait_limit_ns(int64_t ns) {
    if (ns < 1000 || ns > 60000000000ll) return GQ_ERR_ARG;
    g_peer_wait_ns.store((unsigned long long)ns);
    return GQ_OK;
}

extern "C" int gq_read_status(const void *workspace_dev, int64_t workspace_bytes, void *stream) {
    if (!workspace_dev || workspace_bytes < 256) return GQ_ERR_ARG;
    int v = 0;
    GQ_CUDA(cudaMemcpyAsync(&v, workspace_dev, sizeof v, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    GQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return v;
}
