/*
 * gq_b200 — C ABI of the B200 (sm_100a) GGUF quantized-linear path.
 *
 * Drop-in boundary for the GGUF LinearMethod of the reference's vLLM plugin: everything the plugin's
 * load step (process_weights_after_loading) and per-call step (apply) hand to a kernel goes through
 * these entry points.  The reference has no C ABI of its own for this path — its launcher is
 * Python/Triton (gguf-plugin/gluon/interface.py, gguf-plugin/gluon/tiles_grouped.py) — so each entry
 * point cites the reference function it replaces.
 *
 * Conventions
 *   - Every function returns an int status: 0 ok; < 0 the arguments were rejected on the host and
 *     nothing was launched (GQ_ERR_*); > 0 is only ever reported through gq_read_status / gq_device_status (a kernel hit a
 *     bounded wait's limit).  Nothing aborts, traps or spins without a limit.
 *   - Pointers named *_dev are device pointers owned by the caller; `stream` is a cudaStream_t passed
 *     as void*.  No entry point allocates or frees device memory, or synchronises, except where stated.
 *   - GGML type ids: Q4_0 2, Q5_0 6, Q8_0 8, Q2_K 10, Q3_K 11, Q4_K 12, Q5_K 13, Q6_K 14, IQ2_XXS 16, IQ2_XS 17,
 *     IQ3_XXS 18, IQ4_NL 20, IQ3_S 21, IQ2_S 22, IQ4_XS 23, IQ1_M 29.  K must be a multiple of 256.
 *   - Thread safety: re-entrant; one call at a time per workspace buffer.
 */
#ifndef GQ_B200_H
#define GQ_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GQ_ERR_TYPE (-1)        /* unsupported GGML type */
#define GQ_ERR_SHAPE (-2)       /* K not a multiple of 256, negative sizes, M over the entry point's limit */
#define GQ_ERR_ARG (-3)         /* null pointer, misaligned pointer, inconsistent descriptor */
#define GQ_ERR_WORKSPACE (-4)   /* workspace too small */
#define GQ_ERR_CUDA (-5)        /* a CUDA runtime call failed; see gq_last_cuda_error */
#define GQ_ERR_LIMIT (-6)       /* size beyond a documented fixed maximum */

#define GQ_DESC_WORDS 8         /* int32 words per descriptor row */
#define GQ_MAX_GEMV_ROWS 64     /* largest batch gq_gemv_grouped accepts */

/* ---- format facts (host) ---------------------------------------------------------------------- */

/* Bytes of one row's 256-weight segment of raw GGUF blocks; 0 for an unsupported type.
 * Reference: gguf-plugin/gluon/tiles.py:24-36 (TILE_TYPES block sizes), kq_tiles.py:22, q2k.py:34. */
int gq_bytes_per_256(int type);

/* Bytes of the packed (tile-major) form of an [n_out, K] tensor: ceil(n_out/64) * (K/256) * 64 *
 * bytes_per_256.  < 0 on a bad argument.
 * Reference: the tile tensor shape [ceil(n/64), nb, 64, row_bytes] of gguf-plugin/gluon/tiles.py:128-130. */
int64_t gq_packed_bytes(int type, int64_t n_out, int64_t K);

/* The repack map of one 16-row slab: map[p] = row * bytes_per_256 + byte for packed byte p,
 * 0 <= p < 16 * bytes_per_256 (a permutation).  `map` has room for 16 * bytes_per_256 int32.
 * Reference: kq_tiles.tile_map (gguf-plugin/test_gguf_rco_cpu.py:255-266 checks its map the same way). */
int gq_slab_map(int type, int32_t *map);

/* ---- load time --------------------------------------------------------------------------------- */

/* Raw GGUF rows -> packed tiles.  raw_dev: uint8 [n_out, (K/256)*bytes_per_256], row stride
 * raw_row_stride bytes (>= the row's bytes; any alignment).  out_dev: gq_packed_bytes bytes, 16-byte
 * aligned.  Rows past n_out in the last tile are written as zeros.
 * Reference: repack_tiles (gguf-plugin/gluon/tiles.py:128-130) called from _create_tiles
 * (gguf-plugin/patches/gguf-tiles-all-types.patch:73-131). */
int gq_repack(int type, const void *raw_dev, int64_t n_out, int64_t K, int64_t raw_row_stride, void *out_dev, void *stream);

/* Packed tiles -> raw GGUF rows (bit-exact inverse of gq_repack).
 * Reference: unrepack_tiles (gguf-plugin/gluon/tiles.py:39-67, kq_tiles.py:100-125). */
int gq_unrepack(int type, const void *tiles_dev, int64_t n_out, int64_t K, void *raw_dev, int64_t raw_row_stride, void *stream);

/* Packed tiles -> dequantised weights [n_out, K], row stride ld elements.  out_dtype 0: fp32, every
 * value bit-identical to gguf.quants.dequantize; 1: bf16 (the fp32 value rounded to nearest even).
 * Reference: dequantize_tiles (gguf-plugin/gluon/tiles.py:141-149), dequantize_iq3s_tiles
 * (gguf-plugin/gluon/iq3s_tile_dequant.py:22-63). */
int gq_dequant(int type, const void *tiles_dev, int64_t n_out, int64_t K, void *out_dev, int out_dtype, int64_t ld, void *stream);

/* Descriptor table of a run of shards that share K and sit back to back in one packed buffer
 * (shard i's tiles start at byte offset sum_{j<i} gq_packed_bytes(j)).  One row of GQ_DESC_WORDS int32
 * per (64-row tile, k-range): {tile byte offset / 16, type, first output column, valid rows, kb0, kb1,
 * split index, 0}.  k-ranges are the balanced partition [(s*nb)/S, ((s+1)*nb)/S).  Host function;
 * desc_host has room for gq_desc_rows(...) rows.  Returns the number of rows written, or < 0.
 * Reference: descriptors / prepare_grouped_layer (gguf-plugin/gluon/tiles_grouped.py:253-299). */
int64_t gq_desc_rows(int n_shards, const int64_t *n_outs, int split);
int64_t gq_build_descs(int n_shards, const int32_t *types, const int64_t *n_outs, int64_t K, int split, int32_t *desc_host);

/* Split-K of a grouped launch: n_tiles output tiles, nb k-blocks, M batch rows, avg_bytes_per_256 of
 * the run, on a device with sm_count SMs.  Always in [1, nb] and at most 8 (the split then stays inside
 * one thread-block cluster); any other value in [1, nb] is also valid for the calls below.
 * Reference: grouped_split_for (gguf-plugin/gluon/tiles_grouped.py:209-250), re-derived for 148 SMs. */
int gq_split_for(int64_t n_tiles, int64_t nb, int64_t M, int avg_bytes_per_256, int sm_count);

/* Facts of a run the launchers size shared memory and pick a kernel by, packed in one int:
 *   bits 0..15   the largest bytes_per_256 of the run's types (a stage of the weight ring holds a tile of any shard)
 *   bit 16       the run holds a codebook type (IQ3_S, IQ3_XXS, IQ2_XXS, IQ2_XS, IQ2_S, IQ1_M)
 *   bits 17..21  the GGML type id when every shard has the same type (the per-type kernel serves it), else 0
 *   bits 22..27  which codebook types: IQ3_S, IQ3_XXS, IQ2_XXS, IQ2_XS, IQ2_S, IQ1_M in this order (their grid tables are
 *                staged in shared memory)
 * < 0 on an unsupported type.
 * Reference: meta["max_rw"] and the NEW mask (gguf-plugin/gluon/tiles_grouped.py:181-202,1239-1265). */
int gq_run_info(int n_shards, const int32_t *types);

/* ---- per call ---------------------------------------------------------------------------------- */

/* Workspace bytes a call with these sizes needs (activation staging, split-K partials, status). */
int64_t gq_workspace_bytes(int64_t M, int64_t K, int64_t n_total, int split);

/* Y[M, n_total] = X[M, K] . W^T for a run of packed shards, 1 <= M <= GQ_MAX_GEMV_ROWS.
 *   x_dev     bf16 [M, K], row stride ldx elements
 *   packed_dev, desc_dev, n_desc, split   the run's tiles and the descriptor table built for `split`
 *   run_info  gq_run_info of the run's types
 *   y_dev     bf16, row stride ldy elements; the run writes columns [0, n_total)
 *   workspace_dev  at least gq_workspace_bytes(M, K, n_total, split) bytes, 256-byte aligned
 * Launches: activation preparation and the grouped kernel; splits up to 8 are reduced inside the kernel
 * (one thread-block cluster per tile, fixed summation order), larger ones by a third launch that sums fp32
 * partials from the workspace.  M == 0 is a no-op.  Reference: gluon_mul_mat_tiles_grouped for M <= 32 and the bm-64 wide form
 * (gguf-plugin/gluon/interface.py:141-188), quantize_activations_256, grouped_gemm, sum_partials
 * (gguf-plugin/gluon/tiles_grouped.py:110-162,1204-1275). */
int gq_gemv_grouped(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                    int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *workspace_dev,
                    int64_t workspace_bytes, void *stream);

/* The same call with its launches selectable: phases bit 0 = activation preparation (x -> workspace),
 * bit 1 = the grouped kernel, bit 2 = the split-K partial sum.  gq_gemv_grouped is phases = 7.  A caller
 * that multiplies the same x by several runs prepares once and passes phases = 6 for the others, with the
 * same workspace (its activation area depends only on M and K); a benchmark times bit 1 alone.
 * Reference: interface.py:164,174 quantises once per layer call for the same reason. */
int gq_gemv_grouped_phases(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                           int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                           void *workspace_dev, int64_t workspace_bytes, void *stream, int phases);

/* gq_gemv_grouped plus a hint: next_packed_dev / next_bytes name the packed weights the caller will multiply
 * next (the following layer).  While this launch computes, idle lanes of its copy warps ask the L2 (126 MB on
 * B200) to fetch them, so the next launch starts on L2 hits instead of a cold DRAM burst.  A null pointer or
 * zero bytes means no hint; the result is the same either way.
 * Reference: none — the reference's launches start cold; its Ada card's L2 (64 MB) is smaller than a layer. */
int gq_gemv_grouped_prefetch(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                             int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                             void *workspace_dev, int64_t workspace_bytes, void *stream, const void *next_packed_dev,
                             int64_t next_bytes);

/* gq_gemv_grouped of pre(x), the op in front of the layer folded into the activation preparation (1..16 rows):
 *   GQ_PRE_SILU_MUL     x_dev is the [M, 2K] output of gate_up_proj (ldx >= 2K); the layer multiplies
 *                       silu(x[:, :K]) * x[:, K:2K] — vLLM's silu_and_mul in front of down_proj;
 *   GQ_PRE_ADD_RMSNORM  x_dev is [M, K]; the layer multiplies RMSNorm(x + residual_in) * norm_weight and
 *                       residual_out receives x + residual_in — vLLM's fused_add_rms_norm in front of qkv_proj and
 *                       gate_up_proj.  residual_in and residual_out (bf16 [M, ld_res]) are both given or both null
 *                       (plain RMSNorm) and never the same memory; norm_weight_dev is bf16 [K];
 *   GQ_PRE_NONE         gq_gemv_grouped.
 * Intermediate values are rounded to bf16 where the unfused kernels round, so the result is that of the unfused
 * sequence (the row's mean square is summed in another order: a last-bit difference of the normalised value can
 * appear).  More than 16 rows: GQ_ERR_SHAPE.
 * Reference: none — the reference serves the model with stock vLLM's separate kernels around its linear method
 * (gguf-tiles-all-types.patch:203-262 takes the finished activation). */
#define GQ_PRE_NONE 0
#define GQ_PRE_SILU_MUL 1
#define GQ_PRE_ADD_RMSNORM 2
int gq_gemv_grouped_pre(const void *x_dev, int64_t M, int64_t K, int64_t ldx, int pre_op, const void *norm_weight_dev,
                        const void *residual_in_dev, void *residual_out_dev, int64_t ld_res, float eps, const void *packed_dev,
                        const int32_t *desc_dev, int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                        void *workspace_dev, int64_t workspace_bytes, void *stream);

/* gq_gemv_grouped without a workspace argument, for callers that cannot allocate device memory at the
 * point of the call — a plugin op running where the framework's allocator is off limits (inside another
 * library's callback, under a fixed memory plan, or in a process that handed all of its device memory to a
 * pool it does not own).  It has no counterpart in the reference, whose launcher always allocates through
 * torch.  The scratch (prepared activations, split-K partials, the status word) lives in a fixed 8 MiB
 * buffer built into the library's device image; every GPU that loads the library holds those 8 MiB until the
 * process exits.  gq_static_workspace_limit() returns that size; a call whose gq_workspace_bytes(M, K,
 * n_total, split) exceeds it is rejected with GQ_ERR_LIMIT and a message in gq_last_cuda_error, nothing
 * launched.  The entry point calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on a device looks the buffer's address up (a host-side query); make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one buffer, and it keeps the previous call's contents.  The status word
 *     is cleared at the start of every call; nothing else needs a clean slate.  Two calls whose kernels overlap
 *     on the GPU (different streams, no ordering between them) race on the buffer: keep them on one stream
 *     or order them with events.
 * Arguments and results are those of gq_gemv_grouped. */
int64_t gq_static_workspace_limit(void);
int gq_gemv_grouped_static(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                           int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *stream);

/* Small-message all-reduce (sum, bf16) for the row-parallel layers under tensor parallelism, one process per
 * GPU.  Every rank owns a buffer of gq_allreduce_buffer_bytes(world, max_bytes) bytes that all ranks have
 * mapped (peer-accessible: e.g. torch.distributed._symmetric_memory), zeroed once before the first call;
 * peer_buffers[p] is rank p's buffer as seen from the calling process (host array of `world` addresses).
 * in_dev / out_dev: bf16, n_bytes a multiple of 16, at most max_bytes (the value the buffers were sized
 * with); out may alias in.  Every rank must make the same sequence of calls.  The kernel pushes its data
 * into the peers' buffers with plain stores, waits with a limit for the peers' flags (a timeout sets the
 * status word at byte 2*8*16*4 + 16*4 of the rank's own buffer) and sums from its own memory in rank order.
 * Reference: none — the reference leaves the collective to vLLM (docs/multi-gpu.md:8-13). */
int64_t gq_allreduce_buffer_bytes(int world, int64_t max_bytes);
int gq_allreduce_push(const void *in_dev, void *out_dev, int64_t n_bytes, int rank, int world, const uint64_t *peer_buffers,
                      int64_t max_bytes, void *stream);

/* gq_gemv_grouped fused with the all-reduce of a row-parallel layer: every rank passes its K shard of x and of
 * the weights; on return (in stream order) y holds the sum over ranks of the ranks' bf16 partial outputs, on
 * every rank.  The exchange happens in the kernel's epilogue, per 16 output columns: a warp stores its block into
 * its rank's slot of every rank's buffer (plain stores through peer pointers) as 8-byte words {two bf16 values,
 * call number}; the receiver polls the words of its own memory until they carry this call's number (with a time
 * limit: a timeout sets the workspace's status word to 1) and sums them in rank order — the arithmetic of
 * gq_gemv_grouped followed by gq_allreduce_push, without the second launch and without fences at system scope.
 * peer_buffers[p] is rank p's buffer of gq_fused_allreduce_buffer_bytes(world, max_m, max_n_total) bytes as seen
 * from this process (peer-mapped, 256-byte aligned, zeroed once before the first call); M <= max_m, n_total <=
 * max_n_total; n_total and every shard's n_out even (status word 2 otherwise); with more than one rank a buffer serves ONE n_total: the first
 * call fixes it and a call with another is rejected with GQ_ERR_ARG (word positions depend on the width while call
 * numbers are kept per 16-column unit, so a second width could take a stale word for a current one); split must be 1 or reduce inside
 * the kernel (<= 8); every rank makes the same sequence of calls on a buffer.  No loads from remote memory, no
 * multicast.  Reference: none — the reference has no collective on this path (docs/multi-gpu.md:8-13). */
int64_t gq_fused_allreduce_buffer_bytes(int world, int64_t max_m, int64_t max_n_total);
int gq_gemv_grouped_allreduce(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                              int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *workspace_dev,
                              int64_t workspace_bytes, int rank, int world, const uint64_t *peer_buffers, int64_t max_m,
                              int64_t max_n_total, void *stream);

/* gq_gemv_grouped_allreduce with silu_and_mul folded into the activation preparation (GQ_PRE_SILU_MUL of gq_gemv_grouped_pre): the
 * row-parallel down_proj of a tensor-parallel decoder block in one call.  x_dev is this rank's [M, 2K] input, gate in columns 0..K-1
 * and up in K..2K-1 of ITS K columns (ldx >= 2K); 1..16 rows.  Reference: none. */
int gq_gemv_grouped_allreduce_silu_mul(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                                       int64_t n_desc, int split, int run_info, void *y_dev, int64_t ldy, int64_t n_total,
                                       void *workspace_dev, int64_t workspace_bytes, int rank, int world, const uint64_t *peer_buffers,
                                       int64_t max_m, int64_t max_n_total, void *stream);

/* Workspace bytes of gq_gemm_prefill for a batch of M rows, a run of n_desc tiles and n_total output columns
 * (activations re-laid out for the tensor-core operand, row scales, status, and fp32 partial outputs when the call
 * will split K).  Depends on the current device's SM count. */
int64_t gq_prefill_workspace_bytes(int64_t M, int64_t K, int64_t n_total, int64_t n_desc);

/* Y[M, n_total] = X[M, K] . W^T for a run of packed shards at any M (meant for M > GQ_MAX_GEMV_ROWS): the
 * large-batch path.  desc_dev is the run's descriptor table built with split = 1 (one row per 64-row tile); run_info is
 * gq_run_info of the run's types (sizes the packed-tile ring in shared memory).
 * Each CTA streams two tiles' packed k-blocks through a shared-memory ring (bulk copies), dequantises them into a
 * second ring as fp16 and feeds tcgen05.mma with the fp32 accumulator in tensor memory; the dequantised weights never
 * reach HBM.  A launch too small to give every SM a CTA splits K over grid.z and a second launch adds the fp32 partial
 * outputs in split order.  workspace_dev: at least gq_prefill_workspace_bytes(M, K, n_total, n_desc) bytes, 1024-byte
 * aligned; x_dev 16-byte aligned with ldx a multiple of 8.
 * Reference: the wide forms (bm 64 / 128) and the dequantise + cuBLAS path of gluon_mul_mat_tiles_grouped
 * (gguf-plugin/gluon/interface.py:159-188), dequantize_tiles (gguf-plugin/gluon/tiles.py:141-149). */
int gq_gemm_prefill(const void *x_dev, int64_t M, int64_t K, int64_t ldx, const void *packed_dev, const int32_t *desc_dev,
                    int64_t n_desc, int run_info, void *y_dev, int64_t ldy, int64_t n_total, void *workspace_dev,
                    int64_t workspace_bytes, void *stream);

/* Reads the device status word of the last call on this workspace (synchronises the stream): 0, or
 * a positive GQ_DEV_* code (1: a bounded wait ran out; 2: a shape or a tile's type contradicts the call's arguments —
 * an odd column count in the fused all-reduce, a tile that is not of the single type run_info names, a codebook type run_info
 * does not announce; the CTA concerned computed nothing). */
int gq_read_status(const void *workspace_dev, int64_t workspace_bytes, void *stream);

/* The largest device status code any kernel of this library has reported on the current device since the word was
 * last cleared (synchronises the stream; clear != 0 resets it after reading): 0, or a positive GQ_DEV_* code.  Every
 * kernel that sets a workspace's status word sets this one too, so a caller that frees its workspace after each call,
 * or uses the entry point without a workspace argument, still sees a timeout.  Meant to be called between steps.
 * Reference: none (the reference's kernels have no waits that can run out). */
int gq_device_status(int clear, void *stream);

/* Time limit, in nanoseconds, of the waits for another GPU's data in gq_allreduce_push and
 * gq_gemv_grouped_allreduce (default 4 s; 1 us .. 60 s).  Applies to launches made after the call, process-wide.
 * A wait that runs out sets the status words and leaves y incomplete; the context stays usable.
 * Reference: none. */
int gq_set_peer_wait_limit_ns(int64_t ns);

/* Text of the last CUDA runtime error seen by this library in the calling thread ("" if none). */
const char *gq_last_cuda_error(void);

/* Number of kernels this library has launched in the calling process (for benchmark bookkeeping). */
int64_t gq_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* GQ_B200_H */
