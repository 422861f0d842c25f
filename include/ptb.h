/*
 * ptb.h -- C ABI of the B200 (sm_100a) FP8 quantize / GEMM / grouped-GEMM library.
 *
 * Every entry point takes raw device pointers, explicit sizes/strides and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t).  The caller allocates every output and workspace.  All
 * work is enqueued on the given stream; no call synchronises the host with the device (except
 * ptb_gemm_status and ptb_copy_segments_status, which read one word back).  Calls are re-entrant.
 * The library keeps no state between calls, with three stated exceptions:
 * (1) ptb_quant_fp8_rowwise_noalloc reduces into one fixed device array that all of its calls
 * share; (2) the GEMM kernels record a wait that ran out
 * in one device word per GPU, shared by all streams and read with ptb_gemm_status, and the peer
 * copies do the same for a bad rank number or a flag wait that ran out (ptb_copy_segments_status);
 * (3) per-device one-time set-up (kernel attributes, the address of that array) is cached in the
 * process.
 *
 * Alignment: FP8 outputs of the blockwise quantise entry points (block1d, block1d_dual, block2d,
 * segment_row_col) must be 8-byte aligned, GEMM operands 16-byte aligned with leading dimensions
 * that are multiples of 16 bytes (PTB_ERR_ALIGN otherwise).  The tensorwise / rowwise quantise
 * entry points accept any alignment and fall back to narrower accesses.
 *
 * Return value: 0 on success; a negative value for an argument error (PTB_ERR_*); a positive
 * value is a cudaError_t reported by the CUDA runtime or driver.  ptb_last_error() returns a
 * description of the last failure on the calling thread.
 *
 * Each declaration names the interface of the reference project (Primus-Turbo) it replaces,
 * as file:line inside that project.
 */
#ifndef PTB_H_
#define PTB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PTB_VERSION 100

typedef void *ptb_stream_t; /* cudaStream_t */

/* element types */
#define PTB_F32 0
#define PTB_F16 1
#define PTB_BF16 2
#define PTB_E4M3 3 /* float8_e4m3fn (OCP), max 448   */
#define PTB_E5M2 4 /* float8_e5m2   (OCP), max 57344 */

/* scaling granularity; values match ScalingGranularity in
 * primus_turbo/pytorch/core/low_precision.py:125-133 */
#define PTB_TENSORWISE 1
#define PTB_ROWWISE 2
#define PTB_BLOCKWISE 3

/* argument errors */
#define PTB_ERR_ARG (-1)         /* null pointer, negative size, unknown enum         */
#define PTB_ERR_UNSUPPORTED (-2) /* valid request outside what the kernels implement  */
#define PTB_ERR_ALIGN (-3)       /* pointer / leading dimension not 16-byte aligned   */
#define PTB_ERR_DRIVER (-4)      /* CUDA driver entry point unavailable               */
#define PTB_ERR_TOO_LARGE (-5)   /* size beyond a stated static limit                 */

int ptb_version(void);
const char *ptb_last_error(void);

/* ------------------------------------------------------------------ quantize ----------------- */

/* Bytes of workspace ptb_quant_fp8_tensorwise needs (one amax word, padded). */
#define PTB_TENSORWISE_WS_BYTES 256

/* Tensorwise: amax over all n elements, scale = fmax/max(amax,1e-12), scale_inv = 1/scale,
 * q = cast(clamp(x*scale)).  Writes q[n] and scale_inv[1].  workspace: PTB_TENSORWISE_WS_BYTES,
 * cleared by the call itself.
 * Replaces torch op quantize_fp8_tensorwise (csrc/pytorch/bindings_pytorch.cpp:31,
 * csrc/pytorch/quantization/quantization.cpp:42-88). */
int ptb_quant_fp8_tensorwise(const void *x, int x_dtype, int64_t n, void *q, int q_dtype,
                             float *scale_inv, void *workspace, ptb_stream_t stream);

/* Tensorwise with a caller-given scale (device scalar): scale_inv = 1/scale.
 * Replaces the scale_opt branch of quantize_fp8_tensorwise (quantization.cpp:53-56). */
int ptb_quant_fp8_tensorwise_with_scale(const void *x, int x_dtype, int64_t n, const float *scale,
                                        void *q, int q_dtype, float *scale_inv,
                                        ptb_stream_t stream);

/* Rowwise: x viewed as [B, M, N], one scale per (b, n) over the M axis; scale_inv is [B,1,N].
 * N == 1 is the "axis is the last dimension" case.  workspace: B*N floats (only read when
 * N > 1; cleared by the call).
 * Replaces torch op quantize_fp8_rowwise (bindings_pytorch.cpp:33, quantization.cpp:108-206). */
int ptb_quant_fp8_rowwise(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N, void *q,
                          int q_dtype, float *scale_inv, void *workspace, ptb_stream_t stream);

/* Rowwise quantize that allocates nothing and needs no workspace argument.
 * For hosts that are not allowed to obtain device memory on the library's behalf: an inference or
 * training runtime that hands a plugin only its input and output buffers and owns every other byte
 * of the device, or a service that forbids cudaMalloc after start-up because the call stalls the
 * whole device.  Same arithmetic and outputs as ptb_quant_fp8_rowwise; the column-amax scratch is a
 * fixed 256 KiB array inside the library, so B*N may not exceed 65536 (PTB_ERR_TOO_LARGE otherwise;
 * N == 1, the reduction over the innermost axis, uses no scratch and has no such limit).
 * The first call on each device looks the array's device address up (cudaGetSymbolAddress) and
 * should therefore be made before any stream capture starts.  All calls share the one array, which
 * keeps whatever the previous call left in it (each call clears the part it uses): two calls that
 * can overlap on the GPU, e.g. on different streams, race and must be ordered by the caller.
 * No counterpart in the reference. */
int ptb_quant_fp8_rowwise_noalloc(const void *x, int x_dtype, int64_t B, int64_t M, int64_t N,
                                  void *q, int q_dtype, float *scale_inv, ptb_stream_t stream);

/* 1-D blockwise (block = 128): axis 1 -> scale_inv [M, ceil(N/128)]; axis 0 -> [ceil(M/128), N].
 * Replaces primus_turbo::quant_fp8_blockwise_impl
 * (primus_turbo/pytorch/kernels/quantization/quantization_impl.py:74-118). */
int ptb_quant_fp8_block1d(const void *x, int x_dtype, int64_t M, int64_t N, int axis, void *q,
                          int q_dtype, float *scale_inv, ptb_stream_t stream);

/* Both 1-D blockwise copies from one read of x; both copies are [M,N] (not transposed).
 * Replaces primus_turbo::quant_fp8_blockwise_dual_impl (quantization_impl.py:229-274). */
int ptb_quant_fp8_block1d_dual(const void *x, int x_dtype, int64_t M, int64_t N, void *q_row,
                               float *s_row, void *q_col, float *s_col, int q_dtype,
                               ptb_stream_t stream);

/* 2-D blockwise (one scale per 128x128 tile) of w [B, M, N]; scale_inv [B, ceil(M/128),
 * ceil(N/128)].  Replaces torch op quantize_fp8_blockwise_for_weight
 * (bindings_pytorch.cpp:37, quantization.cpp:1442-1476). */
int ptb_quant_fp8_block2d(const void *w, int w_dtype, int64_t B, int64_t M, int64_t N, void *q,
                          int q_dtype, float *scale_inv, ptb_stream_t stream);

/* Grouped activation quantize, one read of x [M, N]:
 *   q_row [M, N], s_row [ceil(N/128), M] (row scales stored transposed);
 *   q_col_padded [M + 128*G, N]: group g occupies rows [var_k_offs[g], +len_g) followed by zero
 *   rows up to a multiple of 128; s_col_padded [ceil((M+128*G)/128), N] on group-relative
 *   128-row blocks; var_k_lens[G] = ceil(len/128)*128 and its exclusive prefix var_k_offs[G+1].
 * Rows at or beyond group_offs[G] (row outputs) / var_k_offs[G] (padded outputs) are not written.
 * block_table: optional workspace of ceil((M + 128*G) / 128) * 8 bytes (8-byte aligned), written by the
 * call: with it every tile finds its source rows with one load; NULL makes every tile scan the G
 * offsets instead (same results).
 * M == 0 (no row at all, e.g. an expert-parallel rank whose experts received nothing): x, q_row and s_row
 * may be NULL; var_k_lens / var_k_offs and the block table are still written (every group empty).
 * Replaces torch op quantize_fp8_blockwise_segment_m_row_col (bindings_pytorch.cpp:35,
 * quantization.cpp:1382-1439). */
int ptb_quant_fp8_segment_row_col(const void *x, int x_dtype, int64_t M, int64_t N, int64_t G,
                                  const int64_t *group_lens, const int64_t *group_offs,
                                  void *q_row, void *q_col_padded, float *s_row,
                                  float *s_col_padded, int64_t *var_k_lens, int64_t *var_k_offs,
                                  void *block_table, int q_dtype, ptb_stream_t stream);

/* SwiGLU with routing probabilities: out[t, j] = (u / (1 + exp(-u))) * x[t, H + j] * probs[t], u = x[t, j],
 * x [rows, 2H] bf16 / fp16, probs fp32 [rows], row_mask int64 [rows] or NULL (0: the row is written as zeros);
 * fp32 arithmetic, one rounding to dtype.  H % 8 == 0.
 * Replaces swiglu_fwd_with_probs (primus_turbo/pytorch/kernels/activation/swiglu_impl.py:20-57,
 * primus_turbo/triton/activation/swiglu_kernel.py:11-57,145-184). */
int ptb_swiglu_probs_fwd(const void *x, int dtype, const float *probs, const int64_t *row_mask,
                         int64_t rows, int64_t H, void *out, ptb_stream_t stream);

/* Backward of the above: grad_x [rows, 2H] and grad_probs [rows] = sum_j grad_out * silu(u) * x[t, H + j].
 * Replaces swiglu_bwd_with_probs (swiglu_impl.py:60-111, swiglu_kernel.py:60-142,187-248). */
int ptb_swiglu_probs_bwd(const void *grad_out, const void *x, int dtype, const float *probs,
                         const int64_t *row_mask, int64_t rows, int64_t H, void *grad_x,
                         float *grad_probs, ptb_stream_t stream);

/* ptb_quant_fp8_segment_row_col applied to SwiGLU-with-probabilities of x [M, 2N] without writing the
 * activation: every tile computes act = round_to_dtype(swiglu(x)) in registers and quantises it, so the
 * six outputs equal ptb_swiglu_probs_fwd followed by ptb_quant_fp8_segment_row_col byte for byte while
 * moving 6 instead of 10 bytes per activation element.  N % 8 == 0; x bf16 / fp16, 16-byte aligned.
 * M == 0: x, probs, q_row and s_row may be NULL, as for ptb_quant_fp8_segment_row_col.
 * Fuses the reference's swiglu_with_probs (primus_turbo/pytorch/ops/activation.py:23-83) with its
 * grouped activation quantise (quantization_impl.py:379-464); the reference runs them as two kernels. */
int ptb_swiglu_quant_fp8_segment_row_col(const void *x, int x_dtype, const float *probs, int64_t M,
                                         int64_t N, int64_t G, const int64_t *group_offs,
                                         void *q_row, void *q_col_padded, float *s_row,
                                         float *s_col_padded, int64_t *var_k_lens,
                                         int64_t *var_k_offs, void *block_table, int q_dtype,
                                         ptb_stream_t stream);

/* ------------------------------------------------------------------ dequantize --------------- */
/* out = cast(float(q) * scale_inv).  Replace dequantize_fp8_tensorwise / dequantize_fp8_rowwise
 * (bindings_pytorch.cpp:43-46) and primus_turbo::dequant_fp8_blockwise_impl /
 * dequant_fp8_blockwise_for_weight_impl (quantization_impl.py:139-227). */
int ptb_dequant_fp8_tensorwise(const void *q, int q_dtype, int64_t n, const float *scale_inv,
                               void *out, int out_dtype, ptb_stream_t stream);
int ptb_dequant_fp8_rowwise(const void *q, int q_dtype, int64_t B, int64_t M, int64_t N,
                            const float *scale_inv, void *out, int out_dtype, ptb_stream_t stream);
int ptb_dequant_fp8_block1d(const void *q, int q_dtype, int64_t M, int64_t N, int axis,
                            const float *scale_inv, void *out, int out_dtype, ptb_stream_t stream);
int ptb_dequant_fp8_block2d(const void *q, int q_dtype, int64_t B, int64_t M, int64_t N,
                            const float *scale_inv, void *out, int out_dtype, ptb_stream_t stream);

/* ------------------------------------------------------------------ helpers ------------------ */
/* Exclusive prefix sum of int64 group lengths: offs[G+1].
 * Replaces torch op grouped_gemm_compute_offs (bindings_pytorch.cpp:129,
 * csrc/pytorch/grouped_gemm/ck_grouped_gemm.cpp:63-80). */
int ptb_group_offs(const int64_t *group_lens, int64_t G, int64_t *group_offs, ptb_stream_t stream);

/* Byte transpose [B, M, N] -> [B, N, M] of 1-byte elements.
 * Replaces torch op transpose_2d (bindings_pytorch.cpp:41) for FP8 payloads. */
int ptb_transpose_2d_u8(const void *in, int64_t B, int64_t M, int64_t N, void *out,
                        ptb_stream_t stream);

/* ------------------------------------------------------------------ row movement ------------- */
/* Copies row segments from src_base to up to 16 destination buffers in one launch:
 *   segments: device int64 [nseg][4] = {first source row, first destination row, rows,
 *   destination index}; dst_bases: host array of n_ranks device pointers (peer memory mapped into this
 *   process, or local memory); rows are row_bytes bytes (a multiple of 16; all bases 16-byte aligned).
 * This is the expert-parallel dispatch / combine of ranks on one node: every rank writes its rows
 * straight to their expert-major position in the owner's buffer with plain stores over NVLink.  The
 * kernel waits on nothing -- the callers order themselves with a collective afterwards.  A segment
 * naming a destination outside [0, n_ranks) is skipped and recorded (ptb_copy_segments_status).
 * num_ctas <= 0 uses one CTA per SM.  At most 8192 segments.
 * Stands where the reference calls its DeepEP port's dispatch / combine
 * (primus_turbo/pytorch/ops/moe/moe_dispatch_combine.py:20-101,
 * primus_turbo/pytorch/kernels/moe/moe_dispatch_combine_impl.py). */
int ptb_copy_segments(const void *src_base, void *const *dst_bases, int n_ranks,
                      const int64_t *segments, int64_t nseg, int64_t row_bytes, int num_ctas,
                      ptb_stream_t stream);

/* ptb_copy_segments that also tells every destination when this rank's rows have landed: after the
 * copies (every thread fences its stores at system scope, the last CTA to finish acts) the kernel stores
 * `seq` with release semantics into flag_slots[r] for every r -- this rank's 32-bit slot in rank r's flag
 * array (peer-mapped like the buffers).  done_counter: a zeroed 32-bit word in local memory that the
 * kernel leaves zero.  Runs (and signals) even when nseg == 0.  Sequence numbers of one slot must grow.
 * ptb_wait_flags launches one warp that waits until flags[0..n) (local memory) have all reached seq;
 * after 20 s it gives up, sets ptb_copy_segments_status to 2 and lets the stream go on.  Together they
 * replace the collective that otherwise orders the ranks after an exchange.  n <= 32.
 * No counterpart in the reference (its DeepEP port keeps such flags inside its own buffers). */
int ptb_copy_segments_signal(const void *src_base, void *const *dst_bases, int n_ranks,
                             const int64_t *segments, int64_t nseg, int64_t row_bytes, int num_ctas,
                             void *const *flag_slots, void *done_counter, uint32_t seq,
                             ptb_stream_t stream);
int ptb_wait_flags(const void *flags, int n, uint32_t seq, ptb_stream_t stream);

/* Lets kernels launched on the current device address memory that lives on peer_device (a device index of
 * this process): cudaDeviceEnablePeerAccess, treating "already enabled" as success.  Memory of another
 * process opened through a CUDA IPC handle is mapped for the device that was current when it was
 * opened; a kernel on a different device may only touch it after this call.  PTB_ERR_UNSUPPORTED when
 * the two devices have no peer path.  No counterpart in the reference. */
int ptb_enable_peer_access(int peer_device);

/* Reads (and optionally clears) the status word: 1 when a copy's segment table named a bad
 * destination, 2 when a flag wait ran out of time.  Synchronises with the device.  No counterpart in the reference. */
int ptb_copy_segments_status(int *status, int reset);

/* out[i, :] = in[index[i], :] for n_out rows of row_bytes bytes (a multiple of 16); an index outside
 * [0, n_in) writes a zero row.  The row gather of the MoE token permutation
 * (csrc/kernels/moe_permute/moe_permute.cu, primus_turbo/pytorch/ops/moe/permutation.py:281-369:
 * ``inp.index_select(0, sorted_indices)``). */
int ptb_gather_rows(const void *in, const int64_t *index, int64_t n_out, int64_t n_in,
                    int64_t row_bytes, void *out, ptb_stream_t stream);

/* MoE token permutation, index part.  routing_map [T, E], one byte per entry (non-zero: token t is routed
 * to expert e).  Writes row_id_map [T, E] int32 -- the row of (t, e) in the expert-major permuted order
 * (experts in increasing id, tokens in increasing id inside an expert), or -1 where the token is not
 * routed or the row falls at or beyond `capacity` -- tokens_per_expert [E] int64 and, if non-NULL,
 * sorted_indices [capacity] int64 (the token id of every permuted row; rows past the routed total are
 * left untouched).  workspace: ceil(T/256) * E * 4 bytes rounded up to 16, plus (E + 1) * 8 bytes.
 * E <= 1024.  Replaces permutation.make_row_id_map and the mask-to-index part of token_permute
 * (primus_turbo/pytorch/ops/moe/permutation.py:18-112,281-369; csrc/kernels/moe_permute/moe_permute.cu). */
int ptb_moe_row_id_map(const void *routing_map, int64_t T, int64_t E, int64_t capacity,
                       int32_t *row_id_map, int64_t *tokens_per_expert, int64_t *sorted_indices,
                       void *workspace, ptb_stream_t stream);

/* out[i, :] = cast(float(in[index[i], :]) * weights[i]) over rows of H elements of type dtype (PTB_F32 /
 * PTB_F16 / PTB_BF16); an index outside [0, n_in) writes a zero row.  The backward pass of the weighted
 * un-permute (permutation.py:151-279 in the reference). */
int ptb_gather_rows_scaled(const void *in, int dtype, const int64_t *index, const float *weights,
                           int64_t n_out, int64_t n_in, int64_t H, void *out, ptb_stream_t stream);

/* Un-permute: out[t, :] = sum over the experts e with row_id_map[t, e] >= 0, in increasing e, of
 * in[row_id_map[t, e], :] * (probs ? probs[t, e] : 1), accumulated in fp32 with separate multiply and
 * add (the value a sequential fp32 scatter-add gives), cast to dtype.  probs: fp32 [T, E] or NULL.
 * Replaces token_unpermute's scatter_add (permutation.py:371-436). */
int ptb_unpermute_rows(const void *in, int dtype, const int32_t *row_id_map, const float *probs,
                       int64_t T, int64_t E, int64_t H, void *out, ptb_stream_t stream);

/* Backward of ptb_unpermute_rows: grad_in[row_id_map[t, e], :] = grad_out[t, :] * p(t, e) and, if
 * grad_probs is non-NULL, grad_probs[t, e] = dot(grad_out[t, :], fwd_in[row_id_map[t, e], :]) (0 where
 * the token is not routed).  Rows of grad_in no token maps to are left untouched. */
int ptb_unpermute_rows_bwd(const void *grad_out, int dtype, const void *fwd_in,
                           const int32_t *row_id_map, const float *probs, int64_t T, int64_t E,
                           int64_t H, void *grad_in, float *grad_probs, ptb_stream_t stream);

/* ------------------------------------------------------------------ GEMM --------------------- */
/* C[M,N] = op(A)[M,K] . op(B)[K,N], FP8 operands, fp32 accumulation, c_dtype output.
 *   a: [M,K] (trans_a = 0, lda = row pitch in elements) or [K,M] (trans_a = 1)
 *   b: [K,N] (trans_b = 0) or [N,K] (trans_b = 1)
 * granularity:
 *   PTB_TENSORWISE  C = acc * (a_scale[0]*b_scale[0])
 *   PTB_ROWWISE     C = acc * (a_scale[m*a_scale_stride_m] * b_scale[n*b_scale_stride_n])
 *   PTB_BLOCKWISE   per 128-wide contraction block kb:
 *        acc += partial_kb * a_scale[m*a_scale_stride_m + kb*a_scale_stride_k]
 *                          * b_scale[(b_block_2d ? n/128 : n)*b_scale_stride_n + kb*b_scale_stride_k]
 * Pointers and leading dimensions must be 16-byte aligned.  num_sms <= 0 uses every SM.
 * Replaces primus_turbo::gemm_fp8_impl
 * (primus_turbo/pytorch/kernels/gemm/gemm_fp8_impl.py:438-467), i.e. the torch ops
 * hipblaslt_gemm_fp8 and ck_gemm_fp8 (csrc/pytorch/gemm/ck_gemm.cpp:32-98) and the Triton
 * kernels in primus_turbo/triton/gemm/gemm_fp8_kernel.py. */
int ptb_gemm_fp8(const void *a, int a_dtype, int trans_a, int64_t lda, const void *b, int b_dtype,
                 int trans_b, int64_t ldb, void *c, int c_dtype, int64_t ldc, int64_t M, int64_t N,
                 int64_t K, int granularity, const float *a_scale, int64_t a_scale_stride_m,
                 int64_t a_scale_stride_k, const float *b_scale, int64_t b_scale_stride_n,
                 int64_t b_scale_stride_k, int b_block_2d, int num_sms, ptb_stream_t stream);

/* ------------------------------------------------------------------ MXFP8 (1x32 blocks, E8M0 scales) */
/* Quantise x[G][M][N] (bf16/fp16, contiguous; G = 1 for a matrix) in one pass into
 *   q_row[G][M][N_pad]  + s_row[G][M][N_pad/32]   blocks of 32 along a row,
 *   q_col[G][N][M_pad]  + s_col[G][N][M_pad/32]   blocks of 32 along a column, stored TRANSPOSED,
 * N_pad / M_pad = N / M rounded up to 128; the padding holds zero bytes with scale byte 0.  A scale byte
 * is a biased power-of-two exponent (E8M0).  Either direction may be omitted (both its pointers NULL).
 * row_2d_block / col_2d_block != 0: one scale per 32x32 tile for that direction.  N % 32 == 0; x and
 * the FP8 outputs 16-byte aligned.
 * Replaces the torch ops quantize_mxfp8 / quantize_mxfp8_dual
 * (csrc/pytorch/quantization/quantization.cpp:736-966, kernels csrc/kernels/quantization/quantization_mxfp8.cu);
 * the reference's shuffled layouts (scale or data pre-shuffle for its own GEMM back ends) are not offered. */
int ptb_quant_mxfp8(const void *x, int x_dtype, int64_t G, int64_t M, int64_t N, void *q_row, void *s_row,
                    void *q_col, void *s_col, int row_2d_block, int col_2d_block, int q_dtype,
                    ptb_stream_t stream);

/* Grouped form of ptb_quant_mxfp8 for x[M][N] whose rows form G groups (group_offs: device int64
 * [G+1]): every group is quantised on its own, its rows padded with zeros to `row_align` rows (1 or 32)
 * in the row-direction output and to 128 rows in the column-direction output:
 *   q_row[M_row][N_pad] + s_row[M_row][N_pad/32]      M_row >= M + G*(row_align-1): only rows that
 *                                                     exist are written, at row_offs_padded[g] + i;
 *   q_col[N][M_col] + s_col[N][M_col/32], transposed, M_col = ceil((M + G*128)/128)*128: group g's
 *                                                     rows at columns col_offs_padded[g] + i; every
 *                                                     other column is written as zero.
 * A block whose maximum is zero takes scale byte 127 (1.0), as the reference's grouped kernel does.
 * Also written: the padded lengths and offsets of both layouts (device int64 [G] / [G+1]).
 * block_table: workspace of 16 bytes per 128-row block of the column layout (M_col/128 blocks),
 * 16-byte aligned.  M == 0: x (and, with row_align 1, q_row / s_row) may be NULL; the layouts and the
 * zero columns are still written.  Replaces grouped_quantize_mxfp8_dual
 * (csrc/pytorch/quantization/quantization.cpp:1075-1195; the reference's row layout is row_align = 32). */
int ptb_quant_mxfp8_grouped(const void *x, int x_dtype, int64_t M, int64_t N, const int64_t *group_offs,
                            int64_t G, int64_t row_align, void *q_row, void *s_row, void *q_col,
                            void *s_col, int64_t *row_lens_padded, int64_t *row_offs_padded,
                            int64_t *col_lens_padded, int64_t *col_offs_padded, void *block_table,
                            int row_2d_block, int col_2d_block, int q_dtype, ptb_stream_t stream);

/* out = cast(float(q[R][C]) * 2^(scale byte - 127)) (byte 0 multiplies by 0.0f as the reference does),
 * scales[R][C/32]; transpose_out != 0 writes out[C][R] (the column-direction data come back as
 * [M_pad][N]).  Replaces dequantize_mxfp8 (quantization.cpp:283-358, dequantization_mxfp8.cu:47-100). */
int ptb_dequant_mxfp8(const void *q, int q_dtype, int64_t R, int64_t C, const void *scales,
                      int transpose_out, void *out, int out_dtype, ptb_stream_t stream);

/* C[M,N] = A[M,K] . B[N,K]^T with one E8M0 scale per 32 contraction elements of every A and B row,
 * applied by the block-scaled tensor-core instruction (tcgen05.mma kind::mxf8f6f4.block_scale); fp32
 * accumulation over the whole K, c_dtype output.  K is the padded extent (a multiple of 128);
 * a_sf[M][a_sf_ld], b_sf[N][b_sf_ld] bytes with a_sf_ld, b_sf_ld >= K/32, multiples of 4, 4-byte
 * aligned bases.  Every MX GEMM of the reference is this NT form (forward, dgrad and wgrad use the
 * row- and column-direction copies: primus_turbo/pytorch/ops/gemm_fp8.py:582-640).  Replaces
 * gemm_fp8_impl with granularity MX_BLOCKWISE (kernels/gemm/gemm_fp8_impl.py:438-467). */
int ptb_gemm_mxfp8(const void *a, int a_dtype, int64_t lda, const void *a_sf, int64_t a_sf_ld,
                   const void *b, int b_dtype, int64_t ldb, const void *b_sf, int64_t b_sf_ld, void *c,
                   int c_dtype, int64_t ldc, int64_t M, int64_t N, int64_t K, int num_sms,
                   ptb_stream_t stream);

/* Grouped forms of ptb_gemm_mxfp8.
 *   ptb_grouped_gemm_mxfp8: out[offs[g]:offs[g+1], :] = a[offs[g]:offs[g+1], :] . b[g]^T with a [M_total, K]
 *   (+ a_sf [M_total, a_sf_ld]), b [G, N, K] and b_sf [G, N, K/32] contiguous; rows >= offs[G] zeroed.
 *   ptb_grouped_gemm_mxfp8_variable_k: out[g] = lhs[:, offs[g]:offs[g+1]] . rhs[:, offs[g]:offs[g+1]]^T with the
 *   transposed column copies lhs [OUT_M, rows_padded], rhs [OUT_N, rows_padded] of the grouped quantiser
 *   (offsets multiples of 128: its col_offs_padded); an empty group gives a zero matrix.
 * At most 1024 groups.  Replace grouped_gemm_fp8_impl / grouped_gemm_fp8_variable_k_impl with granularity
 * MX_BLOCKWISE (primus_turbo/pytorch/ops/grouped_gemm_fp8.py:571-795). */
int ptb_grouped_gemm_mxfp8(const void *a, int a_dtype, int64_t lda, const void *a_sf, int64_t a_sf_ld,
                           const void *b, int b_dtype, const void *b_sf, void *out, int out_dtype,
                           int64_t ldc, const int64_t *group_offs, int64_t G, int64_t M_total, int64_t N,
                           int64_t K, int num_sms, ptb_stream_t stream);
int ptb_grouped_gemm_mxfp8_variable_k(const void *lhs, int lhs_dtype, int64_t ld_lhs, const void *lhs_sf,
                                      int64_t lhs_sf_ld, const void *rhs, int rhs_dtype, int64_t ld_rhs,
                                      const void *rhs_sf, int64_t rhs_sf_ld, void *out, int out_dtype,
                                      const int64_t *group_offs_padded, int64_t G, int64_t rows_padded,
                                      int64_t OUT_M, int64_t OUT_N, int num_sms, ptb_stream_t stream);

/* Grouped GEMM over row segments of a (forward and dgrad of the MoE experts):
 *   out[offs[g]:offs[g+1], :] = a[offs[g]:offs[g+1], :] . op(b[g]),   rows >= offs[G] zeroed.
 *   a [M_total, K]; b [G, N, K] (trans_b = 1) or [G, K, N] (trans_b = 0), contiguous;
 *   group_offs: device int64 [G+1].  Scales as in ptb_gemm_fp8 with an extra group stride on b
 *   (blockwise: a_scale is indexed by absolute row; b_scale by (g, n/128, kb)).
 * At most 1024 groups per call (the kernel keeps its tile table in shared memory;
 * PTB_ERR_TOO_LARGE beyond that -- split the call).
 * Replaces primus_turbo::grouped_gemm_fp8_impl
 * (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp8_impl.py:817-859) including its
 * tail-zeroing launch. */
int ptb_grouped_gemm_fp8(const void *a, int a_dtype, int64_t lda, const void *b, int b_dtype,
                         int trans_b, void *out, int out_dtype, int64_t ldc,
                         const int64_t *group_offs, int64_t G, int64_t M_total, int64_t N,
                         int64_t K, int granularity, const float *a_scale,
                         int64_t a_scale_stride_m, int64_t a_scale_stride_k, const float *b_scale,
                         int64_t b_scale_stride_g, int64_t b_scale_stride_n,
                         int64_t b_scale_stride_k, int num_sms, ptb_stream_t stream);

/* Variable-K grouped GEMM (wgrad): out[g] [OUT_M, OUT_N] = lhs_g^T . rhs_g where the contraction
 * runs over rows [group_offs[g], group_offs[g+1]) of lhs [rows, OUT_M] and rhs [rows, OUT_N].
 * Empty groups produce zeros.
 *   PTB_BLOCKWISE:  every group offset is a multiple of 128 (segment-padded operands); scales are
 *                   [rows/128, OUT_M] and [rows/128, OUT_N], applied per 128-row block.
 *   PTB_ROWWISE:    lhs_scale[OUT_M], rhs_scale[OUT_N] applied to the finished tile; any offsets.
 *   PTB_TENSORWISE: lhs_scale[1], rhs_scale[1]; any offsets.
 * With unpadded offsets the rows of lhs / rhs outside a group's range never reach its result,
 * whatever bytes they hold.  At most 1024 groups per call.
 * Replaces primus_turbo::grouped_gemm_fp8_variable_k_impl (grouped_gemm_fp8_impl.py:862-901). */
int ptb_grouped_gemm_fp8_variable_k(const void *lhs, int lhs_dtype, int64_t ld_lhs,
                                    const void *rhs, int rhs_dtype, int64_t ld_rhs, void *out,
                                    int out_dtype, const int64_t *group_offs, int64_t G,
                                    int64_t rows, int64_t OUT_M, int64_t OUT_N, int granularity,
                                    const float *lhs_scale, const float *rhs_scale, int num_sms,
                                    ptb_stream_t stream);

/* Every device-side wait in the GEMM kernels is bounded (2 s); a kernel whose wait runs out
 * records a non-zero code (1 copy producer, 2 MMA issuer, 3 epilogue, 4 scale loader) and
 * leaves normally.  This call copies that code to *status (a host pointer) and optionally
 * clears it.  It synchronises with the device.  The code is one word per GPU, shared by every
 * stream and caller of the library in the process: a non-zero value says that some GEMM launched
 * since the last reset gave up, not which one.  No counterpart in the reference. */
int ptb_gemm_status(int *status, int reset);

/* Launches one warp that waits, with the same bounded wait, on a barrier nothing arrives on: after
 * the limit (2 s) the kernel records status code 9 and returns normally.  It lets a host check the
 * give-up path and its reporting without provoking a fault.  No counterpart in the reference. */
int ptb_gemm_wait_selftest(ptb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PTB_H_ */
