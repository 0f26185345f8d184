/*
 * mslk_b200 -- C ABI of the B200 (sm_100a) low-precision GEMM path.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer on the
 * current CUDA device unless stated otherwise, every function enqueues its
 * work on `stream` (a cudaStream_t passed as void*) and returns without
 * synchronising the host, so all entry points may be captured in a CUDA graph.
 * Return value: 0 on success, non-zero on a rejected argument or a CUDA launch
 * error; the message is available from mslk_b200_last_error() (thread-local).
 *
 * Each entry point names the reference (meta-pytorch/MSLK) interface it
 * replaces.
 */
#ifndef MSLK_B200_H_
#define MSLK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSLK_B200_ABI_VERSION 1

/* element type codes for high-precision inputs */
#define MSLK_B200_F32 0
#define MSLK_B200_BF16 1
#define MSLK_B200_F16 2

/* bias kinds of f8f8bf16_rowwise */
#define MSLK_B200_BIAS_NONE 0
#define MSLK_B200_BIAS_F32 1
#define MSLK_B200_BIAS_BF16 2

int mslk_b200_abi_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char *mslk_b200_last_error(void);

/*
 * Reads (and clears) the device-side status word of the current device after
 * synchronising it.  0 = no kernel reported a problem.  A kernel whose bounded
 * pipeline wait expired stores a non-zero code here and exits cleanly instead
 * of hanging.  This call synchronises the device; do not use it under capture.
 */
int mslk_b200_device_status(int *status_out);

/*
 * Self-test of the bounded waits every pipeline kernel of this library uses: launches one tiny CTA that
 * waits on an mbarrier nothing ever arrives on, with `limit_ns` (<= 100 ms) as the limit instead of the
 * kernels' 2 s.  The wait gives up by itself: the kernel stores the epilogue-timeout code (3) in the device
 * status word, writes 1 to *returned_flag (device int, may be NULL) and returns normally -- the context stays
 * usable.  The reference's nearest analogue is the launch-error check of
 * include/mslk/utils/kernel_launcher.cuh:420-448; it has no device-side wait bound.
 */
int mslk_b200_selftest_wait_timeout(uint64_t limit_ns, int *returned_flag, void *stream);

/*
 * Per-row FP8 (e4m3fn) quantization.
 * Replaces: mslk/quantize/triton/fp8_quantize.py:36-207 (_kernel_quantize_fp8_row)
 *           as launched by triton_quantize_fp8_row (:210-316).
 *
 * x is read as a 4-D tensor [B, M, N, K] of `dtype` with ELEMENT strides
 * sb, sm, sn, sk.  Row r = (b*M + m)*N + n gets
 *     scale[r] = min(max(amax_r, eps), *scale_ub) / 448      (scale_ub may be NULL)
 *     q[r, k]  = e4m3_rn_satfinite(x[r, k] / scale[r])        k <  K
 *     q[r, k]  = 0                                            K <= k < K_out
 * with IEEE fp32 divisions.  zero_start_index_M (int64 [B*M], may be NULL) marks
 * rows n >= zero_start_index_M[b*M+m] as all-zero.  q is contiguous
 * [B*M*N, K_out] bytes, scale is fp32 [B*M*N].
 */
int mslk_b200_quantize_fp8_row(const void *x, int dtype, int64_t B, int64_t M, int64_t N,
                               int64_t K, int64_t K_out, int64_t sb, int64_t sm, int64_t sn,
                               int64_t sk, const float *scale_ub,
                               const int64_t *zero_start_index_M, float eps, void *q,
                               float *scale, void *stream);

/*
 * Rowwise-scaled FP8 GEMM:  y[m,n] = bf16((x_scale[m] * sum_k xq[m,k]*wq[n,k]) * w_scale[n] (+ bias[n])).
 * Replaces: csrc/gemm/cutlass/f8f8bf16_rowwise.cu:183-206 (f8f8bf16_rowwise / _out)
 *           and f8f8bf16_rowwise/f8f8bf16_rowwise_common.cuh:44-346 (the kernel).
 * xq [M,K] and wq [N,K] are contiguous e4m3fn bytes, K % 16 == 0; y is contiguous
 * bf16 [M,N].  bias ([N], fp32 or bf16 per bias_kind) may be NULL.
 */
int mslk_b200_f8f8bf16_rowwise(const void *xq, const void *wq, const float *x_scale,
                               const float *w_scale, const void *bias, int bias_kind, void *y,
                               int64_t M, int64_t N, int64_t K, void *stream);

/*
 * N-sharded GEMM fused with the all-gather of its output (tensor parallelism inside one node).
 * Rank `rank` of `world` (<= 8) holds the weight rows [rank*N_local, (rank+1)*N_local) and computes
 * its [M, N_local] column block; the kernel's epilogue stores that block at column rank*N_local of
 * EVERY rank's row-major [M, world*N_local] bf16 output: y_bases is a HOST array of `world` device
 * pointers, y_bases[rank] the local buffer, the others peer-mapped buffers of the other GPUs
 * (plain stores over NVLink, no separate collective, no re-layout copy).  The caller synchronises
 * the ranks afterwards (any barrier on the same streams) before a rank reads columns it did not
 * write.  New with respect to the reference, whose operator is single-GPU
 * (csrc/gemm/cutlass/f8f8bf16_rowwise.cu:183-206).
 */
int mslk_b200_f8f8bf16_rowwise_allgather(const void *xq, const void *wq_shard, const float *x_scale,
                                         const float *w_scale_shard, const void *bias_shard,
                                         int bias_kind, void *const *y_bases, int world, int rank,
                                         int64_t M, int64_t N_local, int64_t K, void *stream);

/*
 * K-sharded GEMM fused with the data movement of a reduce-scatter over the token dimension.
 * Rank `rank` of `world` multiplies its K slices (xq_kshard [M, K_local], wq_kshard [N, K_local];
 * x_scale / w_scale are the scales of the UNSHARDED rows, so the scaled partial products add up)
 * and its epilogue deposits rows [o*M/world, (o+1)*M/world) of the partial product in slot `rank`
 * of owner o's staging buffer: stage_bases is a HOST array of `world` device pointers to bf16
 * [world, M/world, N] buffers (stage_bases[rank] local, the others peer-mapped), written with TMA
 * stores over NVLink tile by tile while the GEMM runs.  After the ranks have synchronised, every
 * rank calls mslk_b200_reduce_slots_bf16 on its own staging buffer to get its [M/world, N] rows of
 * the sum (fp32 accumulation in rank order).  Needs M % (32*world) == 0, N % 64 == 0.
 * New with respect to the reference (single-GPU operator).
 */
int mslk_b200_f8f8bf16_rowwise_scatter(const void *xq_kshard, const void *wq_kshard,
                                       const float *x_scale, const float *w_scale,
                                       void *const *stage_bases, int world, int rank, int64_t M,
                                       int64_t N, int64_t K_local, void *stream);
int mslk_b200_reduce_slots_bf16(const void *slots_base, int slots, int64_t rows, int64_t cols,
                                void *out, void *stream);

/*
 * Same operation with caller-provided scratch memory (opt-in split-K for few tokens, M <= 32).
 * With a workspace of at least mslk_b200_f8f8bf16_rowwise_workspace_bytes(M, N, K) bytes the
 * weights are streamed by a kernel that splits the K dimension over several CTAs; partial sums and
 * completion tickets live in `workspace`, the sum is formed in split order (bit-reproducible).
 * A null or too small workspace is legal and means the same kernels as
 * mslk_b200_f8f8bf16_rowwise.  The operator layer does not use the split: on the Llama-3-8B
 * projection shapes measured on a B200 the unsplit 32-column tiles were faster.  The workspace
 * needs no initialisation and may be reused by later calls on the same stream; calls that may
 * overlap on the GPU need separate workspaces.
 * Replaces: the workspace the reference allocates inside its op,
 *           csrc/gemm/cutlass/f8f8bf16_rowwise/f8f8bf16_rowwise_common.cuh:316-334.
 */
size_t mslk_b200_f8f8bf16_rowwise_workspace_bytes(int64_t M, int64_t N, int64_t K);
int mslk_b200_f8f8bf16_rowwise_ws(const void *xq, const void *wq, const float *x_scale,
                                  const float *w_scale, const void *bias, int bias_kind, void *y,
                                  int64_t M, int64_t N, int64_t K, void *workspace,
                                  size_t workspace_bytes, void *stream);

/*
 * The few-token GEMM for hosts that cannot allocate device memory when they call (all HBM
 * already handed to a KV-cache pool, a memory plan frozen at start-up, or a thread that must
 * not run cudaMalloc because it stalls the device).  The split-K scratch is an 8 MiB array
 * built into the library image (held by every GPU that loads the library until exit); the call
 * allocates and frees nothing.  Serves 1 <= M <= 128, N >= 128, K % 16 == 0 as long as the
 * split-K scratch of the shape fits the 8 MiB (always true for M <= 32; for more tokens only
 * small N*K do); a shape that needs more is rejected with a message, never truncated.  The first call on a
 * device looks up the array's device address: make that call outside stream capture.  Up to 32
 * tokens the kernel splits K inside thread-block clusters and does not touch the array, so such
 * calls may overlap freely.  With more tokens all calls on a GPU share the array -- the tickets in
 * it are cleared on the stream before each launch, the partial sums are overwritten -- so calls
 * that could overlap on one GPU must be ordered by the caller.  Same arithmetic and arguments as
 * mslk_b200_f8f8bf16_rowwise.
 * This entry point has no counterpart in the reference (its op always allocates its workspace).
 */
int mslk_b200_f8f8bf16_rowwise_noalloc(const void *xq, const void *wq, const float *x_scale,
                                       const float *w_scale, const void *bias, int bias_kind,
                                       void *y, int64_t M, int64_t N, int64_t K, void *stream);

/*
 * Grouped (stacked) rowwise FP8 GEMM for MoE experts.
 * Replaces: csrc/gemm/cutlass/f8f8bf16_rowwise_grouped.cu:342-368
 *           (f8f8bf16_rowwise_grouped_stacked) with its argument-setup kernel and
 *           grouped kernel, f8f8bf16_rowwise_grouped_sm100/
 *           f8f8bf16_rowwise_grouped_common.cuh:148-213,225-606.
 * xq [total_M,K], wq [G,N,K], x_scale [total_M], w_scale [G*N], y [total_M,N] bf16.
 * M_sizes is int64 [G] ON THE DEVICE (never read by the host); group g owns rows
 * [sum_{i<g} M_sizes[i], +M_sizes[g]).  Rows past the sum are left untouched.
 */
int mslk_b200_f8f8bf16_rowwise_grouped_stacked(const void *xq, const void *wq,
                                               const float *x_scale, const float *w_scale,
                                               const int64_t *M_sizes, int64_t G,
                                               int64_t total_M, int64_t N, int64_t K, void *y,
                                               void *stream);

/*
 * Batched rowwise-scaled FP8 GEMM:  y[b] = f8f8bf16_rowwise(xq[b], wq[b], x_scale[b], w_scale[b], bias[b]).
 * Replaces: csrc/gemm/cutlass/f8f8bf16_rowwise_batched.cu:20-139 and
 *           f8f8bf16_rowwise_batched/f8f8bf16_rowwise_batched_common.cuh:40-340.
 * xq [B,M,K], wq [B,N,K] e4m3 contiguous; x_scale [B,M], w_scale [B,N] fp32; bias [B,N]
 * (kind as for mslk_b200_f8f8bf16_rowwise, may be NULL); y [B,M,N] bf16.  One launch: the
 * batches are scheduled as B equal groups of the grouped kernel.  B <= 1024.
 */
int mslk_b200_f8f8bf16_rowwise_batched(const void *xq, const void *wq, const float *x_scale,
                                       const float *w_scale, const void *bias, int bias_kind,
                                       void *y, int64_t B, int64_t M, int64_t N, int64_t K,
                                       void *stream);

/*
 * The grouped GEMM with the MoE combine fused into its epilogue: stacked row r of the product is ADDED
 * atomically to row scatter_indices[r] of y (bf16 [y_rows, N], which the caller has initialised) instead
 * of being stored at row r.  Replaces: mslk/gemm/triton/grouped_gemm.py:1112-1137
 * (grouped_gemm_fp8_rowwise with _output_tensor / _scatter_add_indices; epilogue :386-402).
 * Indices are int32 or int64 on the device (`index_bits`).  With several rows landing on one output row
 * the sum depends on the order of the atomics, as in the reference.  An index outside [0, y_rows) skips
 * the row and sets bit 0x200 of the device status word.
 */
int mslk_b200_f8f8bf16_rowwise_grouped_stacked_scatter_add(
    const void *xq, const void *wq, const float *x_scale, const float *w_scale, const int64_t *M_sizes,
    int64_t G, int64_t total_M, int64_t N, int64_t K, const void *scatter_indices, int index_bits,
    void *y, int64_t y_rows, void *stream);

/*
 * NVFP4 quantization (e2m1 data, one e4m3 scale per 16 elements in the 128x4
 * swizzled layout, optional fp32 per-tensor global scale read from the device).
 * Replaces: mslk/quantize/triton/quantize_kernels/nvfp4.py:62-296.
 * x is bf16 [M,K] with row stride `row_stride` elements, K % 16 == 0.
 * q is [M, K/2] bytes (element 2j in the low nibble); scales is
 * [ceil(M/128)*128 * ceil(K/64)*4] bytes and is written completely (padding = 0).
 */
int mslk_b200_quantize_nvfp4(const void *x, int64_t M, int64_t K, int64_t row_stride,
                             const float *global_scale, void *q, void *scales, void *stream);
/* The same with the input type given: dtype = MSLK_B200_BF16 or MSLK_B200_F16 (the reference's kernel takes either). */
int mslk_b200_quantize_nvfp4_dt(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                const float *global_scale, void *q, void *scales, void *stream);

/*
 * NVFP4 GEMM:  y = bf16(*global_scale * sum_blocks (sx*sw) * sum_16 x^*w^).
 * Replaces: csrc/gemm/cutlass/f4f4bf16.cu:6413-6473 (NVFP4 branch) and
 *           f4f4bf16/f4f4bf16_common.cuh:78-315.
 * xq [M,K/2], wq [N,K/2] packed e2m1; x_scale / w_scale swizzled e4m3 as produced
 * by mslk_b200_quantize_nvfp4; global_scale is a device fp32 scalar; K % 32 == 0.
 */
int mslk_b200_f4f4bf16(const void *xq, const void *wq, const void *x_scale,
                       const void *w_scale, const float *global_scale, void *y, int64_t M,
                       int64_t N, int64_t K, void *stream);

/*
 * Same GEMM with caller-provided scratch memory.  With 1 <= M <= 128 tokens the weight-streaming
 * kernel may split K over several CTAs per 128 weight rows; the fp32 partial tiles and completion
 * counters then live in `workspace` (mslk_b200_f4f4bf16_workspace_bytes(M, N, K) bytes, 0 when the
 * shape needs none; 16-byte aligned, contents irrelevant on entry, not shared by calls that may run
 * at the same time).  Without workspace (null or too small) the same kernel runs unsplit.
 */
size_t mslk_b200_f4f4bf16_workspace_bytes(int64_t M, int64_t N, int64_t K);
int mslk_b200_f4f4bf16_ws(const void *xq, const void *wq, const void *x_scale,
                          const void *w_scale, const float *global_scale, void *y, int64_t M,
                          int64_t N, int64_t K, void *workspace, size_t workspace_bytes,
                          void *stream);

/*
 * MXFP4 quantization: e2m1 data with one e8m0 (power-of-two) scale per group of `group_size` elements (32 = OCP MXFP4,
 * 16 = the reference's MXFP4-16 recipe), scales in the same 128 x 4 swizzled layout as the NVFP4 scales, no global scale.
 * Replaces: mslk/quantize/triton/quantize_kernels/mx4.py:28-355 (quantize_mx4_kernel + quantize_mx4) with
 *           fp4_primitives/scale.py:96-265 (shared exponent, normalize, e8m0 encode).
 * x is bf16 or fp16 [M, K] with row stride `row_stride` elements, K % group_size == 0.  rounding_mode follows the
 * reference's RoundingMode: 0 nearest (floor(log2(max) + 0.5)), 1 floor, 2 even, 4 ceil (its default); stochastic (3)
 * needs a seed and goes through the _seeded entry point below.
 * q is [M, K/2] bytes; scales is [ceil(M/128)*128 * ceil(K/group_size/4)*4] bytes, written completely (padding = 0).
 */
int mslk_b200_quantize_mx4(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride, int group_size,
                           int rounding_mode, void *q, void *scales, void *stream);

/*
 * The same with the seed of the stochastic mode (rounding_mode 3; the other modes ignore it): the shared exponent and the
 * conversion of every element are perturbed by two Philox-4x32-7 streams keyed by `seed`, counter = the group's /
 * element's index (mslk/quantize/triton/fp4_primitives/scale.py:213-261, tl.randint(seed, offset, n_rounds=7)); the
 * reference passes the caller's seed masked to 63 bits, or the CUDA generator's initial seed
 * (mslk/quantize/triton/quantize_kernels/__init__.py:20-44).  Same seed, same bytes as the reference's kernel.
 */
int mslk_b200_quantize_mx4_seeded(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride, int group_size,
                                  int rounding_mode, uint64_t seed, void *q, void *scales, void *stream);

/*
 * MXFP4 quantization of stacked segments (MoE activations): segment g owns m_sizes[g] (device int64 [G]) consecutive
 * rows of x [M, K]; its scale rows start on a 128-row boundary of the padded scale matrix, at sum_{i<g} roundup(m_i, 128)
 * -- the x_scale layout of mslk_b200_f4f4bf16_grouped_stacked_mx.
 * Replaces: mslk/quantize/triton/quantize_kernels/mx4_stacked.py:34-360 (quantize_mx4_stacked).
 * q is [M, K/2] bytes; scales is [(M + 127 G) * ceil(K/group_size/4)*4] bytes (the reference's upper bound, no host
 * read of the sizes), written completely: everything that is not a scale of a live row is 0.  G <= 1024.
 */
int mslk_b200_quantize_mx4_stacked(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                   const int64_t *m_sizes, int64_t G, int group_size, int rounding_mode, void *q,
                                   void *scales, void *stream);

/* Stacked form with the seed of the stochastic mode; the random streams are indexed by the row of the padded scale
 * matrix, as in the reference's kernel (mslk/quantize/triton/quantize_kernels/mx4_stacked.py:128-146). */
int mslk_b200_quantize_mx4_stacked_seeded(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                          const int64_t *m_sizes, int64_t G, int group_size, int rounding_mode,
                                          uint64_t seed, void *q, void *scales, void *stream);

/*
 * MXFP4 GEMMs:  y = bf16(sum_blocks 2^(sx-127) * 2^(sw-127) * sum_block x^ * w^), the forms of f4f4bf16,
 * f4f4bf16_grouped_stacked and f4f4bf16_grouped_mm the reference runs when no global scale is given
 * (csrc/gemm/cutlass/f4f4bf16.cu:6413-6473 MXFP4 / MXFP4_16 branches; f4f4bf16_grouped.cu:321-475 with use_mx).
 * Operands as for the NVFP4 entry points, scales as mslk_b200_quantize_mx4 writes them (grouped: every group's scale
 * rows start on a 128-row boundary); block_size = 32 or 16; K % 32 == 0.
 */
int mslk_b200_f4f4bf16_mx(const void *xq, const void *wq, const void *x_scale, const void *w_scale, void *y, int64_t M,
                          int64_t N, int64_t K, int block_size, void *stream);
int mslk_b200_f4f4bf16_grouped_stacked_mx(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                          const int64_t *M_sizes, const int64_t *starting_row_after_padding,
                                          int64_t G, int64_t total_M, int64_t N, int64_t K, int block_size, void *y,
                                          void *stream);
int mslk_b200_f4f4bf16_grouped_mm_mx(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                     const int32_t *offsets, int64_t G, int64_t total_M, int64_t N, int64_t K,
                                     int block_size, void *y, void *stream);

/*
 * Diagnostics of the CTA-pair NVFP4 kernel's pipeline.  `dev_counters` is a device array of seven 64-bit
 * counters (zeroed by the caller) or NULL to switch the measurement off; while set, every launch of the pair
 * kernel adds SM clock cycles summed over its CTA pairs: [0] the MMA-issuing lane waiting for operand stages
 * to arrive, [1] the same lane waiting for the epilogue to hand back the accumulator, [2] that lane's whole
 * loop, [3] the leader's TMA-issuing lane waiting for free stages, [4] the leader's first epilogue warp between the
 * accumulator becoming ready and handing it back (reading the columns the next tile's accumulator overlaps), [5] that
 * warp waiting for the accumulator, [6] the same warp reading its remaining columns.  No counterpart in the reference.
 */
int mslk_b200_debug_nvfp4_pair_timers(unsigned long long *dev_counters);

/*
 * K-grouped ("2D-2D") FP4 GEMM:  y[g] = X[:, k_{g-1}:k_g] * W[:, k_{g-1}:k_g]^T  for G groups along K (the weight-gradient
 * shape of a grouped layer).  Replaces: csrc/gemm/cutlass/f4f4bf16_grouped.cu:434-446 (f4f4bf16_grouped_mm with 2D XQ
 * and 2D WQ) with include/mslk/gemm/cutlass/grouped_common.cuh:104-213.
 * xq [M, total_K/2], wq [N, total_K/2] packed e2m1 (the reference passes wq as the transposed view [total_K, N]);
 * k_end_offsets: device int32 [G] END offsets along K, multiples of 32, non-decreasing, <= total_K (a group that breaks
 * this yields zeros and sets bit 0x400 of the device status word; an empty group yields zeros).  Scales: one swizzled
 * block per group, [ceil(M/128)*128 (or N) rows][ceil(K_g/block/4)*4 columns], the blocks following each other;
 * global_scale fp32 [G] selects NVFP4 (e4m3 scales per 16), NULL selects MXFP4 with block_size 32 or 16 (e8m0).
 * x_scale_bytes / w_scale_bytes: sizes of the two scale tensors; offsets whose padded scale blocks would not fit are
 * rejected on the device the same way (zeros, bit 0x400), the kernel never reads past these sizes.
 * y [G, M, N] bf16.  G <= 1024.
 */
int mslk_b200_f4f4bf16_grouped_mm_2d2d(const void *xq, const void *wq, const void *x_scale, const void *w_scale,
                                       const int32_t *k_end_offsets, const float *global_scale, int64_t G, int64_t M,
                                       int64_t N, int64_t total_K, int block_size, size_t x_scale_bytes,
                                       size_t w_scale_bytes, void *y, void *stream);

/*
 * Grouped (stacked) NVFP4 GEMM for mixture-of-experts layers: group g multiplies its m_g stacked rows
 * of xq by its own weight block wq[g] and scales the result by global_scale[g].
 * Replaces: csrc/gemm/cutlass/f4f4bf16_grouped.cu:321-374 (f4f4bf16_grouped_stacked, NVFP4 mode) with
 *           f4f4bf16_grouped/f4f4bf16_grouped_common.cuh:57-148, and :376-475 (f4f4bf16_grouped_mm, 2D-3D
 *           NVFP4 case) with include/mslk/gemm/cutlass/grouped_common.cuh:215-300.
 * xq [total_M, K/2], wq [G, N, K/2] packed e2m1; x_scale: swizzled e4m3 atoms of the padded scale
 * matrix in which every group starts on a 128-row boundary (what mslk_b200_quantize_nvfp4_stacked
 * writes); w_scale: [G][roundup(N,128)][K/16] swizzled per group; global_scale fp32 [G]; y [total_M, N]
 * bf16.  Group sizes come from the device: int64 M_sizes [G] (stacked form) or int32 END offsets [G]
 * (grouped_mm form).  starting_row_after_padding (int64 [G+1], first scale row of every group, multiples
 * of 128) may be NULL: the groups are then taken to follow each other, each padded to 128 rows.
 * Rows past the sum of the sizes are left untouched.  K % 32 == 0, G <= 1024.
 */
int mslk_b200_f4f4bf16_grouped_stacked(const void *xq, const void *wq, const void *x_scale,
                                       const void *w_scale, const int64_t *M_sizes,
                                       const float *global_scale,
                                       const int64_t *starting_row_after_padding, int64_t G,
                                       int64_t total_M, int64_t N, int64_t K, void *y, void *stream);
int mslk_b200_f4f4bf16_grouped_mm(const void *xq, const void *wq, const void *x_scale,
                                  const void *w_scale, const int32_t *offsets,
                                  const float *global_scale, int64_t G, int64_t total_M, int64_t N,
                                  int64_t K, void *y, void *stream);

/*
 * NVFP4 quantization of stacked groups with one global scale per group.
 * Replaces: mslk/quantize/triton/legacy/quantize_stacked.py:22-178,315-400 (nvfp4_quantize_stacked).
 * x bf16 [M, K] (row stride in elements), m_sizes int64 [G] and global_scale fp32 [G] on the device.
 * q [M, K/2]; scales: buffer of (M + 127*G) x roundup(K/16, 4) bytes holding the swizzled atoms of the
 * padded scale matrix; the blocks of all groups present are written completely (padding = 0), the
 * unused tail of the buffer is not touched.  Rows past sum(m_sizes) are not quantized.
 */
int mslk_b200_quantize_nvfp4_stacked(const void *x, int64_t M, int64_t K, int64_t row_stride,
                                     const int64_t *m_sizes, int64_t G, const float *global_scale,
                                     void *q, void *scales, void *stream);
int mslk_b200_quantize_nvfp4_stacked_dt(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                        const int64_t *m_sizes, int64_t G, const float *global_scale, void *q,
                                        void *scales, void *stream);   /* dtype: MSLK_B200_BF16 or MSLK_B200_F16 */

/*
 * Per-group NVFP4 global scale:  global_scale[g] = 2688 / max|x[rows of g]| (1e-8 for an all-zero group,
 * FLT_MAX for a group without rows), tensor_idx[r] = group of row r (int64 [M], may be NULL).
 * Replaces: mslk/quantize/triton/legacy/global_scale.py:40-230 (calculate_group_max).
 */
int mslk_b200_calculate_group_max(const void *x, int64_t M, int64_t K, int64_t row_stride,
                                  const int64_t *m_sizes, int64_t G, float *global_scale,
                                  int64_t *tensor_idx, void *stream);
int mslk_b200_calculate_group_max_dt(const void *x, int dtype, int64_t M, int64_t K, int64_t row_stride,
                                     const int64_t *m_sizes, int64_t G, float *global_scale, int64_t *tensor_idx,
                                     void *stream);   /* dtype: MSLK_B200_BF16 or MSLK_B200_F16 */

/*
 * Fused SwiGLU + per-row FP8 quantization:  y = x0 * sigmoid(x0) * x1 (fp32),
 *     rmax = min(max(max_k |y|, 1e-12), *scale_ub)        (scale_ub may be NULL)
 *     q[r, k] = e4m3_rn_satfinite(y * (448 / rmax)),  inv_scale[r] = 1 / (448 / rmax).
 * Replaces: mslk/moe/activation.py:72-133 (silu_mul_quant) and its kernel
 *           _mslk_silu_mul_quant (:220-294); sigmoid and the divisions use the same
 *           approximate instructions that kernel lowers to, so outputs agree bit for bit.
 * x0, x1: [T, D] of `dtype` (MSLK_B200_BF16 or MSLK_B200_F16), unit inner stride, row
 * strides stride0 / stride1 in elements.  q: [T, D] bytes contiguous; inv_scale: fp32 [T].
 * valid_token_count (device int32 scalar, may be NULL): rows >= *valid_token_count are
 * neither read nor written.
 */
int mslk_b200_silu_mul_quant(const void *x0, const void *x1, int dtype, int64_t T, int64_t D,
                             int64_t stride0, int64_t stride1, const float *scale_ub,
                             const int *valid_token_count, void *q, float *inv_scale,
                             void *stream);

/*
 * SwiGLU without quantization: y = x0 * sigmoid(x0) * x1, y [T, D] contiguous in the
 * input dtype.  Replaces: mslk/moe/activation.py:25-69 (silu_mul), kernel :181-217.
 */
int mslk_b200_silu_mul(const void *x0, const void *x1, int dtype, int64_t T, int64_t D,
                       int64_t stride0, int64_t stride1, const int *valid_token_count, void *y,
                       void *stream);

/* element type code of int32 tensors, accepted by the scatter-add entry points only */
#define MSLK_B200_I32 3

/*
 * Token gather (MoE dispatch):  out[i, :] = dtype(f32(x[tok[i], :]) * f32(scores[tok[i], exp[i]])), i < a.
 * Replaces: mslk/moe/gather_scatter.py:18-93 (gather_scale_dense_tokens), kernel :431-486.
 * x [T, D] contiguous bf16/fp16; token_indices / expert_indices [a] of 32- or 64-bit integers
 * (`*_index_bits`); scores [T, E] of scores_dtype (MSLK_B200_F32/BF16/F16) with element strides
 * stride_t, stride_e; out [a, D] in the dtype of x.  Rows i >= *valid_token_count (device int32,
 * may be NULL) are skipped.  An index outside [0, T) x [0, E) skips the row and sets bit 0x100
 * of the device status word.
 */
int mslk_b200_gather_scale_dense_tokens(const void *x, int dtype, int64_t T, int64_t D,
                                        const void *token_indices, int token_index_bits,
                                        const void *expert_indices, int expert_index_bits,
                                        const void *scores, int scores_dtype, int64_t E,
                                        int64_t stride_t, int64_t stride_e, int64_t a,
                                        const int *valid_token_count, void *out, void *stream);

/*
 * The same gather fused with per-row FP8 quantization:  v = f32(x[tok[i]]) * score,
 *     rmax = min(max(max_k |v|, 1e-12), *scale_ub),  os = 448 / rmax,
 *     q[i, k] = e4m3_rn_satfinite(v[k] * os),  inv_scale[i] = 1 / os.
 * Replaces: mslk/moe/gather_scatter.py:96-169 (gather_scale_quant_dense_tokens), kernel :537-655
 * (same approximate divisions, so q and inv_scale agree bit for bit).  q [a, D] bytes, inv_scale fp32 [a].
 */
int mslk_b200_gather_scale_quant_dense_tokens(const void *x, int dtype, int64_t T, int64_t D,
                                              const void *token_indices, int token_index_bits,
                                              const void *expert_indices, int expert_index_bits,
                                              const void *scores, int scores_dtype, int64_t E,
                                              int64_t stride_t, int64_t stride_e, int64_t a,
                                              const float *scale_ub, const int *valid_token_count,
                                              void *q, float *inv_scale, void *stream);

/*
 * Token scatter-add (MoE combine):  out_tokens[tok[i], :] += in_tokens[i, :] for i < min(a, *valid_token_count),
 * atomically, in the tensors' dtype (MSLK_B200_BF16 / F16 / F32 / I32; 16-byte vector reductions).
 * Replaces: mslk/moe/gather_scatter.py:172-226 (scatter_add_dense_tokens), kernel :489-526.
 * out_tokens [T, D], in_tokens [a, D] contiguous.  With several contributions per output row the
 * floating-point sum depends on the order the atomics land in, as it does in the reference.
 * An index outside [0, T) skips the row and sets bit 0x200 of the device status word.
 */
int mslk_b200_scatter_add_dense_tokens(void *out_tokens, int64_t T, const void *in_tokens, int dtype,
                                       int64_t a, int64_t D, const void *token_indices,
                                       int token_index_bits, const int *valid_token_count,
                                       void *stream);

/*
 * Scatter-add of expert-parallel padded buffers:  for every stacked row i < sum(token_counts),
 * out_tokens[tok[i], :] += in_tokens[rank(i), i, :], rank(i) = (expert owning row i) / (E / EP).
 * Replaces: mslk/moe/gather_scatter.py:229-282 (scatter_add_padded_tokens), kernel :677-740.
 * in_tokens [EP, T_K, D], token_counts [E] (32- or 64-bit, on the device), token_indices [T_K],
 * out_tokens [T, D].  E % EP == 0, E <= 1024.
 */
int mslk_b200_scatter_add_padded_tokens(const void *in_tokens, int dtype, int64_t EP, int64_t T_K,
                                        int64_t D, const void *token_counts, int count_bits,
                                        int64_t E, const void *token_indices, int token_index_bits,
                                        void *out_tokens, int64_t T, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MSLK_B200_H_ */
