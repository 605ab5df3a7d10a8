/*
 * actnn_b200 -- C ABI of the B200 (sm_100a) activation compress / decompress kernels.
 *
 * Drop-in boundary for the native extensions of ucbrise/actnn
 * (actnn/actnn/cpp_extension/{minimax,quantization,calc_precision}*).  The reference
 * binds those as pybind11 torch extensions that take and return torch::Tensor; this
 * library exposes the same operations one level lower: plain device pointers, explicit
 * sizes, a dtype tag and a cudaStream_t.  A binding layer (python/ctypes here, or the
 * reference's own .cc files) allocates the outputs and forwards the pointers.
 *
 * Conventions
 *   - every pointer is a device pointer on the current device unless stated otherwise;
 *   - no entry point allocates, frees or synchronises; all work is queued on `stream`;
 *   - every entry point returns an actnn_status (0 = queued successfully); arguments are
 *     validated on the host before anything is launched;
 *   - activations are viewed as [N, G, group_size] (sample, group, element), contiguous,
 *     each sample zero-padded to a whole number of groups by the caller, as the
 *     reference's schemes do (actnn/actnn/qscheme.py:61-71);
 *   - `dtype` is the element type of the activation; per-group statistics (min, max,
 *     scale) carry `stat_dtype`, which equals `dtype` except that float32 activations may
 *     keep bfloat16 statistics (the reference's storage format, actnn/actnn/ops.py:115-116);
 *   - the arithmetic is the reference's "simulate" branch (actnn/actnn/ops.py:23-41,56-57)
 *     with every intermediate rounded to `dtype`, so codes and packed bytes are bit-exact
 *     against it for the same rounding noise;
 *   - rounding noise: pass `noise` (device array, same shape and dtype as the activation,
 *     values in [-0.5, 0.5]) to inject it, or NULL to draw it in registers from
 *     Philox4x32-10 keyed by (seed, offset); actnn_noise_fill() materialises exactly that
 *     stream.  `stochastic == 0` rounds to nearest without noise.
 *   - a NaN input yields some valid code (0 or the largest); it never corrupts its neighbours.
 */
#ifndef ACTNN_B200_H_
#define ACTNN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* actnn_stream_t;        /* == cudaStream_t */

typedef enum {
  ACTNN_F32 = 0,
  ACTNN_F16 = 1,
  ACTNN_BF16 = 2
} actnn_dtype;

typedef enum {
  ACTNN_OK = 0,
  ACTNN_ERR_NULL = 1,         /* a required pointer is NULL */
  ACTNN_ERR_DTYPE = 2,        /* dtype / stat_dtype not supported by this entry point */
  ACTNN_ERR_SHAPE = 3,        /* negative size, size overflow, unsupported group size */
  ACTNN_ERR_BITS = 4,         /* bit width outside the supported set */
  ACTNN_ERR_ALIGN = 5,        /* pointer not aligned for vector access */
  ACTNN_ERR_ARG = 6,          /* any other invalid argument (e.g. stochastic rounding off where the reference requires it) */
  ACTNN_ERR_LAUNCH = 7,       /* the CUDA runtime refused the launch; see cudaGetLastError() */
  ACTNN_ERR_CAPACITY = 8      /* problem larger than a fixed internal buffer */
} actnn_status;

/* Human-readable text for a status code (static storage). */
const char* actnn_status_string(int status);
/* Library ABI version, bumped on any signature change. */
int actnn_abi_version(void);

/* ------------------------------------------------------------------------------------
 * Per-group min / max.
 * Replaces: minimax(data) -> (min, max), actnn/actnn/cpp_extension/minimax.cc:7-11 and
 * minimax_cuda_kernel.cu:23-89.  data[rows, cols] -> mn[rows], mx[rows], all `dtype`.
 * The reference requires cols % 32 == 0 && cols > 32; so does this.  cols == 256 takes
 * the vectorised path (one warp per row, 128/256-bit loads).
 */
int actnn_minimax(const void* data, void* mn, void* mx, int64_t rows, int64_t cols,
                  int dtype, actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Mixed-precision bit stream (per-sample bit widths, int32 words).
 * Layout (actnn/actnn/cpp_extension/quantization_cuda_kernel.cu:51-79): the block of
 * (sample n, group g) starts at word (P[n-1]*G*gs + bits[n]*g*gs) / 32, P the inclusive
 * prefix sum of bits; bit i of element d sits in word (d*b+i) % W at bit (d*b+i) / W,
 * W = gs*b/32.
 *
 * actnn_bits_prefix: word_offsets[n] = first word of sample n, word_offsets[N] = total
 * words.  Replaces the torch::cumsum + .item() of quantization_cuda_kernel.cu:97-98 /
 * :182 without a host sync.  One thread block; N <= 2^20.
 */
int actnn_bits_prefix(const int32_t* bits, int64_t N, int64_t G, int64_t group_size,
                      int64_t* word_offsets, actnn_stream_t stream);

/* Replaces: pack_mixed_precision(data, min, max, bits, stochastic) -> (packed, scale),
 * actnn/actnn/cpp_extension/quantization.cc:46-57, quantization_cuda_kernel.cu:37-142.
 * data[N,G,gs], mn/mx[N,G] in `dtype`; bits[N] in 1..8; word_offsets from
 * actnn_bits_prefix; writes packed (word_offsets[N] words) and scale[N,G] (`stat_dtype`).
 * If mn_out is not NULL the minimum is also re-written there in `stat_dtype`.
 * group_size must be 256. */
int actnn_pack_mixed(const void* data, const void* mn, const void* mx, const int32_t* bits,
                     const int64_t* word_offsets, int32_t* packed, void* scale, void* mn_out,
                     int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                     int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                     actnn_stream_t stream);

/* Replaces: unpack_mixed_precision(data, bits, scale, min, N, num_groups, group_size),
 * actnn/actnn/cpp_extension/quantization.cc:59-73, quantization_cuda_kernel.cu:145-205.
 * out[N,G,gs] in `dtype` = code / scale + min. */
int actnn_unpack_mixed(const int32_t* packed, const int32_t* bits, const int64_t* word_offsets,
                       const void* scale, const void* mn, void* out,
                       int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                       actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Single-precision (uniform bit width) byte stream, int8.
 * Layout (quantization_cuda_kernel.cu:236-257): byte (no*G + g)*gs + d holds samples
 * no*wpt + ni (wpt = 8 / bits) at bit offset ni*bits; length
 * bits * N_round * G * gs / 8 + 1 with N rounded up to a multiple of wpt (the trailing
 * byte is written as zero).  bits in {1, 2, 4, 8}; group_size must be 256.
 *
 * Replaces: pack_single_precision(data, min, max, bits, stochastic) -> (packed, scale),
 * actnn/actnn/cpp_extension/quantization.cc:77-87, quantization_cuda_kernel.cu:225-330. */
int actnn_pack_single(const void* data, const void* mn, const void* mx, int bits,
                      int8_t* packed, void* scale, void* mn_out,
                      int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                      int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                      actnn_stream_t stream);

/* Replaces: unpack_single_precision(data, bits, scale, min, N, num_groups, group_size),
 * actnn/actnn/cpp_extension/quantization.cc:89-102, quantization_cuda_kernel.cu:333-405. */
int actnn_unpack_single(const int8_t* packed, int bits, const void* scale, const void* mn,
                        void* out, int64_t N, int64_t G, int64_t group_size, int dtype,
                        int stat_dtype, actnn_stream_t stream);

/* Fused single pass: per-group min/max + stochastic rounding + pack, reading the
 * activation once.  Replaces the sequence minimax -> pack_single_precision that
 * no_scheme_compute_quantization_bits + quantize_and_pack issue for uniform-bit layers
 * (actnn/actnn/ops.py:77-96, 44-48).  Writes packed, scale[N,G] and mn[N,G]
 * (`stat_dtype`); mx_out may be NULL. */
int actnn_compress_single(const void* data, int bits, int8_t* packed, void* scale, void* mn_out,
                          void* mx_out, int64_t N, int64_t G, int64_t group_size, int dtype,
                          int stat_dtype, int stochastic, const void* noise, uint64_t seed,
                          uint64_t offset, actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Bit allocation on the device.
 *
 * actnn_range_sqr: per-sample sensitivity base, Range_sqr[n] =
 * float(norm_T(mx[n,:] - mn[n,:]))^2 * (group_size / num_pixels), the expression of
 * actnn/actnn/qscheme.py:80 / qbnscheme.py:42; then C[n] = coeff * Range_sqr[n] *
 * (grad_scale ? *grad_scale : 1) in float32 (qscheme.py:84).  grad_scale is a device
 * pointer to one float or NULL. */
int actnn_range_sqr(const void* mn, const void* mx, int64_t N, int64_t G, int stat_dtype,
                    float range_factor, float coeff, const float* grad_scale, float* C,
                    actnn_stream_t stream);

/* Per-sample squared gradient norm, out[n] = sum_f float(grad[n, f])^2.
 * Replaces the torch expression of QScheme.set_scale, actnn/actnn/qscheme.py:47-55
 * (grad.view(N, -1).float().norm(dim=1).square()) with one read of the gradient. */
int actnn_sample_sumsq(const void* grad, float* out, int64_t N, int64_t F, int dtype,
                       actnn_stream_t stream);

/* Replaces: calc_precision(b, C, w, target) -> b,
 * actnn/actnn/cpp_extension/calc_precision.cc:9-50 (a CPU priority queue there; here a
 * weighted radix select over the (initial_bits-1)*N candidate decrements, identical
 * results including tie-breaks).  C[N] float32, w[N] int32 or NULL (all ones),
 * b_out[N] int32, every entry starting from `initial_bits` (1..15; 1 leaves nothing to remove).  If word_offsets is
 * not NULL it receives what actnn_bits_prefix would (needs G, group_size).
 * N <= 2^20.  Small unit-weight problems run in one thread block.  `workspace` (optional,
 * actnn_calc_precision_workspace() bytes, 8-byte aligned, contents unspecified before and
 * after) lets weighted or large problems without word offsets run as a sequence of
 * multi-block launches instead of one block; pass NULL / 0 to do without. */
int64_t actnn_calc_precision_workspace(void);
int actnn_calc_precision(const float* C, const int32_t* w, int64_t N, int initial_bits,
                         double target, int32_t* b_out, int64_t* word_offsets,
                         int64_t G, int64_t group_size, void* workspace, int64_t workspace_bytes,
                         actnn_stream_t stream);

/* The adaptive compress of one activation as one call: per-group min/max, sensitivities,
 * greedy allocation at `target` total bits, scale + stochastic rounding + mixed-precision
 * pack.  Replaces the sequence QScheme.compute_quantization_bits -> quantize_and_pack,
 * actnn/actnn/qscheme.py:57-94 and actnn/actnn/ops.py:44-48 (there: ~15 launches, two host
 * copies and a CPU heap).  Outputs: packed (the caller sizes it for the bit total the greedy
 * will reach: min(initial_bits*N, max(target, N)) * G * group_size / 32 words), scale and
 * mn_out [N,G] (`stat_dtype`), bits_out [N], word_offsets_out [N+1], C_out [N] (float32
 * sensitivities, kept by the caller for the per-layer allocation).
 * `workspace` is caller-provided scratch of at least actnn_compress_mixed_workspace(N, G,
 * dtype) bytes, 256-byte aligned; it holds the per-group min / max between the kernels and
 * its content afterwards is unspecified.  Arguments otherwise as in actnn_range_sqr,
 * actnn_calc_precision and actnn_pack_mixed. */
int64_t actnn_compress_mixed_workspace(int64_t N, int64_t G, int dtype);
int actnn_compress_mixed(const void* data, int32_t* packed, void* scale, void* mn_out,
                         int32_t* bits_out, int64_t* word_offsets_out, float* C_out,
                         void* workspace, int64_t workspace_bytes, int64_t N, int64_t G,
                         int64_t group_size, int dtype, int stat_dtype, float range_factor,
                         float coeff, const float* grad_scale, int initial_bits, double target,
                         int stochastic, const void* noise, uint64_t seed, uint64_t offset,
                         actnn_stream_t stream);

/* actnn_compress_mixed for callers that cannot hand over scratch memory.  (This entry point
 * has no counterpart in the reference.)
 * Who needs it: code that only works with pointers it was given -- a plug-in of a host
 * framework that owns all device memory and offers no allocator, or a job whose device
 * memory was planned out in advance so that one more cudaMalloc may fail or upset the plan.
 * Same arguments and results as actnn_compress_mixed without `workspace`: the per-group
 * min / max go to an array of actnn_compress_mixed_static_capacity() bytes (4 MiB + 256) that is
 * part of the library image, i.e. resident on every GPU that loads the library until the
 * process ends.  Limits and rules:
 *   - actnn_compress_mixed_workspace(N, G, dtype) must not exceed the capacity (N*G up to
 *     1 Mi groups of 16-bit data, 512 Ki of float32); larger problems return
 *     ACTNN_ERR_CAPACITY and nothing is launched;
 *   - the first call on a device looks up the array's device address (with that device
 *     current); make that first call before any stream capture begins;
 *   - every call on a device uses the same array and leaves its last contents behind (no
 *     part of it needs clearing: each call overwrites what it reads); two calls that may
 *     overlap on the GPU (different streams) race on it -- serialise them;
 *   - it never calls cudaMalloc, cudaFree or any allocating routine. */
int64_t actnn_compress_mixed_static_capacity(void);
int actnn_compress_mixed_static(const void* data, int32_t* packed, void* scale, void* mn_out,
                                int32_t* bits_out, int64_t* word_offsets_out, float* C_out,
                                int64_t N, int64_t G, int64_t group_size, int dtype, int stat_dtype,
                                float range_factor, float coeff, const float* grad_scale,
                                int initial_bits, double target, int stochastic, const void* noise,
                                uint64_t seed, uint64_t offset, actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Batch-norm statistics and the codec's per-group min / max from ONE read of x.
 * Replaces, for a quantized batch norm in training mode, the pair of reads the reference
 * makes: the statistics inside at::cudnn_batch_norm (backward_func.cc:87, called at
 * actnn/actnn/ops.py:456-458; torch.batch_norm_stats at ops.py:515 for the synchronised
 * layer) and the min / max of QBNScheme.compute_quantization_bits (qbnscheme.py:28-40).
 *   x           [N, C, HW] contiguous (NCHW), dtype float32 / float16 / bfloat16
 *   mn, mx      [N * C * HW / 256] in x's dtype: min / max of every 256-element group of the
 *               flattened samples (what actnn_minimax returns for the same tensor)
 *   save_mean, save_invstd  float32 [C]; running_mean / running_var (may be NULL) are updated
 *               with `momentum` exactly as actnn_batch_norm_forward does
 *   weight, bias  only used to fill the coefficients kept in the workspace; may be NULL
 * Geometry: HW % 8 == 0, HW >= 256 and C * HW % 256 == 0 (every layer of a ResNet down to
 * 16x16 maps); anything else returns ACTNN_ERR_SHAPE and the caller takes the two-read path.
 * actnn_batch_norm_stats_minimax_workspace returns the scratch bytes (-1: unsupported). */
int64_t actnn_batch_norm_stats_minimax_workspace(int64_t N, int64_t C, int64_t HW);
int actnn_batch_norm_stats_minimax(const void* x, void* mn, void* mx, const float* weight, const float* bias,
                                   float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                                   int64_t N, int64_t C, int64_t HW, double momentum, double eps, int dtype,
                                   void* workspace, int64_t workspace_bytes, actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * actnn_compress_mixed for an activation whose per-group min / max are already known (from
 * actnn_batch_norm_stats_minimax or actnn_minimax): sensitivities, greedy allocation and pack,
 * i.e. QBNScheme.compute_quantization_bits from its line qbnscheme.py:42 on, followed by
 * pack_mixed_precision (quantization.cc:46-57).  `mn` / `mx` must be the true group extrema.
 * `ticket_workspace`: 256 bytes of scratch, 256-byte aligned.  Other arguments as
 * actnn_compress_mixed. */
int actnn_compress_mixed_prestat(const void* data, const void* mn, const void* mx, int32_t* packed, void* scale,
                                 void* mn_out, int32_t* bits_out, int64_t* word_offsets_out, float* C_out,
                                 void* ticket_workspace, int64_t N, int64_t G, int64_t group_size, int dtype,
                                 int stat_dtype, float range_factor, float coeff, const float* grad_scale,
                                 int initial_bits, double target, int stochastic, const void* noise, uint64_t seed,
                                 uint64_t offset, actnn_stream_t stream);

/* actnn_compress_mixed_prestat (same replaced reference code: qbnscheme.py:42-52, quantization.cc:46-57) with a
 * ticket word that the caller keeps for this purpose only: zero before the first call, left at zero by every
 * call, touched by nothing else, used by one stream at a time.  The per-call clear of the ticket is skipped. */
int actnn_compress_mixed_prestat_kept(const void* data, const void* mn, const void* mx, int32_t* packed, void* scale,
                                      void* mn_out, int32_t* bits_out, int64_t* word_offsets_out, float* C_out,
                                      void* ticket_workspace, int64_t N, int64_t G, int64_t group_size, int dtype,
                                      int stat_dtype, float range_factor, float coeff, const float* grad_scale,
                                      int initial_bits, double target, int stochastic, const void* noise,
                                      uint64_t seed, uint64_t offset, actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Mask ops.  The saved mask is 1 bit per element: bit (e % 8) of byte e / 8, padded to
 * whole int32 words (mask_words = ceil(numel / 32)).
 *
 * Replaces: act_quantized_relu forward / backward,
 * actnn/actnn/cpp_extension/quantization.cc:106-124, quantization_cuda_kernel.cu:411-508. */
int actnn_relu_forward(const void* x, void* y, int32_t* mask, int64_t numel, int dtype,
                       actnn_stream_t stream);

/* The same pass, which also leaves the min and the max of every 256 consecutive OUTPUTS in mn[g] / mx[g]
 * (g = element / 256; numel % 256 == 0), bit-identical to actnn_minimax(y).  The layer that consumes y
 * (a convolution: actnn/actnn/ops.py:99-118 quantizes its input with QScheme.compute_quantization_bits,
 * qscheme.py:57-94, whose first step is that min / max pass) can then compress it with
 * actnn_compress_mixed_prestat, i.e. without reading y once more for the ranges. */
int actnn_relu_forward_minimax(const void* x, void* y, int32_t* mask, void* mn, void* mx, int64_t numel,
                               int dtype, actnn_stream_t stream);
int actnn_relu_backward(const void* grad_out, const int32_t* mask, void* grad_in,
                        int64_t numel, int dtype, actnn_stream_t stream);

/* Replaces: act_quantized_dropout forward / backward,
 * actnn/actnn/cpp_extension/quantization.cc:128-148, quantization_cuda_kernel.cu:514-627.
 * keep = u > p with u uniform in (0, 1] from Philox (seed, offset), or from the injected
 * float32 array `u`; y = keep ? x / (1 - p) : 0. */
int actnn_dropout_forward(const void* x, void* y, int32_t* mask, int64_t numel, float p,
                          int dtype, const float* u, uint64_t seed, uint64_t offset,
                          actnn_stream_t stream);
int actnn_dropout_backward(const void* grad_out, const int32_t* mask, void* grad_in,
                           int64_t numel, float p, int dtype, actnn_stream_t stream);
/* The uniforms actnn_dropout_forward draws for (seed, offset), as float32. */
int actnn_dropout_uniform_fill(float* u, int64_t numel, uint64_t seed, uint64_t offset,
                               actnn_stream_t stream);

/* Replaces: act_quantized_max_pool2d forward / backward,
 * actnn/actnn/cpp_extension/quantization.cc:152-196, quantization_cuda_kernel.cu:633-754.
 * NCHW; saves the window-local arg-max kh*KW + kw as int8 per output; KH*KW < 16 as in
 * the reference.  Backward gathers (each input sums the windows that selected it), so
 * grad_in needs no zero fill and the result is deterministic. */
int actnn_max_pool2d_forward(const void* x, void* y, int8_t* idx, int64_t N, int64_t C,
                             int64_t H, int64_t W, int KH, int KW, int SH, int SW, int PH,
                             int PW, int DH, int DW, int dtype, actnn_stream_t stream);
int actnn_max_pool2d_backward(const void* grad_out, const int8_t* idx, void* grad_in,
                              int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW,
                              int SH, int SW, int PH, int PW, int DH, int DW, int dtype,
                              actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Training-mode batch normalisation of an NCHW tensor viewed as [N, C, HW] (HW = 1 for a
 * [N, C] input).  Replaces the cuDNN calls the reference's quantized batch-norm operator
 * makes: ext_backward_func.cudnn_batch_norm / cudnn_batch_norm_backward, re-exported at
 * actnn/actnn/cpp_extension/backward_func.cc:87-88 and called at actnn/actnn/ops.py:457-458
 * and actnn/actnn/ops.py:492-493.  Same results (batch statistics with the biased variance,
 * running statistics updated with `momentum` and the unbiased variance, save_mean and
 * save_invstd = 1/sqrt(var + eps) for backward); statistics, weight, bias and their
 * gradients are float32 whatever `dtype` is.  weight / bias NULL mean 1 / 0;
 * running_mean / running_var NULL skip the update; grad_in / grad_weight / grad_bias NULL
 * skip that output.  `workspace` holds per-channel partial sums:
 * actnn_batch_norm_workspace(N, C, HW) bytes for the current device, 16-byte aligned, its
 * contents need not be kept between calls.  Sums are added in a fixed order, so equal
 * inputs give equal bits. */
int64_t actnn_batch_norm_workspace(int64_t N, int64_t C, int64_t HW);
int actnn_batch_norm_forward(const void* x, const float* weight, const float* bias,
                             float* running_mean, float* running_var, void* y, float* save_mean,
                             float* save_invstd, int64_t N, int64_t C, int64_t HW, double momentum,
                             double eps, int dtype, void* workspace, int64_t workspace_bytes,
                             actnn_stream_t stream);
int actnn_batch_norm_backward(const void* x, const void* grad_out, const float* weight,
                              const float* save_mean, const float* save_invstd, void* grad_in,
                              float* grad_weight, float* grad_bias, int64_t N, int64_t C, int64_t HW,
                              int dtype, void* workspace, int64_t workspace_bytes,
                              actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * The four halves of a batch norm whose statistics are combined across ranks in between.
 * Replace the ATen operators the reference's synchronised batch norm calls: batch_norm_stats
 * (actnn/actnn/ops.py:515), batch_norm_elemt (ops.py:554), batch_norm_backward_reduce
 * (ops.py:570-577) and batch_norm_backward_elemt (ops.py:594-603).  Same tensors and meanings as those
 * operators: `mean` / `invstd` are float32 [C]; `sum_dy` = sum of grad_out, `sum_dy_xmu` = sum of
 * grad_out * (x - mean), `grad_weight` = sum_dy_xmu * invstd (sum_dy doubles as grad_bias);
 * `counts` = float32 device array of every rank's elements per channel (summed on the device,
 * so no host read is needed).  y of actnn_batch_norm_forward may be
 * NULL (statistics only); that is what actnn_batch_norm_stats calls.  Workspace as above
 * (the element-wise halves use its first 16 * C bytes). */
int actnn_batch_norm_stats(const void* x, float* mean, float* invstd, int64_t N, int64_t C,
                           int64_t HW, double eps, int dtype, void* workspace,
                           int64_t workspace_bytes, actnn_stream_t stream);
int actnn_batch_norm_elemt(const void* x, const float* weight, const float* bias,
                           const float* mean, const float* invstd, void* y, int64_t N, int64_t C,
                           int64_t HW, int dtype, void* workspace, int64_t workspace_bytes,
                           actnn_stream_t stream);
int actnn_batch_norm_backward_reduce(const void* x, const void* grad_out, const float* weight,
                                     const float* mean, const float* invstd, float* sum_dy,
                                     float* sum_dy_xmu, float* grad_weight, int64_t N, int64_t C,
                                     int64_t HW, int dtype, void* workspace,
                                     int64_t workspace_bytes, actnn_stream_t stream);
int actnn_batch_norm_backward_elemt(const void* x, const void* grad_out, const float* weight,
                                    const float* mean, const float* invstd, const float* sum_dy,
                                    const float* sum_dy_xmu, const float* counts, int64_t n_counts,
                                    void* grad_in, int64_t N, int64_t C, int64_t HW, int dtype,
                                    void* workspace, int64_t workspace_bytes, actnn_stream_t stream);

/* ------------------------------------------------------------------------------------
 * How many bulk-copy waits gave up on the current device since the library was loaded.
 * The opt-in staged pack kernels (environment ACTNN_STAGED_PACK=1) copy their inputs into
 * shared memory with the bulk-copy engine and bound every wait on the completion barrier;
 * a warp whose wait runs out stops and leaves its outputs unwritten.  Zero in every
 * healthy run; reading it synchronises with the device.  No counterpart in the reference. */
int actnn_bulk_wait_failures(uint32_t* count);

/* ------------------------------------------------------------------------------------
 * How many four-group bundles actnn_pack_mixed / actnn_compress_mixed met, on the current
 * device since the library was loaded, whose per-sample width was outside 1..8: nothing is
 * written for such a bundle (the widths live on the device, so the entry point itself cannot
 * refuse them without a synchronisation).  Zero in every healthy run; reading it synchronises
 * with the device.  The reference accepts any width its caller passes
 * (quantization_cuda_kernel.cu:94-142) and has no such check. */
int actnn_bad_width_bundles(uint32_t* count);

/* ------------------------------------------------------------------------------------
 * The rounding noise the pack kernels draw for (seed, offset) when `noise == NULL`,
 * written as a [numel] array of `dtype` indexed like the padded [N, G, 256] activation.
 * No counterpart in the reference (it draws cuRAND numbers it cannot replay); exists so
 * that a CPU oracle can be fed the identical noise. */
int actnn_noise_fill(void* noise, int64_t numel, int dtype, uint64_t seed, uint64_t offset,
                     actnn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif  /* ACTNN_B200_H_ */
