/*
 * nncf_b200 -- C ABI of the B200 (sm_100a) weight-compression kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*; NULL = the legacy default stream).  The caller owns all
 * memory: inputs are read-only unless stated, outputs are caller-allocated device buffers.
 * No entry point allocates or frees device memory, synchronises the device or keeps
 * per-call state.  Return value: 0 on success, a negative NNCFB_E_* code otherwise;
 * nncfb_last_error() returns a human-readable description of the last failure on the
 * calling thread.
 *
 * Each declaration cites the reference interface (nncf 3.2.0, path relative to the
 * reference project root) whose arithmetic it replaces.  "WC" abbreviates
 * src/nncf/quantization/algorithms/weight_compression.
 */
#ifndef NNCF_B200_H_
#define NNCF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NNCFB_ABI_VERSION 2

/* status codes */
#define NNCFB_OK 0
#define NNCFB_E_BAD_ARG (-1)      /* null pointer, bad enum, size <= 0 */
#define NNCFB_E_GROUP_SIZE (-2)   /* reduce %% group_size != 0 (reference: InvalidGroupSizeError) */
#define NNCFB_E_UNSUPPORTED (-3)  /* combination not implemented */
#define NNCFB_E_ALIGNMENT (-4)    /* pointer not aligned as documented */
#define NNCFB_E_CUDA (-5)         /* a CUDA runtime call or launch failed */
#define NNCFB_E_TOO_LARGE (-6)    /* size beyond a documented maximum */
#define NNCFB_E_TIMEOUT (-7)      /* a bounded device-side wait gave up */

/* element types of weights / activations */
#define NNCFB_F32 0
#define NNCFB_F16 1
#define NNCFB_BF16 2
#define NNCFB_I32 3

/* compression modes (same meaning as nncf.parameters.CompressWeightsMode, src/nncf/parameters.py:72-118) */
#define NNCFB_INT8_SYM 0
#define NNCFB_INT8_ASYM 1
#define NNCFB_INT4_SYM 2
#define NNCFB_INT4_ASYM 3
#define NNCFB_NF4 4
#define NNCFB_MXFP4 5
#define NNCFB_FP4 6
#define NNCFB_FP8_E4M3 7
#define NNCFB_MXFP8_E4M3 8

/* layout of codes_out */
#define NNCFB_CODES_NONE 0
#define NNCFB_CODES_BYTE 1   /* one byte per element: int8 (sym), uint8 (asym), format bit pattern (float modes) */
#define NNCFB_CODES_NIBBLE 2 /* 4-bit modes: two codes per byte in flat element order, even index -> low nibble;
                                INT4_SYM codes are stored with the +8 offset of pack_int4 */

/*
 * Arguments of nncfb_quantize.  The weight is viewed as [outer, reduce, inner] (row-major);
 * quantisation parameters are shared by `group_size` consecutive elements along `reduce`
 * (group_size == reduce: per channel).  nn.Linear / nn.Embedding weights have inner == 1.
 * G = reduce / group_size.  All per-group tensors are laid out [outer, G, inner], which is
 * the flat order of the reference's [a1, G, 1, a2] tensors.
 */
typedef struct nncfb_quantize_args {
  const void* weight;     /* device, NNCFB_F32 / F16 / BF16, contiguous */
  int32_t weight_dtype;
  int32_t mode;           /* NNCFB_INT8_SYM ... NNCFB_MXFP8_E4M3 */
  int64_t outer, reduce, inner;
  int64_t group_size;
  const float* pre_scale; /* optional precomputed scale [outer, G, inner]; NULL = compute from the weight */
  const void* pre_zp;     /* optional precomputed zero point [outer, G, inner] (asym modes only) */
  int32_t pre_zp_dtype;   /* NNCFB_I32 or NNCFB_F32 */
  int32_t codes_format;   /* NNCFB_CODES_* */
  void* codes_out;        /* [outer*reduce*inner] bytes, or half that for NNCFB_CODES_NIBBLE; may be NULL */
  float* scale_out;       /* fp32 [outer, G, inner]; may be NULL */
  int32_t* zp_out;        /* int32 [outer, G, inner], asym modes; may be NULL */
  uint16_t* scale_f16_out;/* IEEE fp16 bits of the scale (the decompressor's `_scale` buffer); may be NULL */
  uint8_t* scale_e8m0_out;/* MX modes: biased exponent byte of the power-of-two scale; may be NULL */
  float* values_out;      /* float modes: decoded fp32 grid value per element (the reference's `tensor`); may be NULL */
  float* dq_out;          /* dequantised fp32 weight per element; may be NULL */
  float* sqerr_out;       /* fp32 [outer, G, inner]: sum over the group of (dq - w)^2; may be NULL */
  uint8_t* zp_packed_out; /* asym modes: the zero points as the decompressor stores them (layers.py:1318,1390): one
                             uint8 per group for 8-bit modes; for 4-bit modes two groups per byte in flat group
                             order, even group in the low nibble (pack_uint4 of the zero-point tensor).  4-byte
                             aligned, ((n_groups + 7) / 8) * 4 bytes for 4-bit modes; may be NULL */
} nncfb_quantize_args;

/*
 * Group-wise min/max (or abs-max) reduction, scale / zero-point computation, quantise, clamp,
 * pack and optional dequantise + squared error in ONE pass over the weight.
 *
 * Replaces, bit for bit (fp32 true division, separate zero-point add, round-half-even):
 *   WC/weight_lowering.py:292-326  calculate_integer_quantization_params
 *   src/nncf/quantization/fake_quantize.py:322-350  calculate_scale_zero_point
 *   WC/weight_lowering.py:629-649  _calculate_signed_scale
 *   WC/weight_lowering.py:652-684  _calculate_integer_quantized_weight
 *   WC/weight_lowering.py:451-554  do_integer_quantization / integer_quantize_dequantize_weight
 *   WC/weight_lowering.py:84-128   calculate_float_quantization_params
 *   WC/weight_lowering.py:557-586  _calculate_float_quantized_weight (NF4, E2M1)
 *   WC/fp8_conversion.py:211-228   fp32_to_fp8e4m3
 *   WC/weight_lowering.py:329-374  get_integer_quantization_error (via sqerr_out)
 *   src/nncf/torch/quantization/quantize_functions.py:417-461  pack_uint4 / pack_int4 (NNCFB_CODES_NIBBLE)
 * Alignment: weight, codes_out, values_out, dq_out 16-byte aligned.
 */
int nncfb_quantize(const nncfb_quantize_args* args, void* stream);

/*
 * The per-weight loop of a whole model in as few launches as possible: `items` is a HOST array
 * of n requests.  Consecutive requests that ask for the storage outputs only (codes in their
 * stored format, scale, zero point; integer modes, inner == 1, same mode / dtype / group size)
 * are served by ONE persistent kernel whose descriptor table travels as a kernel parameter;
 * every other request is launched like nncfb_quantize.  Results are identical to n calls of
 * nncfb_quantize.  Replaces the sequential loop of
 * WC/torch_backend.py:442-481 (PTWeightCompressionAlgoBackend.transform_model) and
 * WC/algorithm.py:1198-1211.
 */
int nncfb_quantize_batch(const nncfb_quantize_args* items, int32_t n, void* stream);

/*
 * ScaleEstimation: refined per-group scales for a weight [rows, cols] (groups of `group_size`
 * consecutive columns) from the activation statistics of its input:
 *   importance [cols]        max |X| over the calibration samples (fp32)
 *   x          [cols, n]     per-sample channel means, fp32, row-major (n <= 256)
 * One warp runs the whole sweep of a (row, group): baseline quantisation, `initial_steps`
 * rectifications and `scale_steps` grid points, each scored by mean_n ((W_g - Q_g) X_g)^2
 * (+ weight_penalty * mean (Q - W)^2 when weight_penalty > 0).  Outputs: scale_out fp32 [rows, G],
 * zp_out int32 [rows, G] (asymmetric modes; the zero point of the baseline quantisation).
 * Limits: group_size <= 512 and group_size x n small enough for 200 KiB of shared memory.
 * Replaces WC/scale_estimation.py:160-409 (ScaleEstimation.calculate_quantization_params after
 * process_stats, estimate_scales, get_target_zero_mask).
 */
int nncfb_scale_estimation(const void* weight, int32_t weight_dtype, int64_t rows, int64_t cols, int64_t group_size,
                           int32_t mode, const float* importance, const float* x, int32_t n_samples,
                           int32_t initial_steps, int32_t scale_steps, float weight_penalty, float* scale_out,
                           int32_t* zp_out, void* stream);

/*
 * AWQ alpha grid search for `n_groups` groups of a weight [rows, cols]:
 *   group_index [n_groups]      device int32, group number (column offset / group_size)
 *   group_scale [n_groups, gs]  device fp32, activation magnitudes of the group clipped to
 *                               [quantile(0.1), 100] (WC/awq.py:302-304)
 *   x           [cols, n]       device fp32 per-sample channel means
 *   alphas      [n_alpha]       device fp32 grid (alpha_min + k * step, accumulated like the reference)
 *   prev_w      [cols] or NULL  mean |weight| per channel of the layer the scale is merged into, with
 *                               prev_s = max activation magnitude of that layer, prev_rdim = its
 *                               reduction size and threshold = 0.25 * 65504 (fp16 overflow guard)
 *   scale_io    [cols]          device fp32, holds 1.0 on entry; columns of groups for which a better
 *                               alpha exists receive s^alpha
 * `workspace` is caller-provided scratch of nncfb_awq_workspace_bytes() bytes (per-block partial
 * sums; contents need not be initialised).  Replaces WC/awq.py:243-361 (AWQ._data_aware_step,
 * _clamp_scale).
 */
size_t nncfb_awq_workspace_bytes(int64_t rows, int32_t n_groups, int32_t n_alpha);
int nncfb_awq_search(const void* weight, int32_t weight_dtype, int64_t rows, int64_t cols, int32_t mode,
                     int64_t group_size, const int32_t* group_index, int32_t n_groups, const float* group_scale,
                     const float* x, int32_t n_samples, const float* alphas, int32_t n_alpha, const float* prev_w,
                     float prev_s, float prev_rdim, float threshold, float* scale_io, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * GPTQ Hessian accumulation: hessian [channels, channels] fp32 (device, symmetric) is replaced by
 *   alpha * hessian + beta * X^T X,   X = activation [tokens, channels] (fp32 / fp16 / bf16, channel last).
 * The running form of the reference (H *= n/(n+b); n += b; H += (2/n) X^T X) is alpha = n/(n+b),
 * beta = 2/(n+b) per call.  With allow_tensor_cores != 0 and a 16-bit activation whose channel count is a
 * multiple of 64 (>= 256) the contraction runs on tcgen05 tensor cores (exact 16-bit products, fp32
 * accumulation in tensor memory, operands by TMA); otherwise an fp32 CUDA-core kernel runs.  The
 * tensor-core kernels (this one and the GPTQ trailing update) bound every wait in time (4 s); a launch whose
 * wait ran out stops, frees its tensor memory and raises a per-device sticky flag.  nncfb_hessian_status()
 * (synchronises the stream) returns NNCFB_E_TIMEOUT if any launch on the device gave up since the flag was last
 * read, and clears it: one check after a series of calls sees an error in any of them.  The flag is shared by
 * all streams of the device (a timeout reported after concurrent calls does not say which of them it was); the
 * word the roles of one launch use to stop one another is per launch.  workspace is reserved (may be NULL).
 * Replaces WC/gptq.py:200-242 (GPTQ._calculate_hessian).
 */
int nncfb_hessian_accumulate(float* hessian, int64_t channels, const void* x, int32_t dtype, int64_t tokens,
                             float alpha, float beta, int32_t allow_tensor_cores, void* workspace,
                             size_t workspace_bytes, void* stream);
int nncfb_hessian_status(void* stream);

/*
 * GPTQ blocked column sweep.  weight [rows, cols] fp32 is the tensor-level weight: it is the call's WORKING COPY,
 * updated in place by the trailing updates (pass a clone; its contents after the call are unspecified: on the
 * tensor-core path a block's update of the next block's columns is applied inside that block's sweep and never
 * written back).  hinv [cols, cols] fp32 is the upper Cholesky
 * factor of the inverse damped Hessian.  For every block of `block_size` (<= 128) columns: group parameters
 * at each group start from the tensor-level weight, quantise-dequantise column by column with error feedback
 * inside the block, then weight[:, i2:] -= Err @ hinv[i1:i2, i2:].  Outputs: q_out [rows, cols] fp32
 * dequantised weight, scale_out [rows, G] fp32, zp_out [rows, G] int32 (asymmetric modes).
 * workspace: caller-provided scratch.  nncfb_gptq_workspace_bytes(rows) is the minimum; the trailing update is
 * then an fp32 CUDA-core contraction.  With nncfb_gptq_workspace_bytes_tensor_cores(rows, cols) bytes, and
 * block_size = 128, rows % 8 == 0, cols % 4 == 0, it runs on the tcgen05 tensor cores instead: both fp32
 * operands are split into three bf16 planes and six plane products are accumulated in fp32 in tensor memory
 * (agrees with the fp32 contraction to ~1e-7 relative).  That kernel bounds every wait like the Hessian kernel;
 * nncfb_hessian_status() reports a wait that gave up.  On this path the part of a block's update that the next
 * block does not need yet runs on a stream of the library's own (one non-blocking stream and three events per
 * device and caller stream, created on first use and kept; no device memory), ordered against `stream` by events
 * in both directions: all work is complete, in stream order, when `stream` reaches the end of the call, and the
 * sequence may be captured into a CUDA graph like any fork / join.  Calls on different streams of one device run
 * side by side; calls on the same stream are serialised by a mutex while they enqueue.
 * Replaces WC/gptq.py:297-379 (the loop of GPTQ._quantize_weights).
 */
size_t nncfb_gptq_workspace_bytes(int64_t rows);
size_t nncfb_gptq_workspace_bytes_tensor_cores(int64_t rows, int64_t cols);
int nncfb_gptq_quantize(float* weight, int64_t rows, int64_t cols, const float* hinv, int32_t mode, int64_t group_size,
                        int32_t block_size, float* q_out, float* scale_out, int32_t* zp_out, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * nncfb_gptq_quantize with ScaleEstimation at every group start (GPTQ(scale_estimation=True), WC/gptq.py:319-327):
 * the scale / zero point of a 4-bit integer group come from the candidate search of nncfb_scale_estimation, run on
 * the tensor-level weight of that group as it stands when its block begins.  importance [cols] and x [cols, n_samples]
 * are the layer's statistics after process_stats (WC/activation_stats.py:20-57), as for nncfb_scale_estimation;
 * group_size <= 512.  Other modes ignore the statistics (the reference refines 4-bit integer groups only).
 */
int nncfb_gptq_quantize_se(float* weight, int64_t rows, int64_t cols, const float* hinv, int32_t mode, int64_t group_size,
                           int32_t block_size, const float* importance, const float* x, int32_t n_samples,
                           int32_t initial_steps, int32_t scale_steps, float weight_penalty, float* q_out,
                           float* scale_out, int32_t* zp_out, void* workspace, size_t workspace_bytes, void* stream);

/*
 * nncfb_gptq_quantize for callers that cannot provide scratch memory.  It has no counterpart in the
 * reference.  Who needs it: a program that embeds the library but cannot allocate device memory itself -
 * its runtime handed all of HBM to a private arena at start-up and exposes no allocation hook, or it runs
 * in a loop where cudaMalloc's device-wide synchronisation is forbidden.  Same arguments and results as
 * nncfb_gptq_quantize minus the workspace: the error-column scratch is a fixed 8 MiB array inside the
 * library (held by every GPU that loads the library until the process exits).
 *   - rows <= 16384; larger problems return NNCFB_E_TOO_LARGE (use nncfb_gptq_quantize).
 *   - The first call on a device looks up the array's device address (once per device, with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents (nothing in it needs to be
 *     zero: every value is written before it is read).  Calls whose kernels can overlap on the GPU - other
 *     streams or host threads - race on it: issue them on one stream or serialise them.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 */
int nncfb_gptq_quantize_noalloc(float* weight, int64_t rows, int64_t cols, const float* hinv, int32_t mode,
                                int64_t group_size, int32_t block_size, float* q_out, float* scale_out, int32_t* zp_out,
                                void* stream);

/*
 * Per-channel statistics of an activation [tokens, channels] (channel last) in one pass; every
 * output is optional (NULL):
 *   mean_out    [channels] in the activation's dtype (fp32 accumulate, one rounding)
 *   var_out     [channels] fp32 population variance
 *   absmax_out  [channels] fp32 max |x|
 *   sumsq_out   [channels] fp64 sum of squares
 * Replaces src/nncf/common/tensor_statistics/collectors.py:512-540 (MeanReducer,
 * MeanVarianceReducer, MaxVarianceReducer, MeanAbsMaxReducer) and :924-936 (HAWQ trace input).
 */
int nncfb_channel_stats(const void* x, int32_t dtype, int64_t tokens, int64_t channels, void* mean_out, float* var_out,
                        float* absmax_out, double* sumsq_out, void* stream);

/*
 * fp32-faithful matrix product on the tcgen05 tensor cores:
 *   c[m, n] (row stride ldc) = (accumulate ? c : 0) + alpha * a[m, k] @ b      (all fp32, row-major, device)
 * with b given as [k, n] or, with transpose_b != 0, as [n, k] (c = a b^T).
 * Both operands are split into three bf16 planes (hi + mid + lo = the fp32 value to 2^-27) and the six plane
 * products down to 2^-24 are accumulated in fp32 in tensor memory, smallest first, by the kernel that also does
 * the GPTQ trailing update; c is updated by a bulk tensor reduction (never read into the SM).  Agrees with an
 * fp32 product to about 1e-6 relative.  Needs k % 64 == 0, ldc % 4 == 0, c and workspace 16-byte aligned;
 * workspace >= nncfb_gemm_f32_workspace_bytes(m, n, k) holds the operand planes.  Returns NNCFB_E_UNSUPPORTED
 * (nothing launched) when the shape does not qualify.
 * Used for the dense products inside the inverse factor of the GPTQ Hessian (the trailing updates of a blocked
 * Cholesky factorisation and the triangular inverse), which the reference obtains from fns.linalg.cholesky /
 * cholesky_inverse (WC/gptq.py:293-295).
 */
size_t nncfb_gemm_f32_workspace_bytes(int64_t m, int64_t n, int64_t k);
int nncfb_gemm_f32(const float* a, int64_t lda, const float* b, int64_t ldb, int32_t transpose_b, float* c, int64_t ldc,
                   int64_t m, int64_t n, int64_t k, float alpha, int32_t accumulate, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * Decompression of stored weights in one pass: codes (nibble-packed for 4-bit modes, bytes for 8-bit) +
 * per-group scale (+ zero point) -> n_elements values of out_dtype (NNCFB_F32 / F16 / BF16), groups of
 * `group_size` consecutive elements (any size; multiples of 8 with a 16-byte aligned output and 8-byte aligned
 * codes take the vector kernel, everything else an element-per-thread kernel with the same arithmetic).
 *   integer modes: scale = fp16 [n_groups] (the decompressor's `_scale` buffer); zero_point = uint8 per group
 *                  (INT8_ASYM) or nibble-packed in flat group order (INT4_ASYM), NULL for symmetric modes;
 *                  arithmetic in fp16 exactly as the reference: (x.f16 - zp.f16) * scale.f16, then the cast;
 *   NF4 / FP4 / FP8_E4M3: scale = fp32 [n_groups];   MXFP4 / MXFP8_E4M3: scale = E8M0 bytes [n_groups].
 * Replaces src/nncf/torch/quantization/layers.py:1334-1338,1364-1368,1406-1416,1453-1460 (the forward of the
 * INT8/INT4 weight decompressors) and src/nncf/torch/quantization/quantize_functions.py:389-414,436-473.
 */
int nncfb_decompress(const void* codes, int32_t mode, int64_t n_elements, int64_t group_size, const void* scale,
                     const void* zero_point, void* out, int32_t out_dtype, void* stream);

/*
 * Nibble-pack n byte codes (n even) in flat order: out[i] = (in[2i] & 15) | (in[2i+1] << 4);
 * `add` is added to every code first (8 for signed int4 codes).
 * Replaces src/nncf/torch/quantization/quantize_functions.py:417-461 pack_uint4 / pack_int4.
 */
int nncfb_pack_nibbles(const void* codes, int64_t n, int32_t add, uint8_t* packed_out, void* stream);

/* Inverse of nncfb_pack_nibbles: out[2i] = (in[i] & 15) - sub, out[2i+1] = (in[i] >> 4) - sub (int8 out).
 * Replaces quantize_functions.py:436-444,464-473 unpack_uint4 / unpack_int4. */
int nncfb_unpack_nibbles(const uint8_t* packed, int64_t n_bytes, int32_t sub, int8_t* codes_out, void* stream);

/* Exhaustive-style self check of the in-kernel fp32 division against IEEE division on n
 * pseudo-random operand pairs drawn from `seed`; writes the number of mismatches to
 * *mismatch_out (device int64).  Test hook, no reference counterpart. */
int nncfb_selftest_division(int64_t n, uint64_t seed, int64_t* mismatch_out, void* stream);

/* Self test of the bounded waits of the tensor-core kernels: runs the Hessian kernel on x_bf16
 * [tokens, channels] (256 <= channels <= 1024, multiple of 64; 64 <= tokens <= 4096) with a 1 ms limit per
 * wait and a producer that leaves out the last pipeline stage of every tile, so that the MMA role's wait runs
 * out; every role then stops, tensor memory is released and the kernel returns with `hessian` partly written.
 * Nothing traps or faults.  nncfb_hessian_status() afterwards returns NNCFB_E_TIMEOUT (and clears the flag);
 * later launches are unaffected.  Test hook, no reference counterpart. */
int nncfb_selftest_bounded_wait(float* hessian, int64_t channels, const void* x_bf16, int64_t tokens, void* stream);

/* Library information */
int nncfb_abi_version(void);
const char* nncfb_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* NNCF_B200_H_ */
