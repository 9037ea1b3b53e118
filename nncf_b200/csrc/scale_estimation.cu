// ScaleEstimation: the whole candidate-scale sweep of one (output channel, group) pair in one kernel.
//
// Restates ScaleEstimation.calculate_quantization_params of the reference
// (src/nncf/quantization/algorithms/weight_compression/scale_estimation.py:160-409) after its
// `process_stats` step.  The reference runs 1 + initial_steps + scale_steps rounds, each a chain
// of whole-tensor operations (quantise, dequantise, batched matmul [G, out, gs] x [G, gs, N], mean,
// masked select): about a hundred passes over an fp32 copy of the weight.  Here one warp owns one
// (row, group): its weights, importances and targets stay in registers, the group's activation
// slice X_g [gs, N] is staged once per block in shared memory and shared by all rows of the block,
// and every candidate is scored without touching HBM again.  The weight is read exactly once.
//
// Arithmetic follows the reference step by step (true fp32 divisions, round half to even, the
// `> best` comparison that keeps the incumbent on ties).  Sums (importance normalisation, the
// projections on X, means) are fp32 like the reference's but accumulate in a different order, so
// a candidate whose score ties with the incumbent to the last bit may resolve differently.
#include <algorithm>

#include "quantize_kernels.cuh"

namespace nncfb {

struct SEArgs {
  const void* weight;   // [rows, cols] contiguous, groups along cols
  const float* imp;     // [cols] importance s (max |X| over samples)
  const float* x;       // [cols, n] fp32, row-major
  float* scale_out;     // [rows, G]
  int32_t* zp_out;      // [rows, G] (asym) or null
  int64_t rows, cols;
  int64_t ld;           // elements between weight rows (cols for a contiguous weight; larger for a column slice)
  int64_t out_ld;       // groups per row of scale_out / zp_out (cols / gs unless writing into a wider table)
  int gs, n, np;        // group size, samples, samples padded to a multiple of 64
  int initial_steps, scale_steps;
  float weight_penalty;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// out[c] (c = 0 .. np/64*2 - 1 per lane: columns 2*lane, 2*lane+1 of every 64-column chunk)
// = sum_i v[i] * X[i, col], i ascending.  v is read from the warp's shared buffer.
template <int MAXC>
__device__ __forceinline__ void project(const float* __restrict__ vbuf, const float* __restrict__ xs, int gs, int np,
                                        int lane, float (&acc)[MAXC][2]) {
  const int chunks = np >> 6;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) acc[c][0] = acc[c][1] = 0.0f;
  for (int i = 0; i < gs; i += 4) {
    const float4 d = *reinterpret_cast<const float4*>(vbuf + i);
    const float dv[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float* row = xs + static_cast<size_t>(i + k) * np + 2 * lane;
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        if (c < chunks) {
          const float2 xv = *reinterpret_cast<const float2*>(row + 64 * c);
          acc[c][0] = __fmaf_rn(dv[k], xv.x, acc[c][0]);
          acc[c][1] = __fmaf_rn(dv[k], xv.y, acc[c][1]);
        }
      }
    }
  }
}

constexpr int kSeMaxChunks = 4;   // up to 256 samples
constexpr int kSeRowsPerWarp = 8;

template <typename SrcT, int MODE, int EPL>
__global__ void __launch_bounds__(256) scale_estimation_kernel(const SEArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int gs = a.gs, np = a.np;
  const int gs4 = (gs + 3) & ~3;               // projection walks the group four elements at a time
  float* xs = smem;                            // [gs4, np]
  float* vbufs = smem + static_cast<size_t>(gs4) * np;  // [8 warps][gs4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* vbuf = vbufs + warp * gs4;
  const int64_t G = a.cols / gs;
  const int64_t g = blockIdx.y;
  const SrcT* __restrict__ wsrc = reinterpret_cast<const SrcT*>(a.weight);

  // stage X_g (zero padded to np columns and gs4 rows)
  for (int idx = threadIdx.x; idx < gs4 * np; idx += blockDim.x) {
    const int i = idx / np, c = idx - i * np;
    xs[idx] = (i < gs && c < a.n) ? a.x[(g * gs + i) * a.n + c] : 0.0f;
  }
  for (int i = gs + lane; i < gs4; i += 32) vbuf[i] = 0.0f;
  __syncthreads();

  const float inv_n = 1.0f;  // means divide by n explicitly below
  (void)inv_n;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * 8 + warp) * kSeRowsPerWarp;
  for (int rr = 0; rr < kSeRowsPerWarp; ++rr) {
    const int64_t row = row0 + rr;
    if (row >= a.rows) break;  // warp-uniform
    const SrcT* wrow = wsrc + row * a.ld + g * gs;
    float w[EPL], imp[EPL], tgt[EPL], zm[EPL];
    bool have[EPL];
    float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int i = lane + 32 * j;
      have[j] = i < gs;
      w[j] = have[j] ? to_f32<SrcT>(wrow[i]) : 0.0f;
      imp[j] = have[j] ? a.imp[g * gs + i] : 0.0f;
      if (have[j]) {
        mn = fminf(mn, w[j]);
        mx = fmaxf(mx, w[j]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    // (1) baseline quantisation: scale0, zero point (frozen), targets, zero mask, importance
    Codec<MODE> c0;
    c0.from_stats(mn, mx);
    const float scale0 = c0.scale, zp = c0.zp;
    float denom = 0.0f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      float u = 0.0f;
      if (have[j]) c0.encode(w[j], u);
      tgt[j] = u;
      const bool z = fabsf(u) <= 1e-8f;  // isclose(target, 0)
      zm[j] = z ? 1.0f : 0.0f;
      imp[j] = (z || !have[j]) ? 0.0f : imp[j];
      denom = __fadd_rn(denom, imp[j]);
      if (have[j]) vbuf[lane + 32 * j] = w[j];
    }
    denom = warp_sum(denom);
    const float dn = __fadd_rn(denom, kEps32);
#pragma unroll
    for (int j = 0; j < EPL; ++j) imp[j] = __fdiv_rn(imp[j], dn);
    __syncwarp();
    float fp[kSeMaxChunks][2], qo[kSeMaxChunks][2];
    project<kSeMaxChunks>(vbuf, xs, gs4, np, lane, fp);
    __syncwarp();

    // score of a candidate: mean_n (fp - proj(dq))^2 [+ penalty * mean_i (dq - w)^2]
    auto score = [&](const Codec<MODE>& c, float (&t_out)[EPL], bool want_targets) -> float {
      float pen = 0.0f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        float u = 0.0f;
        if (have[j]) c.encode(w[j], u);
        if (want_targets) t_out[j] = u;
        const float dq = __fmul_rn(u, c.scale);
        if (have[j]) vbuf[lane + 32 * j] = dq;
        const float e = __fsub_rn(dq, w[j]);
        pen = __fmaf_rn(e, e, pen);
      }
      __syncwarp();
      project<kSeMaxChunks>(vbuf, xs, gs4, np, lane, qo);
      __syncwarp();
      float d = 0.0f;
#pragma unroll
      for (int ch = 0; ch < kSeMaxChunks; ++ch) {
        if (ch < (np >> 6)) {
          const float e0 = __fsub_rn(fp[ch][0], qo[ch][0]), e1 = __fsub_rn(fp[ch][1], qo[ch][1]);
          d = __fmaf_rn(e0, e0, d);
          d = __fmaf_rn(e1, e1, d);
        }
      }
      d = __fdiv_rn(warp_sum(d), static_cast<float>(a.n));
      if (a.weight_penalty > 0.0f) {
        pen = __fdiv_rn(warp_sum(pen), static_cast<float>(gs));
        d = __fadd_rn(d, __fmul_rn(a.weight_penalty, pen));
      }
      return d;
    };
    // near-to-ideal scale from the current targets (WC/scale_estimation.py:396-409)
    auto estimate = [&]() -> float {
      float acc = 0.0f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float ideal = __fdiv_rn(fabsf(w[j]), __fadd_rn(fabsf(tgt[j]), zm[j]));
        acc = __fadd_rn(acc, have[j] ? __fmul_rn(ideal, imp[j]) : 0.0f);
      }
      return warp_sum(acc);
    };
    auto retarget = [&](float s) {
      Codec<MODE> c;
      c.from_given(s, zp);
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        float u = 0.0f;
        if (have[j]) c.encode(w[j], u);
        tgt[j] = u;
        zm[j] = (fabsf(u) <= 1e-8f) ? 0.001f : 0.0f;
      }
    };

    float dummy[EPL];
    float best = score(c0, dummy, false);
    float result = scale0;
    const float sign = __fdiv_rn(scale0, fabsf(scale0));
#pragma unroll
    for (int j = 0; j < EPL; ++j) zm[j] = 0.001f * zm[j];

    for (int it = 0; it < a.initial_steps; ++it) {
      const float cand = __fmul_rn(estimate(), sign);
      Codec<MODE> c;
      c.from_given(cand, zp);
      const float d = score(c, dummy, false);
      if (!(d > best)) {
        best = d;
        result = cand;
      }
      if (it < a.initial_steps - 1) retarget(result);
    }
    for (int st = 0; st < a.scale_steps; ++st) {
      const float factor = static_cast<float>(1.0 - 0.05 * st);
      retarget(__fmul_rn(factor, scale0));
      const float cand = __fmul_rn(estimate(), sign);
      Codec<MODE> c;
      c.from_given(cand, zp);
      const float d = score(c, dummy, false);
      if (!(d > best)) {
        best = d;
        result = cand;
      }
    }
    if (lane == 0) {
      a.scale_out[row * a.out_ld + g] = result;
      if (a.zp_out) a.zp_out[row * a.out_ld + g] = static_cast<int32_t>(zp);
    }
  }
}

template <typename SrcT, int MODE>
int launch_se(const SEArgs& a, cudaStream_t st) {
  const int epl = (a.gs + 31) / 32;
  const int gs4 = (a.gs + 3) & ~3;
  const size_t smem = (static_cast<size_t>(gs4) * a.np + 8 * static_cast<size_t>(gs4)) * sizeof(float);
  const dim3 grid(static_cast<unsigned>((a.rows + 8 * kSeRowsPerWarp - 1) / (8 * kSeRowsPerWarp)),
                  static_cast<unsigned>(a.cols / a.gs));
#define NNCFB_SE_LAUNCH(E)                                                                                    \
  do {                                                                                                        \
    NNCFB_CUDA(cudaFuncSetAttribute(scale_estimation_kernel<SrcT, MODE, E>,                                   \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));    \
    scale_estimation_kernel<SrcT, MODE, E><<<grid, 256, smem, st>>>(a);                                       \
  } while (0)
  if (epl <= 1) NNCFB_SE_LAUNCH(1);
  else if (epl <= 2) NNCFB_SE_LAUNCH(2);
  else if (epl <= 4) NNCFB_SE_LAUNCH(4);
  else if (epl <= 8) NNCFB_SE_LAUNCH(8);
  else NNCFB_SE_LAUNCH(16);
#undef NNCFB_SE_LAUNCH
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

template <typename SrcT>
int launch_se_t(const SEArgs& a, int mode, cudaStream_t st) {
  switch (mode) {
    case NNCFB_INT4_SYM: return launch_se<SrcT, NNCFB_INT4_SYM>(a, st);
    case NNCFB_INT4_ASYM: return launch_se<SrcT, NNCFB_INT4_ASYM>(a, st);
    case NNCFB_INT8_SYM: return launch_se<SrcT, NNCFB_INT8_SYM>(a, st);
    case NNCFB_INT8_ASYM: return launch_se<SrcT, NNCFB_INT8_ASYM>(a, st);
    case NNCFB_NF4: return launch_se<SrcT, NNCFB_NF4>(a, st);
    case NNCFB_FP4: return launch_se<SrcT, NNCFB_FP4>(a, st);
    default: break;
  }
  set_error("nncfb_scale_estimation: mode %d is not supported", mode);
  return NNCFB_E_UNSUPPORTED;
}



// Shared by the C entry point and the GPTQ sweep (which refines the groups of one column block at a time:
// `weight` then points into a wider matrix with `ld` elements between rows, and the results go into the
// full [rows, out_ld] tables at the block's first group).
int scale_estimation_launch(const void* weight, int32_t weight_dtype, int64_t rows, int64_t cols, int64_t ld,
                            int64_t group_size, int32_t mode, const float* importance, const float* x, int32_t n_samples,
                            int32_t initial_steps, int32_t scale_steps, float weight_penalty, float* scale_out,
                            int32_t* zp_out, int64_t out_ld, cudaStream_t st) {
  NNCFB_CHECK_ARG(weight && importance && x && scale_out, NNCFB_E_BAD_ARG, "nncfb_scale_estimation: null pointer");
  NNCFB_CHECK_ARG(rows > 0 && cols > 0 && n_samples > 0, NNCFB_E_BAD_ARG, "nncfb_scale_estimation: bad shape");
  NNCFB_CHECK_ARG(group_size > 0 && cols % group_size == 0, NNCFB_E_GROUP_SIZE,
                  "Channel size %lld should be divisible by size of group %lld.", (long long)cols, (long long)group_size);
  NNCFB_CHECK_ARG(!mode_is_asym(mode) || zp_out, NNCFB_E_BAD_ARG, "nncfb_scale_estimation: zp_out is null");
  NNCFB_CHECK_ARG(initial_steps >= 0 && scale_steps >= 0, NNCFB_E_BAD_ARG, "nncfb_scale_estimation: negative steps");
  const int np = ((n_samples + 63) / 64) * 64;
  NNCFB_CHECK_ARG(group_size <= 512, NNCFB_E_TOO_LARGE,
                  "nncfb_scale_estimation: group size %lld exceeds the supported maximum of 512", (long long)group_size);
  NNCFB_CHECK_ARG(np <= 64 * kSeMaxChunks, NNCFB_E_TOO_LARGE,
                  "nncfb_scale_estimation: %d samples exceed the supported maximum of %d", n_samples, 64 * kSeMaxChunks);
  const int gs4 = (static_cast<int>(group_size) + 3) & ~3;
  const size_t smem = (static_cast<size_t>(gs4) * np + 8 * static_cast<size_t>(gs4)) * sizeof(float);
  NNCFB_CHECK_ARG(smem <= 200 * 1024, NNCFB_E_TOO_LARGE,
                  "nncfb_scale_estimation: group_size x samples = %lld x %d needs %zu bytes of shared memory (max 200 KiB)",
                  (long long)group_size, n_samples, smem);
  NNCFB_CHECK_ARG(cols / group_size <= 65535, NNCFB_E_TOO_LARGE, "nncfb_scale_estimation: more than 65535 groups per row");
  SEArgs a;
  a.weight = weight;
  a.imp = importance;
  a.x = x;
  a.scale_out = scale_out;
  a.zp_out = mode_is_asym(mode) ? zp_out : nullptr;
  a.rows = rows;
  a.cols = cols;
  a.ld = ld;
  a.out_ld = out_ld;
  a.gs = static_cast<int>(group_size);
  a.n = n_samples;
  a.np = np;
  a.initial_steps = initial_steps;
  a.scale_steps = scale_steps;
  a.weight_penalty = weight_penalty;
  switch (weight_dtype) {
    case NNCFB_F32: return launch_se_t<float>(a, mode, st);
    case NNCFB_F16: return launch_se_t<__half>(a, mode, st);
    case NNCFB_BF16: return launch_se_t<__nv_bfloat16>(a, mode, st);
    default: break;
  }
  set_error("nncfb_scale_estimation: unsupported weight dtype %d", weight_dtype);
  return NNCFB_E_BAD_ARG;
}

}  // namespace nncfb

extern "C" int nncfb_scale_estimation(const void* weight, int32_t weight_dtype, int64_t rows, int64_t cols,
                                      int64_t group_size, int32_t mode, const float* importance, const float* x,
                                      int32_t n_samples, int32_t initial_steps, int32_t scale_steps,
                                      float weight_penalty, float* scale_out, int32_t* zp_out, void* stream) {
  return nncfb::scale_estimation_launch(weight, weight_dtype, rows, cols, cols, group_size, mode, importance, x, n_samples,
                                        initial_steps, scale_steps, weight_penalty, scale_out, zp_out,
                                        group_size > 0 ? cols / group_size : 0, static_cast<cudaStream_t>(stream));
}
