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
#pragma once

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

// Projection of R vectors at once: out[r][c] (c = 0 .. np/64*2 - 1 per lane: columns 2*lane, 2*lane+1 of
// every 64-column chunk) = sum_i v_r[i] * X[i, col], i ascending.  The vectors are read from the warp's shared
// buffers (row r at vbuf + r * stride); every element of X fetched from shared memory is used for all R rows,
// which is what lifts the kernel off the shared-memory bandwidth limit (R = 1 needs one 8-byte load per two
// multiply-adds).  Each row's sum is accumulated in the same order whatever R is.
template <int R, int MAXC>
__device__ __forceinline__ void project(const float* __restrict__ vbuf, int stride, const float* __restrict__ xs, int gs,
                                        int np, int lane, float (&acc)[R][MAXC][2]) {
  const int chunks = np >> 6;
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc[r][c][0] = acc[r][c][1] = 0.0f;
  for (int i = 0; i < gs; i += 4) {
    float dv[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float4 d = *reinterpret_cast<const float4*>(vbuf + r * stride + i);
      dv[r][0] = d.x; dv[r][1] = d.y; dv[r][2] = d.z; dv[r][3] = d.w;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float* row = xs + static_cast<size_t>(i + k) * np + 2 * lane;
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        if (c < chunks) {
          const float2 xv = *reinterpret_cast<const float2*>(row + 64 * c);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            acc[r][c][0] = __fmaf_rn(dv[r][k], xv.x, acc[r][c][0]);
            acc[r][c][1] = __fmaf_rn(dv[r][k], xv.y, acc[r][c][1]);
          }
        }
      }
    }
  }
}

constexpr int kSeMaxChunks = 4;   // up to 256 samples
constexpr int kSeRowsPerWarp = 8;

// One warp per (8 rows, group), R rows at a time; X_g in shared memory.  Every row goes through the reference's
// sequence (WC/scale_estimation.py:160-377): baseline quantisation, `initial_steps` re-estimates from the kept
// scale, `scale_steps` re-estimates from shrunken baseline scales, keeping a candidate when its output error
// on the calibration samples is not larger.
#ifndef NNCFB_SE_MINBLOCKS
#define NNCFB_SE_MINBLOCKS 2  // resident 256-thread blocks per SM that the register budget must allow
#endif
template <typename SrcT, int MODE, int EPL, int R, int MAXC>
__global__ void __launch_bounds__(256, NNCFB_SE_MINBLOCKS) scale_estimation_kernel(const SEArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int gs = a.gs, np = a.np;
  const int gs4 = (gs + 3) & ~3;               // projection walks the group four elements at a time
  float* xs = smem;                            // [gs4, np]
  float* vbufs = smem + static_cast<size_t>(gs4) * np;  // [8 warps][R][gs4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* vbuf = vbufs + warp * R * gs4;
  const int64_t g = blockIdx.y;
  const SrcT* __restrict__ wsrc = reinterpret_cast<const SrcT*>(a.weight);

  // stage X_g (zero padded to np columns and gs4 rows)
  for (int idx = threadIdx.x; idx < gs4 * np; idx += blockDim.x) {
    const int i = idx / np, c = idx - i * np;
    xs[idx] = (i < gs && c < a.n) ? a.x[(g * gs + i) * a.n + c] : 0.0f;
  }
  for (int r = 0; r < R; ++r)
    for (int i = gs + lane; i < gs4; i += 32) vbuf[r * gs4 + i] = 0.0f;
  __syncthreads();

  bool have[EPL];
  float imp0[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    have[j] = lane + 32 * j < gs;
    imp0[j] = have[j] ? a.imp[g * gs + lane + 32 * j] : 0.0f;
  }
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * 8 + warp) * kSeRowsPerWarp;
  for (int rr = 0; rr < kSeRowsPerWarp; rr += R) {
    if (row0 + rr >= a.rows) break;  // warp-uniform
    // rows beyond the end repeat the last row (their results are not stored)
    int64_t rows[R];
#pragma unroll
    for (int r = 0; r < R; ++r) rows[r] = min(row0 + rr + r, a.rows - 1);
    float w[R][EPL], imp[R][EPL], tgt[R][EPL], zm[R][EPL];
    float scale0[R], zp[R], sign[R], best[R], result[R];
    float fp[R][MAXC][2], qo[R][MAXC][2];
    Codec<MODE> c0[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const SrcT* wrow = wsrc + rows[r] * a.ld + g * gs;
      float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        w[r][j] = have[j] ? to_f32<SrcT>(wrow[lane + 32 * j]) : 0.0f;
        if (have[j]) {
          mn = fminf(mn, w[r][j]);
          mx = fmaxf(mx, w[r][j]);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      // (1) baseline quantisation: scale0, zero point (frozen), targets, zero mask, importance
      c0[r].from_stats(mn, mx);
      scale0[r] = c0[r].scale;
      zp[r] = c0[r].zp;
      float denom = 0.0f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        float u = 0.0f;
        if (have[j]) c0[r].encode(w[r][j], u);
        tgt[r][j] = u;
        const bool z = fabsf(u) <= 1e-8f;  // isclose(target, 0)
        zm[r][j] = z ? 1.0f : 0.0f;
        imp[r][j] = (z || !have[j]) ? 0.0f : imp0[j];
        denom = __fadd_rn(denom, imp[r][j]);
        if (have[j]) vbuf[r * gs4 + lane + 32 * j] = w[r][j];
      }
      denom = warp_sum(denom);
      const float dn = __fadd_rn(denom, kEps32);
#pragma unroll
      for (int j = 0; j < EPL; ++j) imp[r][j] = __fdiv_rn(imp[r][j], dn);
    }
    __syncwarp();
    project<R, MAXC>(vbuf, gs4, xs, gs4, np, lane, fp);
    __syncwarp();

    // scores of one candidate per row: mean_n (fp - proj(dq))^2 [+ penalty * mean_i (dq - w)^2]
    auto score = [&](const Codec<MODE> (&c)[R], float (&d_out)[R]) {
      float pen[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        pen[r] = 0.0f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          float u = 0.0f;
          if (have[j]) c[r].encode(w[r][j], u);
          const float dq = __fmul_rn(u, c[r].scale);
          if (have[j]) vbuf[r * gs4 + lane + 32 * j] = dq;
          const float e = __fsub_rn(dq, w[r][j]);
          pen[r] = __fmaf_rn(e, e, pen[r]);
        }
      }
      __syncwarp();
      project<R, MAXC>(vbuf, gs4, xs, gs4, np, lane, qo);
      __syncwarp();
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float d = 0.0f;
#pragma unroll
        for (int ch = 0; ch < MAXC; ++ch) {
          if (ch < (np >> 6)) {
            const float e0 = __fsub_rn(fp[r][ch][0], qo[r][ch][0]), e1 = __fsub_rn(fp[r][ch][1], qo[r][ch][1]);
            d = __fmaf_rn(e0, e0, d);
            d = __fmaf_rn(e1, e1, d);
          }
        }
        d = __fdiv_rn(warp_sum(d), static_cast<float>(a.n));
        if (a.weight_penalty > 0.0f) {
          const float p = __fdiv_rn(warp_sum(pen[r]), static_cast<float>(gs));
          d = __fadd_rn(d, __fmul_rn(a.weight_penalty, p));
        }
        d_out[r] = d;
      }
    };
    // near-to-ideal scale from the current targets (WC/scale_estimation.py:396-409)
    auto estimate = [&](int r) -> float {
      float acc = 0.0f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float ideal = __fdiv_rn(fabsf(w[r][j]), __fadd_rn(fabsf(tgt[r][j]), zm[r][j]));
        acc = __fadd_rn(acc, have[j] ? __fmul_rn(ideal, imp[r][j]) : 0.0f);
      }
      return warp_sum(acc);
    };
    auto retarget = [&](int r, float s) {
      Codec<MODE> c;
      c.from_given(s, zp[r]);
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        float u = 0.0f;
        if (have[j]) c.encode(w[r][j], u);
        tgt[r][j] = u;
        zm[r][j] = (fabsf(u) <= 1e-8f) ? 0.001f : 0.0f;
      }
    };

    score(c0, best);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      result[r] = scale0[r];
      sign[r] = __fdiv_rn(scale0[r], fabsf(scale0[r]));
#pragma unroll
      for (int j = 0; j < EPL; ++j) zm[r][j] = 0.001f * zm[r][j];
    }
    Codec<MODE> c[R];
    float cand[R], d[R];
    for (int it = 0; it < a.initial_steps; ++it) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        cand[r] = __fmul_rn(estimate(r), sign[r]);
        c[r].from_given(cand[r], zp[r]);
      }
      score(c, d);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (!(d[r] > best[r])) {
          best[r] = d[r];
          result[r] = cand[r];
        }
        if (it < a.initial_steps - 1) retarget(r, result[r]);
      }
    }
    for (int st = 0; st < a.scale_steps; ++st) {
      const float factor = static_cast<float>(1.0 - 0.05 * st);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        retarget(r, __fmul_rn(factor, scale0[r]));
        cand[r] = __fmul_rn(estimate(r), sign[r]);
        c[r].from_given(cand[r], zp[r]);
      }
      score(c, d);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (!(d[r] > best[r])) {
          best[r] = d[r];
          result[r] = cand[r];
        }
      }
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int64_t row = row0 + rr + r;
        if (row < a.rows) {
          a.scale_out[row * a.out_ld + g] = result[r];
          if (a.zp_out) a.zp_out[row * a.out_ld + g] = static_cast<int32_t>(zp[r]);
        }
      }
    }
  }
}

// R rows at a time with MAXC 64-sample chunks of accumulators: 4 x 1 for up to 64 samples (the default subset),
// 2 x 2 up to 128, 1 x 4 up to 256 - the register budget allows about eight accumulator pairs per array.
template <typename SrcT, int MODE, int R, int MAXC>
int launch_se_rc(const SEArgs& a, cudaStream_t st) {
  const int epl = (a.gs + 31) / 32;
  const int gs4 = (a.gs + 3) & ~3;
  const size_t smem = (static_cast<size_t>(gs4) * a.np + 8 * static_cast<size_t>(R) * gs4) * sizeof(float);
  const dim3 grid(static_cast<unsigned>((a.rows + 8 * kSeRowsPerWarp - 1) / (8 * kSeRowsPerWarp)),
                  static_cast<unsigned>(a.cols / a.gs));
#define NNCFB_SE_LAUNCH(E)                                                                                    \
  do {                                                                                                        \
    if constexpr (E * R <= 16) { /* the combinations launch_se() can ask for */                               \
      NNCFB_CUDA(cudaFuncSetAttribute(scale_estimation_kernel<SrcT, MODE, E, R, MAXC>,                        \
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));  \
      scale_estimation_kernel<SrcT, MODE, E, R, MAXC><<<grid, 256, smem, st>>>(a);                            \
    }                                                                                                         \
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

// rows processed together for a group size and a padded sample count
inline int se_rows_at_a_time(int gs, int np) {
  const int chunks = np >> 6, epl = (gs + 31) / 32;
  if (chunks <= 1 && epl <= 4) return 4;
  if (chunks <= 2 && epl <= 8) return 2;
  return 1;
}
inline size_t se_smem_bytes(int gs, int np) {
  const int gs4 = (gs + 3) & ~3;
  return (static_cast<size_t>(gs4) * np + 8 * static_cast<size_t>(se_rows_at_a_time(gs, np)) * gs4) * sizeof(float);
}

template <typename SrcT, int MODE>
int launch_se(const SEArgs& a, cudaStream_t st) {
  switch (se_rows_at_a_time(a.gs, a.np)) {
    case 4: return launch_se_rc<SrcT, MODE, 4, 1>(a, st);
    case 2: return launch_se_rc<SrcT, MODE, 2, 2>(a, st);
    default: return launch_se_rc<SrcT, MODE, 1, 4>(a, st);
  }
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

// One translation unit per source type instantiates its kernels (scale_estimation_f32.cu, _f16.cu, _bf16.cu).
extern template int launch_se_t<float>(const SEArgs&, int, cudaStream_t);
extern template int launch_se_t<__half>(const SEArgs&, int, cudaStream_t);
extern template int launch_se_t<__nv_bfloat16>(const SEArgs&, int, cudaStream_t);

}  // namespace nncfb
