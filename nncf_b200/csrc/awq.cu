// AWQ: the per-group alpha grid search in two launches.
//
// Restates AWQ._data_aware_step of the reference
// (src/nncf/quantization/algorithms/weight_compression/awq.py:243-357): for every group that holds
// one of the top-k activation channels and every alpha of the grid, scale the group's weight
// columns by s^alpha, quantise-dequantise each output channel over the group, apply it to the
// activations divided by the same scale, and keep the alpha with the smallest mean absolute output
// error.  The reference runs ~10 tensor operations per (group, alpha) with a host synchronisation
// each; here
//   awq_score_kernel   one block per (group, run of alphas, 64 output channels): the group's activation
//                      slices (raw and divided by the candidate scale) staged in shared memory, the
//                      alpha-independent outputs W_g X_g computed once per block, four output channels
//                      per warp at a time sharing every activation value they fetch; per-block partial
//                      error sums go to a scratch buffer (deterministic: no atomics);
//   awq_select_kernel  one block per group: reduces the partials in a fixed order, walks the alphas
//                      with the reference's strict '<' rule and writes the winning scale.
#include <algorithm>

#include "quantize_kernels.cuh"

namespace nncfb {

struct AwqArgs {
  const void* weight;       // [rows, cols]
  const int32_t* group_idx; // [n_groups] group number within the row
  const float* gscale;      // [n_groups, gs] clipped activation magnitudes
  const float* x;           // [cols, n]
  const float* alphas;      // [n_alpha]
  const float* prev_w;      // [cols] mean |previous weight| per channel, or null
  float prev_s, prev_rdim, threshold;
  float* scale_io;          // [cols]
  float* part;              // [n_groups, n_alpha, tiles]
  float* pmax;              // [n_groups, tiles]
  int64_t rows, cols;
  int gs, n, np, n_groups, n_alpha, tiles;
};

// s^alpha with the fp16-overflow guard of WC/awq.py:315-335.  The power is evaluated in double
// precision and rounded once, which reproduces a 1-ulp fp32 pow in all but a handful of cases.
__device__ __forceinline__ float awq_candidate(float gs_i, float alpha, const float* prev_w, int64_t col, float prev_s,
                                               float prev_rdim, float threshold) {
  float cur = static_cast<float>(pow(static_cast<double>(gs_i), static_cast<double>(alpha)));
  if (prev_w != nullptr) {
    const float pw = prev_w[col];
    const float mag = __fmul_rn(__fmul_rn(__fdiv_rn(pw, cur), prev_s), prev_rdim);
    const float clamped = __fdiv_rn(__fmul_rn(__fmul_rn(pw, prev_s), prev_rdim), threshold);
    cur = (mag < threshold) ? cur : clamped;
  }
  return cur;
}

constexpr int kAwqRowsPerWarp = 8;

// sum_i v_r[i] * X[i, col] for R vectors at once, i ascending (the same routine as in the ScaleEstimation
// kernel: every activation value fetched from shared memory serves R rows).
template <int R, int MAXC>
__device__ __forceinline__ void awq_project(const float* __restrict__ vbuf, int stride, const float* __restrict__ xs, int gs4,
                                            int np, int lane, float (&acc)[R][MAXC][2]) {
  const int chunks = np >> 6;
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc[r][c][0] = acc[r][c][1] = 0.0f;
  for (int i = 0; i < gs4; i += 4) {
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

// One block: 64 output channels (8 per warp, R at a time) of one group, for a run of consecutive alphas.
// The full-precision outputs W_g X_g do not depend on alpha: they are computed once per block and kept in
// shared memory; per alpha only the candidate scale, the divided activations and the quantised projection
// are redone.  Sums are accumulated per lane in ascending row order and reduced in a fixed order.
template <typename SrcT, int MODE, int EPL, int R, int MAXC>
__global__ void __launch_bounds__(256) awq_score_kernel(const AwqArgs a, const int alphas_per_block) {
  extern __shared__ __align__(16) float smem[];
  const int gs = a.gs, np = a.np;
  const int gs4 = (gs + 3) & ~3;
  float* xs = smem;                                   // raw activations   [gs4, np]
  float* xd = xs + static_cast<size_t>(gs4) * np;     // divided by scale  [gs4, np]
  float* cur = xd + static_cast<size_t>(gs4) * np;    // candidate scale   [gs4]
  float* vbufs = cur + gs4;                           // [8][R][gs4]
  float* fps = vbufs + 8 * R * gs4;                   // [64 rows][np] full-precision outputs
  __shared__ float red_sum[8], red_max[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* vbuf = vbufs + warp * R * gs4;
  const int grp = blockIdx.z, tile = blockIdx.x;
  const int ai0 = blockIdx.y * alphas_per_block, ai1 = min(ai0 + alphas_per_block, a.n_alpha);
  const int64_t off = static_cast<int64_t>(a.group_idx[grp]) * gs;
  const SrcT* __restrict__ wsrc = reinterpret_cast<const SrcT*>(a.weight);

  for (int idx = threadIdx.x; idx < gs4 * np; idx += blockDim.x) {
    const int i = idx / np, c = idx - i * np;
    xs[idx] = (i < gs && c < a.n) ? a.x[(off + i) * a.n + c] : 0.0f;
  }
  for (int r = 0; r < R; ++r)
    for (int i = gs + lane; i < gs4; i += 32) vbuf[r * gs4 + i] = 0.0f;
  __syncthreads();

  bool have[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) have[j] = lane + 32 * j < gs;
  const int64_t row0 = (static_cast<int64_t>(tile) * 8 + warp) * kAwqRowsPerWarp;

  // ---- fp32_out = W_g x X_g for the block's rows ---------------------------------------------------------
  float amax = 0.0f;
  for (int rr = 0; rr < kAwqRowsPerWarp; rr += R) {
    if (row0 + rr >= a.rows) break;  // warp-uniform
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const SrcT* wrow = wsrc + min(row0 + rr + r, a.rows - 1) * a.cols + off;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        if (have[j]) vbuf[r * gs4 + lane + 32 * j] = to_f32<SrcT>(wrow[lane + 32 * j]);
      }
    }
    __syncwarp();
    float fp[R][MAXC][2];
    awq_project<R, MAXC>(vbuf, gs4, xs, gs4, np, lane, fp);
    __syncwarp();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float* dst = fps + static_cast<size_t>(warp * kAwqRowsPerWarp + rr + r) * np + 2 * lane;
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        if (c < (np >> 6)) {
          *reinterpret_cast<float2*>(dst + 64 * c) = make_float2(fp[r][c][0], fp[r][c][1]);
          if (row0 + rr + r < a.rows) amax = fmaxf(amax, fmaxf(fabsf(fp[r][c][0]), fabsf(fp[r][c][1])));
        }
      }
    }
  }

  for (int ai = ai0; ai < ai1; ++ai) {
    const float alpha = a.alphas[ai];
    __syncthreads();  // the previous alpha's readers of cur / xd / red_* are done
    for (int i = threadIdx.x; i < gs4; i += blockDim.x) {
      cur[i] = i < gs ? awq_candidate(a.gscale[static_cast<int64_t>(grp) * gs + i], alpha, a.prev_w, off + i, a.prev_s,
                                      a.prev_rdim, a.threshold)
                      : 1.0f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gs4 * np; idx += blockDim.x) xd[idx] = __fdiv_rn(xs[idx], cur[idx / np]);
    __syncthreads();

    float sum = 0.0f;
    for (int rr = 0; rr < kAwqRowsPerWarp; rr += R) {
      if (row0 + rr >= a.rows) break;
      // scaled weight, per-channel parameters over the group, quantise-dequantise
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const SrcT* wrow = wsrc + min(row0 + rr + r, a.rows - 1) * a.cols + off;
        float ws[EPL];
        float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          ws[j] = have[j] ? __fmul_rn(to_f32<SrcT>(wrow[lane + 32 * j]), cur[lane + 32 * j]) : 0.0f;
          if (have[j]) {
            mn = fminf(mn, ws[j]);
            mx = fmaxf(mx, ws[j]);
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        Codec<MODE> c;
        c.from_stats(mn, mx);
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          float u = 0.0f;
          if (have[j]) {
            c.encode(ws[j], u);
            vbuf[r * gs4 + lane + 32 * j] = __fmul_rn(u, c.scale);
          }
        }
      }
      __syncwarp();
      float qo[R][MAXC][2];
      awq_project<R, MAXC>(vbuf, gs4, xd, gs4, np, lane, qo);
      __syncwarp();
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (row0 + rr + r < a.rows) {
          const float* src = fps + static_cast<size_t>(warp * kAwqRowsPerWarp + rr + r) * np + 2 * lane;
#pragma unroll
          for (int c = 0; c < MAXC; ++c) {
            if (c < (np >> 6)) {
              const float2 f = *reinterpret_cast<const float2*>(src + 64 * c);
              sum = __fadd_rn(sum, fabsf(__fsub_rn(qo[r][c][0], f.x)));
              sum = __fadd_rn(sum, fabsf(__fsub_rn(qo[r][c][1], f.y)));
            }
          }
        }
      }
    }
    float m = amax;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    if (lane == 0) {
      red_sum[warp] = sum;
      red_max[warp] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.0f, mm = 0.0f;
      for (int w8 = 0; w8 < 8; ++w8) {
        s = __fadd_rn(s, red_sum[w8]);
        mm = fmaxf(mm, red_max[w8]);
      }
      a.part[(static_cast<int64_t>(grp) * a.n_alpha + ai) * a.tiles + tile] = s;
      if (ai == 0) a.pmax[static_cast<int64_t>(grp) * a.tiles + tile] = mm;
    }
  }
}

__global__ void __launch_bounds__(128) awq_select_kernel(const AwqArgs a) {
  __shared__ float diffs[1024];
  __shared__ int best_alpha;
  const int grp = blockIdx.x;
  const float count = static_cast<float>(a.rows) * static_cast<float>(a.n);
  for (int ai = threadIdx.x; ai < a.n_alpha; ai += blockDim.x) {
    float s = 0.0f;
    const float* p = a.part + (static_cast<int64_t>(grp) * a.n_alpha + ai) * a.tiles;
    for (int t = 0; t < a.tiles; ++t) s = __fadd_rn(s, p[t]);
    diffs[ai] = __fdiv_rn(s, count);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float min_diff = 0.0f;
    for (int t = 0; t < a.tiles; ++t) min_diff = fmaxf(min_diff, a.pmax[static_cast<int64_t>(grp) * a.tiles + t]);
    int best = -1;
    for (int ai = 0; ai < a.n_alpha; ++ai) {
      if (diffs[ai] < min_diff) {
        min_diff = diffs[ai];
        best = ai;
      }
    }
    best_alpha = best;
  }
  __syncthreads();
  if (best_alpha >= 0) {
    const int64_t off = static_cast<int64_t>(a.group_idx[grp]) * a.gs;
    const float alpha = a.alphas[best_alpha];
    for (int i = threadIdx.x; i < a.gs; i += blockDim.x) {
      a.scale_io[off + i] = awq_candidate(a.gscale[static_cast<int64_t>(grp) * a.gs + i], alpha, a.prev_w, off + i,
                                          a.prev_s, a.prev_rdim, a.threshold);
    }
  }
}

inline int awq_rows_at_a_time(int gs, int np) {
  const int chunks = np >> 6, epl = (gs + 31) / 32;
  if (chunks <= 1 && epl <= 4) return 4;
  if (chunks <= 2 && epl <= 8) return 2;
  return 1;
}
inline size_t awq_smem_bytes(int gs, int np) {
  const int gs4 = (gs + 3) & ~3;
  return (2 * static_cast<size_t>(gs4) * np + gs4 + 8 * static_cast<size_t>(awq_rows_at_a_time(gs, np)) * gs4 +
          static_cast<size_t>(8 * kAwqRowsPerWarp) * np) * sizeof(float);
}

template <typename SrcT, int MODE, int R, int MAXC>
int launch_awq_rc(const AwqArgs& a, cudaStream_t st) {
  const int epl = (a.gs + 31) / 32;
  const size_t smem = awq_smem_bytes(a.gs, a.np);
  // alphas per block: as many as still leave a few blocks per SM (the alpha-independent part is then amortised)
  const int64_t units = static_cast<int64_t>(a.tiles) * a.n_groups * a.n_alpha;
  const int per_block = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(16, units / (8 * sm_count()))));
  const dim3 grid(a.tiles, (a.n_alpha + per_block - 1) / per_block, a.n_groups);
#define NNCFB_AWQ_LAUNCH(E)                                                                                       \
  do {                                                                                                            \
    if constexpr (E * R <= 16) {                                                                                  \
      NNCFB_CUDA(cudaFuncSetAttribute(awq_score_kernel<SrcT, MODE, E, R, MAXC>,                                   \
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));      \
      awq_score_kernel<SrcT, MODE, E, R, MAXC><<<grid, 256, smem, st>>>(a, per_block);                            \
    }                                                                                                             \
  } while (0)
  if (epl <= 1) NNCFB_AWQ_LAUNCH(1);
  else if (epl <= 2) NNCFB_AWQ_LAUNCH(2);
  else if (epl <= 4) NNCFB_AWQ_LAUNCH(4);
  else if (epl <= 8) NNCFB_AWQ_LAUNCH(8);
  else NNCFB_AWQ_LAUNCH(16);
#undef NNCFB_AWQ_LAUNCH
  NNCFB_CUDA(cudaGetLastError());
  awq_select_kernel<<<a.n_groups, 128, 0, st>>>(a);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

template <typename SrcT, int MODE>
int launch_awq(const AwqArgs& a, cudaStream_t st) {
  switch (awq_rows_at_a_time(a.gs, a.np)) {
    case 4: return launch_awq_rc<SrcT, MODE, 4, 1>(a, st);
    case 2: return launch_awq_rc<SrcT, MODE, 2, 2>(a, st);
    default: return launch_awq_rc<SrcT, MODE, 1, 4>(a, st);
  }
}

template <typename SrcT>
int launch_awq_t(const AwqArgs& a, int mode, cudaStream_t st) {
  switch (mode) {
    case NNCFB_INT4_SYM: return launch_awq<SrcT, NNCFB_INT4_SYM>(a, st);
    case NNCFB_INT4_ASYM: return launch_awq<SrcT, NNCFB_INT4_ASYM>(a, st);
    case NNCFB_NF4: return launch_awq<SrcT, NNCFB_NF4>(a, st);
    case NNCFB_FP4: return launch_awq<SrcT, NNCFB_FP4>(a, st);
    case NNCFB_MXFP4: return launch_awq<SrcT, NNCFB_MXFP4>(a, st);
    default: break;
  }
  set_error("nncfb_awq_search: mode %d is not supported (AWQ applies to 4-bit modes)", mode);
  return NNCFB_E_UNSUPPORTED;
}

inline int awq_tiles(int64_t rows) { return static_cast<int>((rows + 8 * kAwqRowsPerWarp - 1) / (8 * kAwqRowsPerWarp)); }

}  // namespace nncfb

using namespace nncfb;

extern "C" size_t nncfb_awq_workspace_bytes(int64_t rows, int32_t n_groups, int32_t n_alpha) {
  if (rows <= 0 || n_groups <= 0 || n_alpha <= 0) return 0;
  const size_t tiles = static_cast<size_t>(awq_tiles(rows));
  return (static_cast<size_t>(n_groups) * n_alpha * tiles + static_cast<size_t>(n_groups) * tiles) * sizeof(float);
}

extern "C" int nncfb_awq_search(const void* weight, int32_t weight_dtype, int64_t rows, int64_t cols, int32_t mode,
                                int64_t group_size, const int32_t* group_index, int32_t n_groups,
                                const float* group_scale, const float* x, int32_t n_samples, const float* alphas,
                                int32_t n_alpha, const float* prev_w, float prev_s, float prev_rdim, float threshold,
                                float* scale_io, void* workspace, size_t workspace_bytes, void* stream) {
  NNCFB_CHECK_ARG(weight && group_index && group_scale && x && alphas && scale_io && workspace, NNCFB_E_BAD_ARG,
                  "nncfb_awq_search: null pointer");
  NNCFB_CHECK_ARG(rows > 0 && cols > 0 && n_samples > 0 && n_groups > 0 && n_alpha > 0, NNCFB_E_BAD_ARG,
                  "nncfb_awq_search: bad shape");
  NNCFB_CHECK_ARG(group_size > 0 && cols % group_size == 0, NNCFB_E_GROUP_SIZE,
                  "Channel size %lld should be divisible by size of group %lld.", (long long)cols, (long long)group_size);
  NNCFB_CHECK_ARG(group_size <= 512, NNCFB_E_TOO_LARGE, "nncfb_awq_search: group size %lld exceeds the maximum of 512",
                  (long long)group_size);
  NNCFB_CHECK_ARG(n_alpha <= 1024, NNCFB_E_TOO_LARGE, "nncfb_awq_search: more than 1024 alpha steps");
  NNCFB_CHECK_ARG(n_groups <= 65535 && n_alpha <= 65535, NNCFB_E_TOO_LARGE, "nncfb_awq_search: grid too large");
  const int np = ((n_samples + 63) / 64) * 64;
  NNCFB_CHECK_ARG(np <= 256, NNCFB_E_TOO_LARGE, "nncfb_awq_search: %d samples exceed the maximum of 256", n_samples);
  const size_t smem = awq_smem_bytes(static_cast<int>(group_size), np);
  NNCFB_CHECK_ARG(smem <= 200 * 1024, NNCFB_E_TOO_LARGE,
                  "nncfb_awq_search: group_size x samples = %lld x %d needs %zu bytes of shared memory (max 200 KiB)",
                  (long long)group_size, n_samples, smem);
  NNCFB_CHECK_ARG(workspace_bytes >= nncfb_awq_workspace_bytes(rows, n_groups, n_alpha), NNCFB_E_BAD_ARG,
                  "nncfb_awq_search: workspace of %zu bytes is smaller than nncfb_awq_workspace_bytes() = %zu",
                  workspace_bytes, nncfb_awq_workspace_bytes(rows, n_groups, n_alpha));
  AwqArgs a;
  a.weight = weight;
  a.group_idx = group_index;
  a.gscale = group_scale;
  a.x = x;
  a.alphas = alphas;
  a.prev_w = prev_w;
  a.prev_s = prev_s;
  a.prev_rdim = prev_rdim;
  a.threshold = threshold;
  a.scale_io = scale_io;
  a.rows = rows;
  a.cols = cols;
  a.gs = static_cast<int>(group_size);
  a.n = n_samples;
  a.np = np;
  a.n_groups = n_groups;
  a.n_alpha = n_alpha;
  a.tiles = awq_tiles(rows);
  a.part = static_cast<float*>(workspace);
  a.pmax = a.part + static_cast<size_t>(n_groups) * n_alpha * a.tiles;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (weight_dtype) {
    case NNCFB_F32: return launch_awq_t<float>(a, mode, st);
    case NNCFB_F16: return launch_awq_t<__half>(a, mode, st);
    case NNCFB_BF16: return launch_awq_t<__nv_bfloat16>(a, mode, st);
    default: break;
  }
  set_error("nncfb_awq_search: unsupported weight dtype %d", weight_dtype);
  return NNCFB_E_BAD_ARG;
}
