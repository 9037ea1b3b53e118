// AWQ: the per-group alpha grid search in two launches.
//
// Restates AWQ._data_aware_step of the reference
// (src/nncf/quantization/algorithms/weight_compression/awq.py:243-357): for every group that holds
// one of the top-k activation channels and every alpha of the grid, scale the group's weight
// columns by s^alpha, quantise-dequantise each output channel over the group, apply it to the
// activations divided by the same scale, and keep the alpha with the smallest mean absolute output
// error.  The reference runs ~10 tensor operations per (group, alpha) with a host synchronisation
// each; here
//   awq_score_kernel   one warp per (group, alpha, output channel): weights in registers, the
//                      group's activation slices (raw and divided by the candidate scale) staged
//                      in shared memory; per-block partial error sums go to a scratch buffer
//                      (deterministic: no atomics);
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

template <typename SrcT, int MODE, int EPL>
__global__ void __launch_bounds__(256) awq_score_kernel(const AwqArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int gs = a.gs, np = a.np;
  const int gs4 = (gs + 3) & ~3;
  float* xs = smem;                                   // raw activations   [gs4, np]
  float* xd = xs + static_cast<size_t>(gs4) * np;     // divided by scale  [gs4, np]
  float* cur = xd + static_cast<size_t>(gs4) * np;    // candidate scale   [gs4]
  float* vbufs = cur + gs4;                           // [8][gs4]
  __shared__ float red_sum[8], red_max[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* vbuf = vbufs + warp * gs4;
  const int grp = blockIdx.z, ai = blockIdx.y, tile = blockIdx.x;
  const int64_t off = static_cast<int64_t>(a.group_idx[grp]) * gs;
  const float alpha = a.alphas[ai];

  for (int i = threadIdx.x; i < gs4; i += blockDim.x) {
    cur[i] = i < gs ? awq_candidate(a.gscale[static_cast<int64_t>(grp) * gs + i], alpha, a.prev_w, off + i, a.prev_s,
                                    a.prev_rdim, a.threshold)
                    : 1.0f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < gs4 * np; idx += blockDim.x) {
    const int i = idx / np, c = idx - i * np;
    const float v = (i < gs && c < a.n) ? a.x[(off + i) * a.n + c] : 0.0f;
    xs[idx] = v;
    xd[idx] = __fdiv_rn(v, cur[i]);
  }
  for (int i = gs + lane; i < gs4; i += 32) vbuf[i] = 0.0f;
  __syncthreads();

  const SrcT* __restrict__ wsrc = reinterpret_cast<const SrcT*>(a.weight);
  float sum = 0.0f, amax = 0.0f;
  const int64_t row0 = (static_cast<int64_t>(tile) * 8 + warp) * kAwqRowsPerWarp;
  for (int rr = 0; rr < kAwqRowsPerWarp; ++rr) {
    const int64_t row = row0 + rr;
    if (row >= a.rows) break;
    const SrcT* wrow = wsrc + row * a.cols + off;
    float w[EPL];
    bool have[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int i = lane + 32 * j;
      have[j] = i < gs;
      w[j] = have[j] ? to_f32<SrcT>(wrow[i]) : 0.0f;
      if (have[j]) vbuf[i] = w[j];
    }
    __syncwarp();
    float fpc[4][2], qoc[4][2];
    // fp32_out = W_g x X_g
    {
      const int chunks = np >> 6;
#pragma unroll
      for (int c = 0; c < 4; ++c) fpc[c][0] = fpc[c][1] = 0.0f;
      for (int i = 0; i < gs4; ++i) {
        const float d = vbuf[i];
        const float* xr = xs + static_cast<size_t>(i) * np + 2 * lane;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c < chunks) {
            const float2 xv = *reinterpret_cast<const float2*>(xr + 64 * c);
            fpc[c][0] = __fmaf_rn(d, xv.x, fpc[c][0]);
            fpc[c][1] = __fmaf_rn(d, xv.y, fpc[c][1]);
          }
        }
      }
    }
    __syncwarp();
    // scaled weight, per-channel parameters over the group, quantise-dequantise
    float ws[EPL];
    float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      ws[j] = have[j] ? __fmul_rn(w[j], cur[lane + 32 * j]) : 0.0f;
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
        vbuf[lane + 32 * j] = __fmul_rn(u, c.scale);
      }
    }
    __syncwarp();
    {
      const int chunks = np >> 6;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) qoc[cc][0] = qoc[cc][1] = 0.0f;
      for (int i = 0; i < gs4; ++i) {
        const float d = vbuf[i];
        const float* xr = xd + static_cast<size_t>(i) * np + 2 * lane;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          if (cc < chunks) {
            const float2 xv = *reinterpret_cast<const float2*>(xr + 64 * cc);
            qoc[cc][0] = __fmaf_rn(d, xv.x, qoc[cc][0]);
            qoc[cc][1] = __fmaf_rn(d, xv.y, qoc[cc][1]);
          }
        }
      }
    }
    __syncwarp();
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      if (cc < (np >> 6)) {
        sum = __fadd_rn(sum, fabsf(__fsub_rn(qoc[cc][0], fpc[cc][0])));
        sum = __fadd_rn(sum, fabsf(__fsub_rn(qoc[cc][1], fpc[cc][1])));
        amax = fmaxf(amax, fmaxf(fabsf(fpc[cc][0]), fabsf(fpc[cc][1])));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  }
  if (lane == 0) {
    red_sum[warp] = sum;
    red_max[warp] = amax;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f, m = 0.0f;
    for (int w8 = 0; w8 < 8; ++w8) {
      s = __fadd_rn(s, red_sum[w8]);
      m = fmaxf(m, red_max[w8]);
    }
    a.part[(static_cast<int64_t>(grp) * a.n_alpha + ai) * a.tiles + tile] = s;
    if (ai == 0) a.pmax[static_cast<int64_t>(grp) * a.tiles + tile] = m;
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

template <typename SrcT, int MODE>
int launch_awq(const AwqArgs& a, cudaStream_t st) {
  const int epl = (a.gs + 31) / 32;
  const int gs4 = (a.gs + 3) & ~3;
  const size_t smem = (2 * static_cast<size_t>(gs4) * a.np + 9 * static_cast<size_t>(gs4)) * sizeof(float);
  const dim3 grid(a.tiles, a.n_alpha, a.n_groups);
#define NNCFB_AWQ_LAUNCH(E)                                                                                      \
  do {                                                                                                           \
    NNCFB_CUDA(cudaFuncSetAttribute(awq_score_kernel<SrcT, MODE, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                    static_cast<int>(smem)));                                                    \
    awq_score_kernel<SrcT, MODE, E><<<grid, 256, smem, st>>>(a);                                                 \
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
  const int gs4 = (static_cast<int>(group_size) + 3) & ~3;
  const size_t smem = (2 * static_cast<size_t>(gs4) * np + 9 * static_cast<size_t>(gs4)) * sizeof(float);
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
