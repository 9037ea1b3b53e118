// Activation statistic reducers: per-channel sum, sum of squares and abs-max of an activation
// [tokens, channels] (channel last) in one pass.
//
// They feed the data-aware algorithms like the reference's reducers do
// (src/nncf/common/tensor_statistics/collectors.py): MeanReducer :512-516 (mean over every axis but
// the channel, result in the activation's dtype), MeanVarianceReducer :519-524, MaxVarianceReducer
// :527-532 (population variance per channel), MeanAbsMaxReducer :535-540 and the HAWQ trace
// :924-936 (sum of squares).  One read of the activation yields all of them.
#include <type_traits>

#include "nncfb_common.cuh"

namespace nncfb {

template <typename SrcT>
__global__ void __launch_bounds__(256) channel_stats_kernel(const SrcT* __restrict__ x, int64_t tokens, int64_t channels,
                                                            void* mean_out, float* var_out, float* absmax_out,
                                                            double* sumsq_out) {
  __shared__ double s_sum[8][64], s_sq[8][64];
  __shared__ float s_max[8][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 64 + 2 * lane;
  double sum[2] = {0.0, 0.0}, sq[2] = {0.0, 0.0};
  float amax[2] = {0.0f, 0.0f};
  for (int64_t t = warp; t < tokens; t += 8) {
    const SrcT* row = x + t * channels;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (c0 + k < channels) {
        const float v = to_f32<SrcT>(row[c0 + k]);
        sum[k] += static_cast<double>(v);
        sq[k] += static_cast<double>(v) * static_cast<double>(v);
        amax[k] = fmaxf(amax[k], fabsf(v));
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    s_sum[warp][2 * lane + k] = sum[k];
    s_sq[warp][2 * lane + k] = sq[k];
    s_max[warp][2 * lane + k] = amax[k];
  }
  __syncthreads();
  if (threadIdx.x < 64) {
    const int64_t c = static_cast<int64_t>(blockIdx.x) * 64 + threadIdx.x;
    if (c < channels) {
      double s = 0.0, q = 0.0;
      float m = 0.0f;
      for (int w = 0; w < 8; ++w) {
        s += s_sum[w][threadIdx.x];
        q += s_sq[w][threadIdx.x];
        m = fmaxf(m, s_max[w][threadIdx.x]);
      }
      const double n = static_cast<double>(tokens);
      const double mean = s / n;
      if (mean_out) {
        const float mf = static_cast<float>(mean);
        if constexpr (sizeof(SrcT) == 4) {
          reinterpret_cast<float*>(mean_out)[c] = mf;
        } else if constexpr (std::is_same<SrcT, __half>::value) {
          reinterpret_cast<__half*>(mean_out)[c] = __float2half_rn(mf);
        } else {
          reinterpret_cast<__nv_bfloat16*>(mean_out)[c] = __float2bfloat16_rn(mf);
        }
      }
      if (var_out) var_out[c] = static_cast<float>(fmax(q / n - mean * mean, 0.0));
      if (absmax_out) absmax_out[c] = m;
      if (sumsq_out) sumsq_out[c] = q;
    }
  }
}

}  // namespace nncfb

using namespace nncfb;

extern "C" int nncfb_channel_stats(const void* x, int32_t dtype, int64_t tokens, int64_t channels, void* mean_out,
                                   float* var_out, float* absmax_out, double* sumsq_out, void* stream) {
  NNCFB_CHECK_ARG(x != nullptr, NNCFB_E_BAD_ARG, "nncfb_channel_stats: x is null");
  NNCFB_CHECK_ARG(tokens > 0 && channels > 0, NNCFB_E_BAD_ARG, "nncfb_channel_stats: bad shape [%lld, %lld]",
                  (long long)tokens, (long long)channels);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((channels + 63) / 64);
  switch (dtype) {
    case NNCFB_F32:
      channel_stats_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), tokens, channels, mean_out,
                                                        var_out, absmax_out, sumsq_out);
      break;
    case NNCFB_F16:
      channel_stats_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), tokens, channels, mean_out,
                                                         var_out, absmax_out, sumsq_out);
      break;
    case NNCFB_BF16:
      channel_stats_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), tokens, channels,
                                                                mean_out, var_out, absmax_out, sumsq_out);
      break;
    default:
      set_error("nncfb_channel_stats: unsupported dtype %d", dtype);
      return NNCFB_E_BAD_ARG;
  }
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}
