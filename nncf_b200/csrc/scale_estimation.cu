// ScaleEstimation: C entry point and the launcher shared with the GPTQ sweep.  The kernel and its per-type
// launchers live in scale_estimation.cuh and are instantiated in scale_estimation_f32.cu / _f16.cu / _bf16.cu.
#include "scale_estimation.cuh"

namespace nncfb {

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
  const size_t smem = se_smem_bytes(static_cast<int>(group_size), np);
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
