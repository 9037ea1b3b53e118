// ScaleEstimation kernels for __nv_bfloat16 weights.
#include "scale_estimation.cuh"

namespace nncfb {
template int launch_se_t<__nv_bfloat16>(const SEArgs&, int, cudaStream_t);
}  // namespace nncfb
