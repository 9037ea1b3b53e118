// ScaleEstimation kernels for float weights.
#include "scale_estimation.cuh"

namespace nncfb {
template int launch_se_t<float>(const SEArgs&, int, cudaStream_t);
}  // namespace nncfb
