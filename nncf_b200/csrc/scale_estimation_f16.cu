// ScaleEstimation kernels for __half weights.
#include "scale_estimation.cuh"

namespace nncfb {
template int launch_se_t<__half>(const SEArgs&, int, cudaStream_t);
}  // namespace nncfb
