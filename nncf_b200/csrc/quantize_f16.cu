// Instantiates the quantisation kernels for __half weights.
#include "quantize_launch.cuh"

namespace nncfb {
int launch_quantize_f16(const QArgs& a, int mode, QuantPath path, cudaStream_t stream) {
  return launch_quantize_t<__half>(a, mode, path, stream);
}
}  // namespace nncfb
