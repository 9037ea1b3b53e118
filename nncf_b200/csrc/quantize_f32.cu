// Instantiates the quantisation kernels for float weights.
#include "quantize_launch.cuh"

namespace nncfb {
int launch_quantize_f32(const QArgs& a, int mode, QuantPath path, cudaStream_t stream) {
  return launch_quantize_t<float>(a, mode, path, stream);
}
}  // namespace nncfb
