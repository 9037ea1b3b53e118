// Instantiates the quantisation kernels for float weights.
#include "quantize_launch.cuh"

namespace nncfb {
int launch_quantize_f32(const QArgs& a, int mode, QuantPath path, cudaStream_t stream) {
  return launch_quantize_t<float>(a, mode, path, stream);
}
int launch_fast_f32(const FastBatch& b, int mode, FastClass cls, cudaStream_t stream) {
  return launch_fast_t<float>(b, mode, cls, stream);
}
}  // namespace nncfb
