// Instantiates the quantisation kernels for __half weights.
#include "quantize_launch.cuh"

namespace nncfb {
int launch_quantize_f16(const QArgs& a, int mode, QuantPath path, cudaStream_t stream) {
  return launch_quantize_t<__half>(a, mode, path, stream);
}
int launch_fast_f16(const FastBatch& b, int mode, FastClass cls, cudaStream_t stream) {
  return launch_fast_t<__half>(b, mode, cls, stream);
}
}  // namespace nncfb
