// Instantiates the quantisation kernels for __nv_bfloat16 weights.
#include "quantize_launch.cuh"

namespace nncfb {
int launch_quantize_bf16(const QArgs& a, int mode, QuantPath path, cudaStream_t stream) {
  return launch_quantize_t<__nv_bfloat16>(a, mode, path, stream);
}
int launch_fast_bf16(const FastBatch& b, int mode, FastClass cls, cudaStream_t stream) {
  return launch_fast_t<__nv_bfloat16>(b, mode, cls, stream);
}
}  // namespace nncfb
