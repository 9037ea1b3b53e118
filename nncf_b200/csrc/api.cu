// Error reporting, device queries and small utility kernels of the C ABI.
#include <cstdarg>
#include <cstdio>

#include "nncfb_common.cuh"

namespace nncfb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return NNCFB_E_CUDA;
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

// ---- nibble pack / unpack ---------------------------------------------------------------------
__global__ void __launch_bounds__(256) pack_nibbles_kernel(const uint8_t* __restrict__ in, int64_t n_bytes_out, int add,
                                                           uint8_t* __restrict__ out) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_bytes_out;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint32_t lo = (static_cast<uint32_t>(in[2 * i]) + add) & 15u;
    const uint32_t hi = (static_cast<uint32_t>(in[2 * i + 1]) + add) & 15u;
    out[i] = static_cast<uint8_t>(lo | (hi << 4));
  }
}

__global__ void __launch_bounds__(256) unpack_nibbles_kernel(const uint8_t* __restrict__ in, int64_t n_bytes, int sub,
                                                             int8_t* __restrict__ out) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_bytes;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int b = in[i];
    out[2 * i] = static_cast<int8_t>((b & 15) - sub);
    out[2 * i + 1] = static_cast<int8_t>((b >> 4) - sub);
  }
}

// ---- division self check ------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t& s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

__global__ void __launch_bounds__(256) division_selftest_kernel(int64_t n, uint64_t seed, unsigned long long* mismatches) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  unsigned long long bad = 0;
  for (int64_t i = tid; i < n; i += stride) {
    uint64_t s = seed + static_cast<uint64_t>(i) * 0x632be59bd9b4e019ull;
    const uint64_t r = splitmix64(s);
    // divisor: random sign/mantissa, exponent within the fast range and a little beyond
    const uint32_t se = 127u - 45u + static_cast<uint32_t>((r >> 40) % 91u);
    const float sdiv = __uint_as_float(((static_cast<uint32_t>(r) & 0x807fffffu)) | (se << 23));
    // quotient target near k + 0.5 half of the time (the cases that decide a code), random otherwise
    const uint64_t r2 = splitmix64(s);
    float w;
    if (r2 & 1u) {
      const float k = static_cast<float>(static_cast<int>((r2 >> 8) % 512u) - 256) + 0.5f;
      const float t = __fmul_rn(k, sdiv);
      // step a few ulps around the product
      const int d = static_cast<int>((r2 >> 20) % 9u) - 4;
      w = __uint_as_float(__float_as_uint(t) + d);
    } else {
      const uint32_t we = se - 12u + static_cast<uint32_t>((r2 >> 40) % 20u);
      w = __uint_as_float((static_cast<uint32_t>(r2 >> 8) & 0x807fffffu) | (we << 23));
      if (r2 & 2u) w = __uint_as_float(__float_as_uint(w) & 0xffff0000u);  // bf16-representable
    }
    const Divisor dv = make_divisor(sdiv);
    const float q = div_by(w, dv);
    const float ref = __fdiv_rn(w, sdiv);
    if (__float_as_uint(q) != __float_as_uint(ref)) ++bad;
    // The batched kernels use the multiply/FMA sequence without a range check, for scales in
    // [2^-23, 2^125] (a computed scale is never below eps).  Check it over that whole range
    // wherever the quotient is finite and not vanishingly small.
    const uint64_t r3 = splitmix64(s);
    const uint32_t se2 = 104u + static_cast<uint32_t>((r3 >> 40) % 149u);  // 2^-23 .. 2^125
    const float s2 = __uint_as_float((static_cast<uint32_t>(r3) & 0x007fffffu) | (se2 << 23));
    const int we2 = static_cast<int>(se2) - 30 + static_cast<int>((r3 >> 48) % 50u);  // quotient 2^-30 .. 2^19
    if (we2 > 0 && we2 < 255) {
      float w2 = __uint_as_float((static_cast<uint32_t>(r3 >> 9) & 0x807fffffu) | (static_cast<uint32_t>(we2) << 23));
      if (r3 & 1u) {  // land next to a rounding tie of the quotient
        const float k = static_cast<float>(static_cast<int>((r3 >> 20) % 512u) - 256) + 0.5f;
        w2 = __uint_as_float(__float_as_uint(__fmul_rn(k, s2)) + static_cast<int>((r3 >> 30) % 9u) - 4);
      }
      const float rr = __frcp_rn(s2);
      const float q0 = __fmul_rn(w2, rr);
      const float e = __fmaf_rn(-s2, q0, w2);
      const float q2 = __fmaf_rn(e, rr, q0);
      const float ref2 = __fdiv_rn(w2, s2);
      if (isfinite(ref2) && isfinite(w2) && __float_as_uint(q2) != __float_as_uint(ref2)) ++bad;
    }
  }
  if (bad) atomicAdd(mismatches, bad);
}

}  // namespace nncfb

using namespace nncfb;

extern "C" int nncfb_abi_version(void) { return NNCFB_ABI_VERSION; }

extern "C" const char* nncfb_last_error(void) { return g_error; }

extern "C" int nncfb_pack_nibbles(const void* codes, int64_t n, int32_t add, uint8_t* packed_out, void* stream) {
  NNCFB_CHECK_ARG(codes && packed_out, NNCFB_E_BAD_ARG, "nncfb_pack_nibbles: null pointer");
  NNCFB_CHECK_ARG(n >= 0 && n % 2 == 0, NNCFB_E_BAD_ARG, "nncfb_pack_nibbles: n=%lld must be even", (long long)n);
  if (n == 0) return NNCFB_OK;
  const int64_t nb = n / 2;
  const int grid = static_cast<int>(std::min<int64_t>((nb + 255) / 256, static_cast<int64_t>(sm_count()) * 16));
  pack_nibbles_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(codes), nb, add,
                                                                           packed_out);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

extern "C" int nncfb_unpack_nibbles(const uint8_t* packed, int64_t n_bytes, int32_t sub, int8_t* codes_out, void* stream) {
  NNCFB_CHECK_ARG(packed && codes_out, NNCFB_E_BAD_ARG, "nncfb_unpack_nibbles: null pointer");
  NNCFB_CHECK_ARG(n_bytes >= 0, NNCFB_E_BAD_ARG, "nncfb_unpack_nibbles: negative size");
  if (n_bytes == 0) return NNCFB_OK;
  const int grid = static_cast<int>(std::min<int64_t>((n_bytes + 255) / 256, static_cast<int64_t>(sm_count()) * 16));
  unpack_nibbles_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(packed, n_bytes, sub, codes_out);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

extern "C" int nncfb_selftest_division(int64_t n, uint64_t seed, int64_t* mismatch_out, void* stream) {
  NNCFB_CHECK_ARG(mismatch_out && n > 0, NNCFB_E_BAD_ARG, "nncfb_selftest_division: bad argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NNCFB_CUDA(cudaMemsetAsync(mismatch_out, 0, sizeof(int64_t), st));
  const int grid = sm_count() * 8;
  division_selftest_kernel<<<grid, 256, 0, st>>>(n, seed, reinterpret_cast<unsigned long long*>(mismatch_out));
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}
