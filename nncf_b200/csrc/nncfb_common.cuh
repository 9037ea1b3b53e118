// Shared host/device helpers of the nncf_b200 CUDA library (sm_100a).
//
// Parity-critical arithmetic lives here: every function states which step of the
// reference (nncf 3.2.0; WC = src/nncf/quantization/algorithms/weight_compression) it
// reproduces bit for bit.  This translation unit set is compiled with -fmad=false so that
// nvcc never contracts a*b+c on its own; fused operations are written explicitly.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nncf_b200.h"

namespace nncfb {

// ---- error reporting (thread-local message returned by nncfb_last_error) -------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define NNCFB_CHECK_ARG(cond, code, ...) \
  do {                                   \
    if (!(cond)) {                       \
      ::nncfb::set_error(__VA_ARGS__);   \
      return (code);                     \
    }                                    \
  } while (0)

#define NNCFB_CUDA(call)                                        \
  do {                                                          \
    cudaError_t e_ = (call);                                    \
    if (e_ != cudaSuccess) return ::nncfb::cuda_fail(e_, #call); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// number of SMs of the current device (cached per device)
int sm_count();

constexpr float kEps32 = 1.1920928955078125e-07f;  // fns.finfo(float32).eps in the reference

// ---- mode traits ----------------------------------------------------------------------
__host__ __device__ constexpr bool mode_is_integer(int m) { return m <= NNCFB_INT4_ASYM; }
__host__ __device__ constexpr bool mode_is_asym(int m) { return m == NNCFB_INT8_ASYM || m == NNCFB_INT4_ASYM; }
__host__ __device__ constexpr int mode_bits(int m) {
  return (m == NNCFB_INT8_SYM || m == NNCFB_INT8_ASYM || m == NNCFB_FP8_E4M3 || m == NNCFB_MXFP8_E4M3) ? 8 : 4;
}
__host__ __device__ constexpr bool mode_is_mx(int m) { return m == NNCFB_MXFP4 || m == NNCFB_MXFP8_E4M3; }

#ifdef __CUDACC__

// ---- loads ----------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// fp32 value as the sum of three bf16 numbers (round to nearest at each step; the two remainders are exact
// in fp32): |v - (hi + mid + lo)| <= 2^-27 |v| for values whose low planes stay clear of the subnormals.
__device__ __forceinline__ void split_bf16x3(float v, __nv_bfloat16& hi, __nv_bfloat16& mid, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(v);
  const float r1 = __fsub_rn(v, __bfloat162float(hi));
  mid = __float2bfloat16_rn(r1);
  const float r2 = __fsub_rn(r1, __bfloat162float(mid));
  lo = __float2bfloat16_rn(r2);
}

// ---- exact fp32 division by a per-group constant -----------------------------------------
// The reference divides every weight by its group's scale with a true IEEE division
// (WC/weight_lowering.py:678, :626).  One division per element is the most expensive step
// of the kernel, so the divisor's correctly rounded reciprocal is computed once per group and
// each quotient is obtained with one multiply and one FMA-based correction (Markstein):
//   q0 = RN(w * r);  e = w - s*q0 (exact in one FMA);  q = RN(q0 + e * r)
// which equals RN(w / s) when r = RN(1/s) and nothing under/overflows.  Divisors outside a
// comfortable exponent range take the plain division instead.
struct Divisor {
  float s;    // the divisor
  float r;    // RN(1 / s)
  bool fast;  // true: correction sequence is exact for this divisor
};

__device__ __forceinline__ Divisor make_divisor(float s) {
  Divisor d;
  d.s = s;
  d.r = __frcp_rn(s);
  const uint32_t e = (__float_as_uint(s) >> 23) & 0xffu;
  d.fast = (e >= 127u - 40u) && (e <= 127u + 40u);
  return d;
}

__device__ __forceinline__ float div_by(float w, const Divisor& d) {
  if (d.fast) {
    const float q0 = __fmul_rn(w, d.r);
    const float e = __fmaf_rn(-d.s, q0, w);
    return __fmaf_rn(e, d.r, q0);
  }
  return __fdiv_rn(w, d.s);
}

// ---- integer quantisation parameters ------------------------------------------------------
struct GroupParams {
  float scale;
  float zp;  // zero point as fp32 (0 for symmetric / float modes)
};

// Symmetric signed scale, WC/weight_lowering.py:629-649:
//   where(|min| >= max, |min|, -max) / 2^(bits-1);  |scale| < eps -> eps
template <int BITS>
__device__ __forceinline__ float signed_scale(float mn, float mx) {
  const float amin = fabsf(mn);
  float s = (amin >= mx) ? amin : -mx;
  s = __fdiv_rn(s, static_cast<float>(1 << (BITS - 1)));
  return (fabsf(s) < kEps32) ? kEps32 : s;
}

// Asymmetric scale and zero point, src/nncf/quantization/fake_quantize.py:322-350 with
// level_low = 0, level_high = 2^bits - 1, narrow_range = False:
//   scale = (max - min) / (levels - 1);  |scale| < eps -> eps
//   zp = clip(int32(0 - round(min / scale)), 0, 2^bits - 1)
template <int BITS>
__device__ __forceinline__ GroupParams asym_params(float mn, float mx) {
  constexpr int kHigh = (1 << BITS) - 1;
  float s = __fdiv_rn(__fsub_rn(mx, mn), static_cast<float>(kHigh));
  s = (fabsf(s) < kEps32) ? kEps32 : s;
  const float z = __fsub_rn(0.0f, rintf(__fdiv_rn(mn, s)));
  // the reference casts to int32 before clipping; clamping in float first gives the same
  // result for every finite z and avoids the undefined out-of-range conversion
  int zi = static_cast<int>(fminf(fmaxf(z, -1.0f), static_cast<float>(kHigh + 1)));
  zi = min(max(zi, 0), kHigh);
  GroupParams p;
  p.scale = s;
  p.zp = static_cast<float>(zi);
  return p;
}

// ---- float (code-book) formats --------------------------------------------------------------
// NF4: 16 levels (WC/constants.py:17-36) and the 15 literal decision boundaries
// (WC/constants.py:84-103).  A value equal to a boundary goes to the lower level
// (searchsorted side='left', WC/weight_lowering.py:574).
__device__ __constant__ const float kNf4Levels[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f, -0.28444138169288635f,
    -0.18477343022823334f, -0.09105003625154495f, 0.0f, 0.07958029955625534f, 0.16093020141124725f,
    0.24611230194568634f, 0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
    0.7229568362236023f, 1.0f};

__device__ __forceinline__ int nf4_index(float x) {
  // branch-free binary search over compile-time constants: idx = #{bounds < x}
  constexpr float b0 = -0.84809643f, b1 = -0.6106329f, b2 = -0.45999527f, b3 = -0.33967942f, b4 = -0.2346074f,
                  b5 = -0.13791174f, b6 = -0.045525018f, b7 = 0.03979015f, b8 = 0.120255254f, b9 = 0.20352125f,
                  b10 = 0.29201376f, b11 = 0.38931254f, b12 = 0.5016634f, b13 = 0.6427869f, b14 = 0.8614784f;
  const bool c3 = x > b7;
  const float t2 = c3 ? b11 : b3;
  const bool c2 = x > t2;
  const float t1 = c3 ? (c2 ? b13 : b9) : (c2 ? b5 : b1);
  const bool c1 = x > t1;
  const float t0 = c3 ? (c2 ? (c1 ? b14 : b12) : (c1 ? b10 : b8)) : (c2 ? (c1 ? b6 : b4) : (c1 ? b2 : b0));
  const bool c0 = x > t0;
  return (c3 ? 8 : 0) + (c2 ? 4 : 0) + (c1 ? 2 : 0) + (c0 ? 1 : 0);
}

// E2M1 (FP4 / MXFP4 element format): nearest of {0, .5, 1, 1.5, 2, 3, 4, 6} with ties to the
// value whose mantissa bit is even, saturating at 6 -- what WC/weight_lowering.py:577-583
// computes on its 15-entry table.  Returns the magnitude index 0..7.
__device__ __forceinline__ int e2m1_index(float a /* |x| */) {
  return (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
}
__device__ __forceinline__ float e2m1_magnitude(int idx) {
  // 0, .5, 1, 1.5, 2, 3, 4, 6  ==  subnormal .5*m for e = 0, else (1 + m/2) * 2^(e-1)
  const int e = idx >> 1, m = idx & 1;
  return e == 0 ? 0.5f * m : __uint_as_float(((126u + e) << 23) | (static_cast<uint32_t>(m) << 22));
}

// fp32 -> fp16 (RNE) -> E4M3 "fn" (RNE, no infinities): fp16 NaN/Inf and everything that
// rounds beyond 448 become NaN (0x7F), fp16 subnormals become signed zero.
// WC/fp8_conversion.py:43-228.
__device__ __forceinline__ uint32_t e4m3_bits(float x) {
  const uint32_t h = __half_as_ushort(__float2half_rn(x));
  const uint32_t sign = (h >> 8) & 0x80u;
  const int e16 = static_cast<int>((h >> 10) & 0x1fu);
  const uint32_t m16 = h & 0x3ffu;
  if (e16 == 31) return sign | 0x7fu;
  if (e16 == 0) return sign;
  const int e8 = e16 - 8;
  const uint32_t sig = m16 | 0x400u;
  int drop = e8 >= 1 ? 7 : 8 - e8;
  drop = min(drop, 31);
  uint32_t kept = sig >> drop;
  const uint32_t rem = sig & ((1u << drop) - 1u);
  const uint32_t half = 1u << (drop - 1);
  kept += (rem > half || (rem == half && (kept & 1u))) ? 1u : 0u;
  uint32_t bits;
  if (e8 >= 1) {
    bits = kept >= 16u ? static_cast<uint32_t>(e8 + 1) << 3 : (static_cast<uint32_t>(e8) << 3) | (kept & 7u);
  } else {
    bits = kept;
  }
  return sign | min(bits, 0x7fu);
}
__device__ __forceinline__ float e4m3_value(uint32_t bits) {
  const uint32_t mag = bits & 0x7fu;
  float v;
  if (mag == 0x7fu) {
    v = __uint_as_float(0x7fc00000u);
  } else {
    const uint32_t e = mag >> 3, m = mag & 7u;
    v = e == 0 ? static_cast<float>(m) * 0.001953125f : __uint_as_float(((120u + e) << 23) | (m << 20));
  }
  return (bits & 0x80u) ? -v : v;
}

// Power-of-two (E8M0) scale of the MX formats, WC/weight_lowering.py:118-126:
//   2 ** clip(ceil(log2(scale)), -127, 127) with log2 evaluated in fp32.
// An fp32 log2 of a value a few ulps above 2^k rounds to exactly k, so ceil() returns k there
// rather than k+1; that window is handled with a double-precision log2 rounded to fp32.
// Returns the exponent; the scale is exp2_int(e).
__device__ __forceinline__ int e8m0_exponent(float scale /* > 0, >= eps */) {
  const uint32_t b = __float_as_uint(scale);
  const int e = static_cast<int>((b >> 23) & 0xffu) - 127;
  const uint32_t m = b & 0x7fffffu;
  int r;
  if (m == 0u) {
    r = e;
  } else if (m < 32u) {
    r = static_cast<int>(ceilf(static_cast<float>(log2(static_cast<double>(scale)))));
  } else {
    r = e + 1;
  }
  return min(max(r, -127), 127);
}
__device__ __forceinline__ float exp2_int(int e) {
  return e > -127 ? __uint_as_float(static_cast<uint32_t>(e + 127) << 23) : __uint_as_float(0x00400000u);
}

#endif  // __CUDACC__

}  // namespace nncfb
