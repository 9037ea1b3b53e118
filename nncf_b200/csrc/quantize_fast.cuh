// Speed-of-light variants of the integer quantisation kernels for the storage path
// (codes + scale [+ zero point] out, parameters computed from the weight itself).
//
// The general kernels in quantize_kernels.cuh are instruction-bound on B200: at ~2.5 B/element of
// HBM traffic the SMs have about a dozen issue slots per element.  This file gets under that
// budget while producing bit-identical results:
//   * min/max on packed bf16x2 / f16x2 pairs, one packed shuffle per reduction step carrying
//     (min, -max) together;
//   * the exact division by the group's scale as multiply + two FMAs (see Divisor) issued as
//     packed fp32x2 instructions (fmul2 / ffma2), selected per group, with the plain IEEE
//     division as the fallback for divisors outside the exact range;
//   * round-half-even by adding 1.5 * 2^23 (one packed add, no float->int conversions) and
//     nibble / byte packing by Horner multiply-adds on the raw bit patterns;
//   * ONE launch for a whole list of tensors (descriptor table in kernel parameters, persistent
//     warps striding over all groups), so a model is not 200+ launch latencies.
#pragma once

#include <type_traits>

#include "quantize_kernels.cuh"

namespace nncfb {

constexpr int kMaxBatchTensors = 256;

// Tuning knobs of the row-group kernel (the defaults are the measured best on B200).
#ifndef NNCFB_ROWS_U
#define NNCFB_ROWS_U 4          // groups in flight per sub-warp
#endif
#ifndef NNCFB_ROWS_MINBLOCKS
#define NNCFB_ROWS_MINBLOCKS 4  // resident 256-thread blocks per SM that the register budget must allow
#endif

struct FastTensor {
  const void* weight;
  uint8_t* codes;
  float* scale;
  int32_t* zp;
  uint16_t* scale_f16;
  uint8_t* e8m0;
  int64_t n_groups;
  uint8_t* zp_packed;  // stored form of the zero points: u8 per group (8-bit modes) or two groups per byte (4-bit)
};

struct FastBatch {
  int n_tensors;
  int codes_nibble;                            // 1: nibble-packed, 0: one byte per code
  int64_t iter_start[kMaxBatchTensors + 1];    // prefix sum of warp iterations per tensor
  FastTensor t[kMaxBatchTensors];
};

constexpr uint32_t kMagicBits = 0x4B400000u;  // 12582912.0f = 1.5 * 2^23

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// (min, -max) of 8 elements packed as two 16-bit floats of the source type (exact: the
// extremes are source values).  For fp32 sources the pair is kept as two floats.
struct MinNegMax {
  uint32_t packed;  // 16-bit sources
  float mn, nmx;    // fp32 sources
};

template <typename SrcT, int VPL>
__device__ __forceinline__ MinNegMax min_negmax(const Raw8<SrcT> (&raw)[VPL]) {
  MinNegMax r;
  if constexpr (sizeof(SrcT) == 2) {
    using V2 = typename std::conditional<std::is_same<SrcT, __half>::value, __half2, __nv_bfloat162>::type;
    V2 lo, hi;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const V2* p = reinterpret_cast<const V2*>(&raw[v].r);
      const V2 l = __hmin2(__hmin2(p[0], p[1]), __hmin2(p[2], p[3]));
      const V2 h = __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3]));
      lo = v == 0 ? l : __hmin2(lo, l);
      hi = v == 0 ? h : __hmax2(hi, h);
    }
    const uint32_t L = *reinterpret_cast<const uint32_t*>(&lo);
    const uint32_t H = *reinterpret_cast<const uint32_t*>(&hi) ^ 0x80008000u;  // negate both halves
    const uint32_t a = __byte_perm(L, H, 0x5410);                               // (lo.x, -hi.x)
    const uint32_t b = __byte_perm(L, H, 0x7632);                               // (lo.y, -hi.y)
    const V2 m = __hmin2(*reinterpret_cast<const V2*>(&a), *reinterpret_cast<const V2*>(&b));
    r.packed = *reinterpret_cast<const uint32_t*>(&m);
    r.mn = r.nmx = 0.0f;
  } else {
    float mn = 0.f, mx = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      float a, b;
      minmax8(raw[v], a, b);
      mn = v == 0 ? a : fminf(mn, a);
      mx = v == 0 ? b : fmaxf(mx, b);
    }
    r.mn = mn;
    r.nmx = -mx;
    r.packed = 0;
  }
  return r;
}

template <typename SrcT>
__device__ __forceinline__ void reduce_step(MinNegMax& m, int offset) {
  if constexpr (sizeof(SrcT) == 2) {
    using V2 = typename std::conditional<std::is_same<SrcT, __half>::value, __half2, __nv_bfloat162>::type;
    const uint32_t o = __shfl_xor_sync(0xffffffffu, m.packed, offset);
    const V2 x = __hmin2(*reinterpret_cast<const V2*>(&m.packed), *reinterpret_cast<const V2*>(&o));
    m.packed = *reinterpret_cast<const uint32_t*>(&x);
  } else {
    m.mn = fminf(m.mn, __shfl_xor_sync(0xffffffffu, m.mn, offset));
    m.nmx = fminf(m.nmx, __shfl_xor_sync(0xffffffffu, m.nmx, offset));
  }
}

template <typename SrcT>
__device__ __forceinline__ void finish_minmax(const MinNegMax& m, float& mn, float& mx) {
  if constexpr (std::is_same<SrcT, __nv_bfloat16>::value) {
    mn = __uint_as_float(m.packed << 16);
    mx = -__uint_as_float(m.packed & 0xffff0000u);
  } else if constexpr (std::is_same<SrcT, __half>::value) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&m.packed));
    mn = f.x;
    mx = -f.y;
  } else {
    mn = m.mn;
    mx = -m.nmx;
  }
}

__device__ __forceinline__ void unpack8_pairs(const Raw8<float>& x, float2 (&v)[4]) {
  v[0] = f2(x.a.x, x.a.y); v[1] = f2(x.a.z, x.a.w); v[2] = f2(x.b.x, x.b.y); v[3] = f2(x.b.z, x.b.w);
}
__device__ __forceinline__ void unpack8_pairs(const Raw8<__nv_bfloat16>& x, float2 (&v)[4]) {
  const uint32_t w[4] = {x.r.x, x.r.y, x.r.z, x.r.w};
#pragma unroll
  // low half by an integer multiply (FMA pipe) rather than a shift: the ALU pipe is the busy one
  for (int i = 0; i < 4; ++i) v[i] = f2(__uint_as_float(w[i] * 65536u), __uint_as_float(w[i] & 0xffff0000u));
}
__device__ __forceinline__ void unpack8_pairs(const Raw8<__half>& x, float2 (&v)[4]) {
  const uint32_t w[4] = {x.r.x, x.r.y, x.r.z, x.r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
}

// Integer codes of 8 elements as Horner-packed bit patterns.
//   NIB: returns one word of 8 nibbles (INT4_SYM with the +8 storage offset);
//   else: returns two words of 4 bytes (signed modes as two's complement).
// The division is the multiply/FMA sequence of `Divisor`: in these kernels the scale is computed
// from the data, so it lies in [eps, 2^125], where the sequence equals the IEEE quotient whenever
// the quotient can decide a code (see exact_quotient).
// CLAMP: 2 = clip to [low, high]; 1 = upper bound only; 0 = no clip.  The caller proves per group
// which bounds a quotient can cross (see int_params); every skipped bound saves one instruction per
// element on the busiest (ALU) pipe.
template <int MODE, int CLAMP>
__device__ __forceinline__ uint2 encode8_int(const float2 (&v)[4], float s, float r, float zp) {
  constexpr bool kAsym = mode_is_asym(MODE);
  constexpr int kBits = mode_bits(MODE);
  constexpr float kLow = kAsym ? 0.0f : -static_cast<float>(1 << (kBits - 1));
  constexpr float kHigh = kAsym ? static_cast<float>((1 << kBits) - 1) : static_cast<float>((1 << (kBits - 1)) - 1);
  constexpr float kBias = kAsym ? 0.0f : static_cast<float>(1 << (kBits - 1));  // digit = code + bias >= 0
  const float2 r2 = f2(r, r), ns2 = f2(-s, -s), zp2 = f2(zp, zp), magic2 = f2(12582912.0f + kBias, 12582912.0f + kBias);
  uint32_t bits[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 q0 = __fmul2_rn(v[i], r2);
    const float2 e = __ffma2_rn(ns2, q0, v[i]);
    float2 q = __ffma2_rn(e, r2, q0);
    if constexpr (kAsym) q = __fadd2_rn(q, zp2);  // separate fp32 add, as the reference does
    // clamp-then-round equals round-then-clamp for integer bounds
    if constexpr (CLAMP == 2) {
      q.x = fmaxf(fminf(q.x, kHigh), kLow);
      q.y = fmaxf(fminf(q.y, kHigh), kLow);
    } else if constexpr (CLAMP == 1) {
      q.x = fminf(q.x, kHigh);
      q.y = fminf(q.y, kHigh);
    }
    const float2 t = __fadd2_rn(q, magic2);  // round half to even into the low mantissa bits
    bits[2 * i] = __float_as_uint(t.x);
    bits[2 * i + 1] = __float_as_uint(t.y);
  }
  uint2 out;
  if constexpr (kBits == 4) {
    uint32_t acc = bits[7];
#pragma unroll
    for (int i = 6; i >= 0; --i) acc = acc * 16u + bits[i];
    out.x = acc - kMagicBits * 0x11111111u;
    out.y = 0u;
  } else {
    uint32_t a0 = bits[3], a1 = bits[7];
#pragma unroll
    for (int i = 2; i >= 0; --i) {
      a0 = a0 * 256u + bits[i];
      a1 = a1 * 256u + bits[4 + i];
    }
    a0 -= kMagicBits * 0x01010101u;
    a1 -= kMagicBits * 0x01010101u;
    if constexpr (!kAsym) {  // offset binary -> two's complement
      a0 ^= 0x80808080u;
      a1 ^= 0x80808080u;
    }
    out.x = a0;
    out.y = a1;
  }
  return out;
}

// Scale and zero point of a group plus `need_clamp`: false only when every quotient of the group
// provably rounds into the code range, so that the clip of WC/weight_lowering.py:682 is a no-op.
//   symmetric: |w| <= 2^(b-1) |s| always (s = m / 2^(b-1) exactly), so codes lie in
//     [-2^(b-1), 2^(b-1)]: the lower bound never binds, the upper one does whenever the weaker
//     extreme is within half a step of the stronger one, so it is always applied (need_clamp only
//     reports non-finite scales);
//   asymmetric: with an unclipped zero point, q + zp lies in [-0.5, levels - 1 + f + 2e-4] where
//     f = min/s - round(min/s); the top rounds out of range only if f is within ~1e-4 of 0.5.
// RN(a / b) for a divisor b whose correctly rounded reciprocal rb is known (Markstein): exact when
// nothing under/overflows, which holds for b in [2^-23, 2^125] and |a / b| >= 2^-80; smaller
// quotients are off by at most an ulp of a number that rounds to code 0 anyway, and quotients that
// overflow give NaN instead of inf, which the clip maps to the same bound.
__device__ __forceinline__ float exact_quotient(float a, float b, float rb) {
  const float q0 = __fmul_rn(a, rb);
  const float e = __fmaf_rn(-b, q0, a);
  return __fmaf_rn(e, rb, q0);
}

template <int MODE>
__device__ __forceinline__ void int_params(float mn, float mx, float& s, float& r, float& zp, bool& need_clamp) {
  constexpr int kBits = mode_bits(MODE);
  if constexpr (mode_is_asym(MODE)) {
    constexpr int kHigh = (1 << kBits) - 1;
    constexpr float kLevels = static_cast<float>(kHigh);
    constexpr float kRcpLevels = 1.0f / kLevels;  // correctly rounded at compile time
    s = exact_quotient(__fsub_rn(mx, mn), kLevels, kRcpLevels);
    s = (fabsf(s) < kEps32) ? kEps32 : s;
    r = __frcp_rn(s);
    const float qm = exact_quotient(mn, s, r);
    const float rq = rintf(qm);
    const float z = __fsub_rn(0.0f, rq);
    const float zc = fminf(fmaxf(z, 0.0f), kLevels);
    zp = zc + 0.0f;  // -0 -> +0
    need_clamp = !(zc == z) || !(__fsub_rn(qm, rq) < 0.49f);
  } else {
    // where(|min| >= max, |min|, -max) / 2^(b-1): the division by a power of two is a multiply
    const float amin = fabsf(mn);
    s = ((amin >= mx) ? amin : -mx) * (1.0f / static_cast<float>(1 << (kBits - 1)));
    s = (fabsf(s) < kEps32) ? kEps32 : s;
    r = __frcp_rn(s);
    zp = 0.0f;
    need_clamp = false;  // the upper bound is always applied, the lower one never binds
  }
}

// ---- float (code-book) modes ---------------------------------------------------------------------------
// NF4 index = number of the reference's 15 decision boundaries (WC/constants.py:84-103) strictly below the
// quotient q in [-1, 1] (searchsorted side='left', WC/weight_lowering.py:574), without a search:
//   k = rint(7 + q * (c1 + q * (c2 + q * c3)))   -- a cubic through the boundaries, three packed FMAs, the
//       last one adding 1.5 * 2^23 + 7 so that k lands in the low mantissa bits;
//   index = k + (q > bound[k])                   -- bound[] is spread over the lanes of the warp, one shuffle.
// The cubic keeps k in {index - 1, index} for every real q in [-1, 1] with 0.034 to spare (fp32 evaluation
// error is below 1e-5), so comparing against the single boundary bound[k] decides the index exactly; k = -1
// reads lane 31, which holds -inf.  tests/test_kernel_constants.py re-derives that margin from these constants.
// The comparison itself is done on the FMA pipe instead of a compare and a predicated add (the integer / compare
// pipe issues at half rate and is this kernel's busiest): the lanes hold -bound * 2^40, and
//   c = saturate(q * 2^40 + (-bound * 2^40))     -- one fused multiply-add, rounded once
// is exactly 1.0f when q > bound and 0.0f otherwise: the scaled difference is exact up to its single rounding,
// it is zero only for q == bound, and two distinct floats near a boundary (|bound| >= 0.039) differ by at least
// 2^-28, i.e. by 2^12 after scaling.  c is then added to the float that carries k in its mantissa.
constexpr float kNf4PolyC1 = 11.72690251f, kNf4PolyC2 = -0.51709913f, kNf4PolyC3 = -4.67530535f;
constexpr float kLutNone = 3.0e38f;
__device__ __constant__ const float kNf4LutBound[32] = {
    -0.8480964303016663f, -0.6106328964233398f, -0.4599952697753906f, -0.33967941999435425f,
    -0.23460739850997925f, -0.13791173696517944f, -0.045525018125772476f, 0.03979014977812767f,
    0.1202552542090416f, 0.2035212516784668f, 0.2920137643814087f, 0.3893125355243683f,
    0.5016633868217468f, 0.6427869200706482f, 0.8614783883094788f, kLutNone,
    kLutNone, kLutNone, kLutNone, kLutNone, kLutNone, kLutNone, kLutNone, kLutNone,
    kLutNone, kLutNone, kLutNone, kLutNone, kLutNone, kLutNone, kLutNone, -kLutNone};
constexpr float kNf4CmpScale = 1099511627776.0f;  // 2^40
// what lane `l` holds for the comparison: -bound[l] * 2^40 (exact), +-1e30 for "no boundary" / "-inf"
__device__ __forceinline__ float nf4_lane_operand(int l) {
  const float b = kNf4LutBound[l];
  if (b > 1.0e38f) return -1.0e30f;   // q > +inf is never true: c = 0
  if (b < -1.0e38f) return 1.0e30f;   // q > -inf is always true: c = 1
  return -b * kNf4CmpScale;
}

__host__ __device__ constexpr bool mode_is_fast_float(int m) {
  return m == NNCFB_NF4 || m == NNCFB_FP4 || m == NNCFB_MXFP4 || m == NNCFB_FP8_E4M3 || m == NNCFB_MXFP8_E4M3;
}

// Scale of a float-mode group, WC/weight_lowering.py:106-126: max|w| (/ 6 for E2M1, / 448 for E4M3), eps guard,
// power of two for MX.  `r` is the correctly rounded reciprocal (exact for a power of two).
template <int MODE>
__device__ __forceinline__ void float_params(float mn, float mx, float& s, float& r, int& e8) {
  float a = fmaxf(fabsf(mn), fabsf(mx));
  if constexpr (MODE == NNCFB_FP4 || MODE == NNCFB_MXFP4) a = exact_quotient(a, 6.0f, 1.0f / 6.0f);
  if constexpr (MODE == NNCFB_FP8_E4M3 || MODE == NNCFB_MXFP8_E4M3) a = exact_quotient(a, 448.0f, 1.0f / 448.0f);
  a = (a < kEps32) ? kEps32 : a;
  e8 = 0;
  if constexpr (mode_is_mx(MODE)) {
    e8 = e8m0_exponent(a);
    s = exp2_int(e8);
    r = exp2_int(-e8);
  } else {
    s = a;
    r = __frcp_rn(a);
  }
}

// Value of `v` held by lane (index & 31).  Written as PTX so that the index, which keeps the 1.5 * 2^23
// pattern in its high bits and is used again as a Horner digit, carries no lane-range assumption.
__device__ __forceinline__ float shfl_low5(float v, uint32_t index) {
  float r;
  asm volatile("shfl.sync.idx.b32 %0, %1, %2, 0x1f, 0xffffffff;" : "=f"(r) : "f"(v), "r"(index));
  return r;
}

// Nibble codes of 8 elements: NF4 table index, or E2M1 bit pattern sign|index (zero is stored as +0).
// E2M1 uses the hardware conversion cvt.rn.satfinite.e2m1x2.f32: round to nearest, ties to the even
// mantissa, saturation at 6 - the rule WC/weight_lowering.py:577-583 implements on its 15-entry table.
template <int MODE>
__device__ __forceinline__ uint32_t encode8_float(const float2 (&v)[4], float s, float r, float lut_operand) {
  const float2 r2 = f2(r, r), ns2 = f2(-s, -s);
  float2 q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (MODE == NNCFB_MXFP4) {
      q[i] = __fmul2_rn(v[i], r2);  // the scale is a power of two: one multiply is the exact quotient
    } else {
      const float2 q0 = __fmul2_rn(v[i], r2);
      const float2 e = __ffma2_rn(ns2, q0, v[i]);
      q[i] = __ffma2_rn(e, r2, q0);
    }
  }
  if constexpr (MODE == NNCFB_NF4) {
    const float2 c1 = f2(kNf4PolyC1, kNf4PolyC1), c2 = f2(kNf4PolyC2, kNf4PolyC2), c3 = f2(kNf4PolyC3, kNf4PolyC3);
    const float2 m7 = f2(12582919.0f, 12582919.0f);
    uint32_t acc = 0;
#pragma unroll
    for (int i = 3; i >= 0; --i) {
      float2 h = __ffma2_rn(q[i], c3, c2);
      h = __ffma2_rn(h, q[i], c1);
      const float2 t = __ffma2_rn(h, q[i], m7);
      uint32_t kx = __float_as_uint(t.x), ky = __float_as_uint(t.y);
      // Opaque to the optimiser from here on: when it can see that kx and ky are the halves of one packed
      // result it was observed (nvcc 12.9, sm_100a) to place digits of the sum below in the wrong nibble.
      asm("" : "+r"(kx), "+r"(ky));
      const float lx = shfl_low5(lut_operand, kx);
      const float ly = shfl_low5(lut_operand, ky);
      const float cx = __saturatef(__fmaf_rn(q[i].x, kNf4CmpScale, lx));   // 1.0f iff q > bound[k]
      const float cy = __saturatef(__fmaf_rn(q[i].y, kNf4CmpScale, ly));
      acc = acc * 16u + __float_as_uint(__fadd_rn(__uint_as_float(ky), cy));
      acc = acc * 16u + __float_as_uint(__fadd_rn(__uint_as_float(kx), cx));
    }
    return acc - kMagicBits * 0x11111111u;
  } else {
    uint32_t w;
    asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
        "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
        : "=r"(w)
        : "f"(q[0].x), "f"(q[0].y), "f"(q[1].x), "f"(q[1].y), "f"(q[2].x), "f"(q[2].y), "f"(q[3].x), "f"(q[3].y));
    // a negative value that rounds to zero is stored as +0: drop the sign of nibbles with zero magnitude
    const uint32_t m = w & 0x77777777u;
    const uint32_t nz = (m | (m >> 1) | (m >> 2)) & 0x11111111u;
    return w & (0x77777777u | (nz * 8u));
  }
}

// E4M3 bytes of 8 elements, WC/fp8_conversion.py:43-228: the quotient is rounded to fp16 and from there to E4M3,
// both to nearest even - the two hardware conversions below.  With the scale taken from the group itself the
// quotient never exceeds 448, so the reference's "beyond 448 becomes NaN" rule and the conversion's saturation
// cannot differ; fp16 subnormals (below 2^-14, far under half the smallest E4M3 step 2^-9) become signed zero
// in both.
template <int MODE>
__device__ __forceinline__ uint2 encode8_fp8(const float2 (&v)[4], float s, float r) {
  const float2 r2 = f2(r, r), ns2 = f2(-s, -s);
  uint32_t b[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 q;
    if constexpr (mode_is_mx(MODE)) {
      q = __fmul2_rn(v[i], r2);  // the scale is a power of two: one multiply is the exact quotient
    } else {
      const float2 q0 = __fmul2_rn(v[i], r2);
      const float2 e = __ffma2_rn(ns2, q0, v[i]);
      q = __ffma2_rn(e, r2, q0);
    }
    const __half2 h = __floats2half2_rn(q.x, q.y);
    uint16_t pair;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(pair) : "r"(*reinterpret_cast<const uint32_t*>(&h)));
    b[i] = pair;  // low byte = element 2 i, high byte = element 2 i + 1
  }
  uint2 out;
  out.x = b[0] | (b[1] << 16);
  out.y = b[2] | (b[3] << 16);
  return out;
}

// =====================================================================================================
// Batched row-group kernel: group_size = 8 * L * VPL (L lanes, VPL 16-byte vectors per lane; lane j
// owns vectors j, j+L, ... of its group so that every warp load and store is fully coalesced).
// =====================================================================================================
// One warp iteration: U * (32 / L) consecutive groups of one tensor.  FULL: every group exists (all but
// the last iteration of a tensor), so the loads, the code stores and the zero fill need no predicates.
template <typename SrcT, int MODE, int L, int VPL, int U, bool FULL>
__device__ __forceinline__ void rows_iteration(const FastTensor& T, const int64_t g0, const int lig, const float lut_bound) {
  constexpr int GPW = 32 / L;
  constexpr int GS = 8 * L * VPL;
  const SrcT* __restrict__ src = reinterpret_cast<const SrcT*>(T.weight);
  const int64_t n_groups = T.n_groups;

  Raw8<SrcT> raw[U][VPL];
#pragma unroll
  for (int p = 0; p < U; ++p) {
    const int64_t g = g0 + p * GPW;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if constexpr (FULL) {
        raw[p][v] = load_raw8<SrcT>(src + g * GS + (lig + v * L) * 8);
      } else {
        raw[p][v] = g < n_groups ? load_raw8<SrcT>(src + g * GS + (lig + v * L) * 8) : zero_raw8<SrcT>();
      }
    }
  }
  // Symmetric integer parameters are a handful of instructions: there the gather costs what it saves.
  if constexpr (GPW * U <= 32 && (mode_is_asym(MODE) || mode_is_fast_float(MODE))) {
    // The iteration's GPW * U groups are consecutive: group (pass p, sub-warp j) = first + p * GPW + j.  Their
    // parameters are computed ONCE, by lane p * GPW + j, instead of once per pass with every lane of a sub-warp
    // repeating the same arithmetic: the reduced (min, -max) pairs are gathered with one shuffle per pass, the
    // parameters go back with three, and scales / zero points leave as one coalesced store.
    const int lane = threadIdx.x & 31;
    const int sub = lane / L;
    MinNegMax mine;
    mine.packed = 0u;
    mine.mn = mine.nmx = 0.0f;
#pragma unroll
    for (int p = 0; p < U; ++p) {
      MinNegMax m = min_negmax<SrcT, VPL>(raw[p]);
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) reduce_step<SrcT>(m, o);
      const int src_lane = (lane % GPW) * L;  // any lane of sub-warp lane % GPW holds that group's result
      MinNegMax t;
      if constexpr (sizeof(SrcT) == 2) {
        t.packed = __shfl_sync(0xffffffffu, m.packed, src_lane);
        t.mn = t.nmx = 0.0f;
      } else {
        t.packed = 0u;
        t.mn = __shfl_sync(0xffffffffu, m.mn, src_lane);
        t.nmx = __shfl_sync(0xffffffffu, m.nmx, src_lane);
      }
      if (lane / GPW == p) mine = t;
    }
    const int64_t first = g0 - sub;                 // first group of the iteration (warp-uniform)
    const bool owner = lane < GPW * U && (FULL || first + lane < n_groups);
    float mn, mx, s, r, zp = 0.0f;
    bool need_clamp = false;
    int e8 = 0;
    finish_minmax<SrcT>(mine, mn, mx);
    if constexpr (mode_is_fast_float(MODE)) {
      float_params<MODE>(mn, mx, s, r, e8);
    } else {
      int_params<MODE>(mn, mx, s, r, zp, need_clamp);
    }
    bool clamp = false;
    if constexpr (mode_is_asym(MODE)) clamp = __any_sync(0xffffffffu, need_clamp && owner);
    // zero point of the next group (lane + 1): the two nibbles of a byte of the packed zero points; `first` and
    // the number of owner lanes are even, so an even lane always owns an even group
    float zp_next = 0.0f;
    if constexpr (mode_is_asym(MODE) && mode_bits(MODE) == 4) zp_next = __shfl_down_sync(0xffffffffu, zp, 1);
    if (owner) {
      const int64_t g = first + lane;
      if constexpr (mode_is_fast_float(MODE)) {
        if (T.scale) T.scale[g] = s;
      } else {
        T.scale[g] = s;
      }
      if (T.scale_f16) T.scale_f16[g] = __half_as_ushort(__float2half_rn(s));
      if constexpr (mode_is_asym(MODE)) {
        if (T.zp) T.zp[g] = static_cast<int32_t>(zp);
        if (T.zp_packed) {
          if constexpr (mode_bits(MODE) == 4) {
            if ((lane & 1) == 0) {
              const bool has_next = FULL || g + 1 < n_groups;
              const uint32_t hi = has_next ? static_cast<uint32_t>(static_cast<int32_t>(zp_next)) : 0u;
              T.zp_packed[g >> 1] = static_cast<uint8_t>(static_cast<uint32_t>(static_cast<int32_t>(zp)) | (hi << 4));
            }
          } else {
            T.zp_packed[g] = static_cast<uint8_t>(static_cast<int32_t>(zp));
          }
        }
      }
      if constexpr (mode_is_mx(MODE)) {
        if (T.e8m0) T.e8m0[g] = static_cast<uint8_t>(e8 + 127);
      }
    }
#pragma unroll
    for (int p = 0; p < U; ++p) {
      const int64_t g = g0 + p * GPW;
      const bool valid = FULL || g < n_groups;
      const int owner_lane = p * GPW + sub;
      const float sp = __shfl_sync(0xffffffffu, s, owner_lane);
      const float rp = __shfl_sync(0xffffffffu, r, owner_lane);
      if constexpr (mode_is_fast_float(MODE)) {
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          float2 x[4];
          unpack8_pairs(raw[p][v], x);
          if constexpr (mode_bits(MODE) == 8) {
            const uint2 w = encode8_fp8<MODE>(x, sp, rp);
            if (valid) __stcs(reinterpret_cast<uint2*>(T.codes + (g * GS + (lig + v * L) * 8)), w);
          } else {
            const uint32_t w = encode8_float<MODE>(x, sp, rp, lut_bound);  // shuffles inside: all lanes
            if (valid) __stcs(reinterpret_cast<uint32_t*>(T.codes + ((g * GS + (lig + v * L) * 8) >> 1)), w);
          }
        }
      } else {
        float zpp = 0.0f;
        if constexpr (mode_is_asym(MODE)) zpp = __shfl_sync(0xffffffffu, zp, owner_lane);
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          float2 x[4];
          unpack8_pairs(raw[p][v], x);
          uint2 w;
          if constexpr (mode_is_asym(MODE)) {
            w = clamp ? encode8_int<MODE, 2>(x, sp, rp, zpp) : encode8_int<MODE, 0>(x, sp, rp, zpp);
          } else {
            w = encode8_int<MODE, 1>(x, sp, rp, zpp);
          }
          if (valid) {
            const int64_t e0 = g * GS + (lig + v * L) * 8;
            if constexpr (mode_bits(MODE) == 4) {
              __stcs(reinterpret_cast<uint32_t*>(T.codes + (e0 >> 1)), w.x);
            } else {
              __stcs(reinterpret_cast<uint2*>(T.codes + e0), w);
            }
          }
        }
      }
    }
    return;
  }
#pragma unroll
  for (int p = 0; p < U; ++p) {
    const int64_t g = g0 + p * GPW;
    const bool valid = FULL || g < n_groups;
    MinNegMax m = min_negmax<SrcT, VPL>(raw[p]);
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) reduce_step<SrcT>(m, o);
    float mn, mx, s, r, zp;
    bool need_clamp;
    finish_minmax<SrcT>(m, mn, mx);
    if constexpr (mode_is_fast_float(MODE)) {
      int e8;
      float_params<MODE>(mn, mx, s, r, e8);
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        float2 x[4];
        unpack8_pairs(raw[p][v], x);
        if constexpr (mode_bits(MODE) == 8) {
          const uint2 w = encode8_fp8<MODE>(x, s, r);
          if (valid) __stcs(reinterpret_cast<uint2*>(T.codes + (g * GS + (lig + v * L) * 8)), w);
        } else {
          const uint32_t w = encode8_float<MODE>(x, s, r, lut_bound);  // shuffles inside: all lanes
          if (valid) __stcs(reinterpret_cast<uint32_t*>(T.codes + ((g * GS + (lig + v * L) * 8) >> 1)), w);
        }
      }
      if (valid && lig == 0) {
        if (T.scale) T.scale[g] = s;
        if (T.scale_f16) T.scale_f16[g] = __half_as_ushort(__float2half_rn(s));
        if constexpr (mode_is_mx(MODE)) {
          if (T.e8m0) T.e8m0[g] = static_cast<uint8_t>(e8 + 127);
        }
      }
    } else {
      int_params<MODE>(mn, mx, s, r, zp, need_clamp);
      bool clamp = false;
      if constexpr (mode_is_asym(MODE)) clamp = __any_sync(0xffffffffu, need_clamp);
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        float2 x[4];
        unpack8_pairs(raw[p][v], x);
        uint2 w;
        if constexpr (mode_is_asym(MODE)) {
          w = clamp ? encode8_int<MODE, 2>(x, s, r, zp) : encode8_int<MODE, 0>(x, s, r, zp);
        } else {
          w = encode8_int<MODE, 1>(x, s, r, zp);
        }
        if (valid) {
          const int64_t e0 = g * GS + (lig + v * L) * 8;
          if constexpr (mode_bits(MODE) == 4) {
            __stcs(reinterpret_cast<uint32_t*>(T.codes + (e0 >> 1)), w.x);
          } else {
            __stcs(reinterpret_cast<uint2*>(T.codes + e0), w);
          }
        }
      }
      const int sub = (threadIdx.x & 31) / L;
      float zp_next = 0.0f;   // zero point of group g + 1, owned by the next sub-warp (g is even iff `sub` is)
      if constexpr (mode_is_asym(MODE) && mode_bits(MODE) == 4) zp_next = __shfl_sync(0xffffffffu, zp, (sub | 1) * L);
      if (valid && lig == 0) {
        T.scale[g] = s;
        if (T.scale_f16) T.scale_f16[g] = __half_as_ushort(__float2half_rn(s));
        if constexpr (mode_is_asym(MODE)) {
          if (T.zp) T.zp[g] = static_cast<int32_t>(zp);
          if (T.zp_packed) {
            if constexpr (mode_bits(MODE) == 4) {
              if ((sub & 1) == 0) {
                const bool has_next = FULL || g + 1 < n_groups;
                const uint32_t hi = has_next ? static_cast<uint32_t>(static_cast<int32_t>(zp_next)) : 0u;
                T.zp_packed[g >> 1] = static_cast<uint8_t>(static_cast<uint32_t>(static_cast<int32_t>(zp)) | (hi << 4));
              }
            } else {
              T.zp_packed[g] = static_cast<uint8_t>(static_cast<int32_t>(zp));
            }
          }
        }
      }
    }
  }
}

template <typename SrcT, int MODE, int L, int VPL, int U>
__global__ void __launch_bounds__(256, NNCFB_ROWS_MINBLOCKS) quant_rows_batch_kernel(const __grid_constant__ FastBatch b) {
  constexpr int GPW = 32 / L;
  const int lane = threadIdx.x & 31;
  const int sub = lane / L;
  const int lig = lane % L;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t total_iters = b.iter_start[b.n_tensors];
  int lo = 0;  // tensor of the current iteration; iterations only move forward
  float lut_bound = 0.0f;
  if constexpr (MODE == NNCFB_NF4) lut_bound = nf4_lane_operand(lane);

  for (int64_t it = warp; it < total_iters; it += n_warps) {
    while (b.iter_start[lo + 1] <= it) ++lo;
    const FastTensor& T = b.t[lo];
    const int64_t first = (it - b.iter_start[lo]) * (GPW * U);  // warp-uniform
    if (first + GPW * U <= T.n_groups) {
      rows_iteration<SrcT, MODE, L, VPL, U, true>(T, first + sub, lig, lut_bound);
    } else {
      rows_iteration<SrcT, MODE, L, VPL, U, false>(T, first + sub, lig, lut_bound);
    }
  }
}

// =====================================================================================================
// Batched per-channel kernel (one group per row, row length % 8 == 0): TPR threads per row keep the
// row in registers (K vectors each); rows longer than TPR*K*8 re-read the tail from L2.
// =====================================================================================================
// One block iteration of the per-channel kernel: 256 / TPR rows.  FULL: every row exists and the row is
// exactly the TPR * K vectors the threads hold, so nothing is predicated and there is no tail loop.
template <typename SrcT, int MODE, int TPR, bool FULL>
__device__ __forceinline__ void channel_iteration(const FastTensor& T, const int64_t g, const int64_t row_len,
                                                  uint32_t* red16, float* red_mn, float* red_nmx) {
  constexpr int K = WideCache<SrcT>::K;
  constexpr int WPR = TPR / 32;   // warps per row
  const int tir = threadIdx.x % TPR;
  const int warp_in_block = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int first_warp = (threadIdx.x / TPR) * WPR;
  const int64_t nvec = row_len >> 3;
  const bool valid = FULL || g < T.n_groups;
  const SrcT* __restrict__ row = reinterpret_cast<const SrcT*>(T.weight) + (valid ? g : 0) * row_len;

  Raw8<SrcT> cache[K];
  bool have[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int64_t j = tir + static_cast<int64_t>(k) * TPR;
    have[k] = FULL || (valid && j < nvec);
    if constexpr (FULL) cache[k] = load_raw8<SrcT>(row + j * 8);
    else cache[k] = have[k] ? load_raw8<SrcT>(row + j * 8) : zero_raw8<SrcT>();
  }
  // thread-local (min, -max), starting from the neutral element (+inf, +inf) so that vectors which
  // do not exist contribute nothing
  MinNegMax m;
  if constexpr (std::is_same<SrcT, __nv_bfloat16>::value) m.packed = 0x7f807f80u;
  else if constexpr (std::is_same<SrcT, __half>::value) m.packed = 0x7c007c00u;
  else m.packed = 0u;
  m.mn = __uint_as_float(0x7f800000u);
  m.nmx = __uint_as_float(0x7f800000u);
  auto fold = [&m](const Raw8<SrcT>& vec) {
    Raw8<SrcT> one[1] = {vec};
    const MinNegMax x = min_negmax<SrcT, 1>(one);
    if constexpr (sizeof(SrcT) == 2) {
      using V2 = typename std::conditional<std::is_same<SrcT, __half>::value, __half2, __nv_bfloat162>::type;
      const V2 y = __hmin2(*reinterpret_cast<const V2*>(&m.packed), *reinterpret_cast<const V2*>(&x.packed));
      m.packed = *reinterpret_cast<const uint32_t*>(&y);
    } else {
      m.mn = fminf(m.mn, x.mn);
      m.nmx = fminf(m.nmx, x.nmx);
    }
  };
  if constexpr (FULL) {
    m = min_negmax<SrcT, K>(cache);  // all K vectors at once: the (min, -max) packing is paid once
  } else {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (have[k]) fold(cache[k]);
    }
    for (int64_t j = tir + static_cast<int64_t>(K) * TPR; valid && j < nvec; j += TPR) fold(load_raw8<SrcT>(row + j * 8));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) reduce_step<SrcT>(m, o);
  if (lane == 0) {
    red16[warp_in_block] = m.packed;
    red_mn[warp_in_block] = m.mn;
    red_nmx[warp_in_block] = m.nmx;
  }
  __syncthreads();
  float mn, mx;
  {
    MinNegMax t;
    t.packed = red16[first_warp];
    t.mn = red_mn[first_warp];
    t.nmx = red_nmx[first_warp];
#pragma unroll
    for (int w = 1; w < WPR; ++w) {
      if constexpr (sizeof(SrcT) == 2) {
        using V2 = typename std::conditional<std::is_same<SrcT, __half>::value, __half2, __nv_bfloat162>::type;
        const uint32_t o = red16[first_warp + w];
        const V2 y = __hmin2(*reinterpret_cast<const V2*>(&t.packed), *reinterpret_cast<const V2*>(&o));
        t.packed = *reinterpret_cast<const uint32_t*>(&y);
      } else {
        t.mn = fminf(t.mn, red_mn[first_warp + w]);
        t.nmx = fminf(t.nmx, red_nmx[first_warp + w]);
      }
    }
    finish_minmax<SrcT>(t, mn, mx);
  }
  float s, r, zp;
  bool clamp;  // uniform over the row, hence over the warp (TPR >= 32)
  int_params<MODE>(mn, mx, s, r, zp, clamp);
  auto encode = [&](const float2 (&x)[4]) -> uint2 {
    if constexpr (mode_is_asym(MODE)) {
      return clamp ? encode8_int<MODE, 2>(x, s, r, zp) : encode8_int<MODE, 0>(x, s, r, zp);
    } else {
      return encode8_int<MODE, 1>(x, s, r, zp);
    }
  };
#pragma unroll
  for (int k = 0; k < K; ++k) {
    if (have[k]) {
      const int64_t j = tir + static_cast<int64_t>(k) * TPR;
      float2 x[4];
      unpack8_pairs(cache[k], x);
      const uint2 w = encode(x);
      const int64_t e0 = g * row_len + j * 8;
      if constexpr (mode_bits(MODE) == 4) {
        __stcs(reinterpret_cast<uint32_t*>(T.codes + (e0 >> 1)), w.x);
      } else {
        __stcs(reinterpret_cast<uint2*>(T.codes + e0), w);
      }
    }
  }
  for (int64_t j = tir + static_cast<int64_t>(K) * TPR; !FULL && valid && j < nvec; j += TPR) {
    float2 x[4];
    unpack8_pairs(load_raw8<SrcT>(row + j * 8), x);
    const uint2 w = encode(x);
    const int64_t e0 = g * row_len + j * 8;
    if constexpr (mode_bits(MODE) == 4) {
      __stcs(reinterpret_cast<uint32_t*>(T.codes + (e0 >> 1)), w.x);
    } else {
      __stcs(reinterpret_cast<uint2*>(T.codes + e0), w);
    }
  }
  if (valid && tir == 0) {
    T.scale[g] = s;
    if (T.scale_f16) T.scale_f16[g] = __half_as_ushort(__float2half_rn(s));
    if constexpr (mode_is_asym(MODE)) {
      if (T.zp) T.zp[g] = static_cast<int32_t>(zp);
      if constexpr (mode_bits(MODE) == 8) {
        if (T.zp_packed) T.zp_packed[g] = static_cast<uint8_t>(static_cast<int32_t>(zp));
      }
    }
  }
}

template <typename SrcT, int MODE, int TPR>
__global__ void __launch_bounds__(256, 3) quant_channel_batch_kernel(const __grid_constant__ FastBatch b,
                                                                     const int64_t row_len) {
  constexpr int K = WideCache<SrcT>::K;
  constexpr int RPB = 256 / TPR;  // rows per block
  __shared__ uint32_t red16[8];
  __shared__ float red_mn[8], red_nmx[8];
  const int rib = threadIdx.x / TPR;
  const bool whole_row = (row_len >> 3) == static_cast<int64_t>(K) * TPR;
  const int64_t total_iters = b.iter_start[b.n_tensors];  // iterations of RPB rows

  int lo = 0;
  for (int64_t it = blockIdx.x; it < total_iters; it += gridDim.x) {
    while (b.iter_start[lo + 1] <= it) ++lo;
    const FastTensor& T = b.t[lo];
    const int64_t first = (it - b.iter_start[lo]) * RPB;  // block-uniform
    if (whole_row && first + RPB <= T.n_groups) {
      channel_iteration<SrcT, MODE, TPR, true>(T, first + rib, row_len, red16, red_mn, red_nmx);
    } else {
      channel_iteration<SrcT, MODE, TPR, false>(T, first + rib, row_len, red16, red_mn, red_nmx);
    }
    __syncthreads();  // red* reused by the next iteration
  }
}

}  // namespace nncfb
