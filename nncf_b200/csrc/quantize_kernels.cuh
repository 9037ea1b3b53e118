// Fused group reduce -> scale / zero point -> quantise -> clamp -> pack kernels.
//
// One pass over the weight in HBM: every element is loaded once (16-byte streaming loads),
// the group statistics are reduced with warp shuffles, and codes, scales, zero points and the
// optional dequantised weight / squared error are written from registers.
//
// Layouts handled here (weight viewed as [outer, reduce, inner], see nncf_b200.h):
//   inner == 1  "row groups": a group is `group_size` consecutive elements
//       quant_subwarp_kernel  group_size in {8,16,...,256}: a sub-warp of group_size/8 lanes per group
//       quant_wide_kernel     group_size % 8 == 0 and >= 512: T threads per group, row kept in registers
//       quant_generic_kernel  any group size / alignment (scalar loads, two passes)
//   inner > 1   "column groups": groups strided by `inner`
//       quant_column_kernel   threads run along `inner` (coalesced), loop over the group
#pragma once

#include "nncfb_common.cuh"

namespace nncfb {

struct QArgs {
  const void* weight;
  const float* pre_scale;
  const void* pre_zp;
  int pre_zp_f32;
  uint8_t* codes;
  int codes_format;
  float* scale_out;
  int32_t* zp_out;
  uint8_t* zp_packed;  // stored form of the zero points (u8 per group, or two 4-bit groups per byte); zeroed by the host
  uint16_t* scale_f16;
  uint8_t* scale_e8m0;
  float* values;
  float* dq;
  float* sqerr;
  int64_t n_groups;  // outer * G * inner
  int64_t group_size;
  int64_t groups_per_row;  // G (column kernel)
  int64_t inner;
  int lanes_per_group;  // sub-warp kernel with a run-time group size
};

// ---- raw 8-element vectors ----------------------------------------------------------------------
template <typename T>
struct Raw8 {
  uint4 r;
};
template <>
struct Raw8<float> {
  float4 a, b;
};

template <typename T>
__device__ __forceinline__ Raw8<T> load_raw8(const T* __restrict__ p) {
  Raw8<T> x;
  x.r = __ldcs(reinterpret_cast<const uint4*>(p));
  return x;
}
template <>
__device__ __forceinline__ Raw8<float> load_raw8<float>(const float* __restrict__ p) {
  Raw8<float> x;
  x.a = __ldcs(reinterpret_cast<const float4*>(p));
  x.b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  return x;
}
template <typename T>
__device__ __forceinline__ Raw8<T> zero_raw8() {
  Raw8<T> x;
  x.r = make_uint4(0u, 0u, 0u, 0u);
  return x;
}
template <>
__device__ __forceinline__ Raw8<float> zero_raw8<float>() {
  Raw8<float> x;
  x.a = make_float4(0.f, 0.f, 0.f, 0.f);
  x.b = x.a;
  return x;
}

__device__ __forceinline__ void unpack8(const Raw8<float>& x, float (&v)[8]) {
  v[0] = x.a.x; v[1] = x.a.y; v[2] = x.a.z; v[3] = x.a.w;
  v[4] = x.b.x; v[5] = x.b.y; v[6] = x.b.z; v[7] = x.b.w;
}
__device__ __forceinline__ void unpack8(const Raw8<__nv_bfloat16>& x, float (&v)[8]) {
  const uint32_t w[4] = {x.r.x, x.r.y, x.r.z, x.r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void unpack8(const Raw8<__half>& x, float (&v)[8]) {
  const uint32_t w[4] = {x.r.x, x.r.y, x.r.z, x.r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// min and max of the 8 elements of a raw vector.  For the 16-bit types the comparison runs on
// packed pairs (exact: min/max never round) and only the two survivors are widened.
__device__ __forceinline__ void minmax8(const Raw8<float>& x, float& mn, float& mx) {
  mn = fminf(fminf(fminf(x.a.x, x.a.y), fminf(x.a.z, x.a.w)), fminf(fminf(x.b.x, x.b.y), fminf(x.b.z, x.b.w)));
  mx = fmaxf(fmaxf(fmaxf(x.a.x, x.a.y), fmaxf(x.a.z, x.a.w)), fmaxf(fmaxf(x.b.x, x.b.y), fmaxf(x.b.z, x.b.w)));
}
__device__ __forceinline__ void minmax8(const Raw8<__nv_bfloat16>& x, float& mn, float& mx) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&x.r);
  const __nv_bfloat162 lo = __hmin2(__hmin2(p[0], p[1]), __hmin2(p[2], p[3]));
  const __nv_bfloat162 hi = __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3]));
  mn = fminf(__low2float(lo), __high2float(lo));
  mx = fmaxf(__low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void minmax8(const Raw8<__half>& x, float& mn, float& mx) {
  const __half2* p = reinterpret_cast<const __half2*>(&x.r);
  const __half2 lo = __hmin2(__hmin2(p[0], p[1]), __hmin2(p[2], p[3]));
  const __half2 hi = __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3]));
  mn = fminf(__low2float(lo), __high2float(lo));
  mx = fmaxf(__low2float(hi), __high2float(hi));
}

// ---- per-group codec ------------------------------------------------------------------------------
// Holds the group's parameters and encodes one element at a time.
template <int MODE>
struct Codec {
  static constexpr bool kInt = mode_is_integer(MODE);
  static constexpr bool kAsym = mode_is_asym(MODE);
  static constexpr int kBits = mode_bits(MODE);
  static constexpr bool kMx = mode_is_mx(MODE);
  static constexpr int kLow = kAsym ? 0 : -(1 << (kBits - 1));
  static constexpr int kHigh = kAsym ? (1 << kBits) - 1 : (1 << (kBits - 1)) - 1;

  Divisor div;
  float scale;
  float zp;
  int e8m0;  // MX modes: exponent of the scale

  // parameters from the group's statistics
  __device__ __forceinline__ void from_stats(float mn, float mx) {
    zp = 0.0f;
    e8m0 = 0;
    if constexpr (kInt) {
      if constexpr (kAsym) {
        const GroupParams p = asym_params<kBits>(mn, mx);
        scale = p.scale;
        zp = p.zp;
      } else {
        scale = signed_scale<kBits>(mn, mx);
      }
    } else {
      // WC/weight_lowering.py:106-126: max|w| (/ format max unless NF4), eps guard, E8M0 for MX
      float s = fmaxf(fabsf(mn), fabsf(mx));
      if constexpr (MODE == NNCFB_MXFP4 || MODE == NNCFB_FP4) s = __fdiv_rn(s, 6.0f);
      if constexpr (MODE == NNCFB_FP8_E4M3 || MODE == NNCFB_MXFP8_E4M3) s = __fdiv_rn(s, 448.0f);
      s = (s < kEps32) ? kEps32 : s;
      if constexpr (kMx) {
        e8m0 = e8m0_exponent(s);
        s = exp2_int(e8m0);
      }
      scale = s;
    }
    div = make_divisor(scale);
  }

  __device__ __forceinline__ void from_given(float s, float z) {
    scale = s;
    zp = z;
    e8m0 = 0;
    if constexpr (kMx) {
      // biased exponent of a power-of-two scale (other values: nearest exponent below)
      e8m0 = static_cast<int>((__float_as_uint(s) >> 23) & 0xffu) - 127;
      e8m0 = max(e8m0, -127);
    }
    div = make_divisor(s);
  }

  // Returns the stored byte (two's complement int8 for symmetric integer modes) and the
  // unscaled decoded value u such that the dequantised weight is u * scale.
  __device__ __forceinline__ uint32_t encode(float w, float& unscaled) const {
    float q = div_by(w, div);
    if constexpr (kInt) {
      // WC/weight_lowering.py:678-682: w / scale, separate "+ zp", round half to even, clip
      if constexpr (kAsym) q = __fadd_rn(q, zp);
      q = rintf(q);
      q = fminf(fmaxf(q, static_cast<float>(kLow)), static_cast<float>(kHigh));
      const int c = static_cast<int>(q);
      unscaled = __fsub_rn(q, zp);  // (int32(q) - zp) as fp32, WC/weight_lowering.py:442-443
      return static_cast<uint32_t>(c) & 0xffu;
    } else if constexpr (MODE == NNCFB_NF4) {
      const int idx = nf4_index(q);
      unscaled = kNf4Levels[idx];
      return static_cast<uint32_t>(idx);
    } else if constexpr (MODE == NNCFB_MXFP4 || MODE == NNCFB_FP4) {
      const int idx = e2m1_index(fabsf(q));
      const float mag = e2m1_magnitude(idx);
      const bool neg = q < 0.0f && idx != 0;
      unscaled = neg ? -mag : mag;
      return static_cast<uint32_t>(idx) | (neg ? 8u : 0u);
    } else {
      const uint32_t b = e4m3_bits(q);
      unscaled = e4m3_value(b);
      return b;
    }
  }

  // nibble stored by NNCFB_CODES_NIBBLE (signed int4 gets the +8 offset of pack_int4)
  __device__ __forceinline__ static uint32_t nibble(uint32_t byte) {
    if constexpr (MODE == NNCFB_INT4_SYM) return (byte + 8u) & 15u;
    return byte & 15u;
  }
};

template <int MODE>
__device__ __forceinline__ void store_group_params(const QArgs& a, int64_t g, const Codec<MODE>& c) {
  if (a.scale_out) a.scale_out[g] = c.scale;
  if (a.scale_f16) a.scale_f16[g] = __half_as_ushort(__float2half_rn(c.scale));
  if constexpr (mode_is_asym(MODE)) {
    if (a.zp_out) a.zp_out[g] = static_cast<int32_t>(c.zp);
    if (a.zp_packed) {
      const uint32_t z = static_cast<uint32_t>(static_cast<int32_t>(c.zp));
      if constexpr (mode_bits(MODE) == 4) {
        // groups are owned by unrelated threads here: each ORs its nibble into the (zeroed) word that holds it
        atomicOr(reinterpret_cast<unsigned int*>(a.zp_packed) + (g >> 3), (z & 15u) << (4 * static_cast<int>(g & 7)));
      } else {
        a.zp_packed[g] = static_cast<uint8_t>(z);
      }
    }
  }
  if constexpr (mode_is_mx(MODE)) {
    if (a.scale_e8m0) a.scale_e8m0[g] = static_cast<uint8_t>(c.e8m0 + 127);
  }
}

__device__ __forceinline__ float load_pre_zp(const QArgs& a, int64_t g) {
  if (!a.pre_zp) return 0.0f;
  return a.pre_zp_f32 ? reinterpret_cast<const float*>(a.pre_zp)[g]
                      : static_cast<float>(reinterpret_cast<const int32_t*>(a.pre_zp)[g]);
}

// Encode 8 consecutive elements held by one lane and write every requested output.
// `e0` is the flat index of the first element (a multiple of 8).  Returns sum (dq - w)^2.
template <int MODE>
__device__ __forceinline__ float encode_store8(const QArgs& a, const Codec<MODE>& c, const float (&v)[8], int64_t e0) {
  uint32_t code[8];
  float u[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) code[i] = c.encode(v[i], u[i]);

  if (a.codes_format == NNCFB_CODES_NIBBLE) {
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) word |= Codec<MODE>::nibble(code[i]) << (4 * i);
    __stcs(reinterpret_cast<uint32_t*>(a.codes + (e0 >> 1)), word);
  } else if (a.codes_format == NNCFB_CODES_BYTE) {
    uint2 w2;
    w2.x = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
    w2.y = code[4] | (code[5] << 8) | (code[6] << 16) | (code[7] << 24);
    __stcs(reinterpret_cast<uint2*>(a.codes + e0), w2);
  }
  if (a.values) {
    __stcs(reinterpret_cast<float4*>(a.values + e0), make_float4(u[0], u[1], u[2], u[3]));
    __stcs(reinterpret_cast<float4*>(a.values + e0) + 1, make_float4(u[4], u[5], u[6], u[7]));
  }
  float err = 0.0f;
  if (a.dq || a.sqerr) {
    float d[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      d[i] = __fmul_rn(u[i], c.scale);
      const float t = __fsub_rn(d[i], v[i]);
      err = __fmaf_rn(t, t, err);
    }
    if (a.dq) {
      __stcs(reinterpret_cast<float4*>(a.dq + e0), make_float4(d[0], d[1], d[2], d[3]));
      __stcs(reinterpret_cast<float4*>(a.dq + e0) + 1, make_float4(d[4], d[5], d[6], d[7]));
    }
  }
  return err;
}

// =====================================================================================================
// Row groups, group_size = 8 * L with L in {1,2,4,8,16,32}: L lanes per group, 8 elements per lane,
// U independent 16-byte loads per lane in flight.  LT > 0 fixes L at compile time.
// =====================================================================================================
template <typename SrcT, int MODE, int LT, int U>
__global__ void __launch_bounds__(256) quant_subwarp_kernel(const QArgs a) {
  const int L = LT > 0 ? LT : a.lanes_per_group;
  const int gpw = 32 / L;  // groups per warp pass
  const int lane = threadIdx.x & 31;
  const int sub = lane / L;
  const int lig = lane - sub * L;  // lane in group
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t per_iter = static_cast<int64_t>(gpw) * U;
  const int64_t n_iters = (a.n_groups + per_iter - 1) / per_iter;
  const SrcT* __restrict__ src = reinterpret_cast<const SrcT*>(a.weight);
  const int64_t gs = static_cast<int64_t>(L) * 8;
  const bool pre = a.pre_scale != nullptr;

  for (int64_t it = warp; it < n_iters; it += n_warps) {
    const int64_t g0 = it * per_iter + sub;
    Raw8<SrcT> raw[U];
#pragma unroll
    for (int p = 0; p < U; ++p) {
      const int64_t g = g0 + static_cast<int64_t>(p) * gpw;
      raw[p] = g < a.n_groups ? load_raw8<SrcT>(src + g * gs + lig * 8) : zero_raw8<SrcT>();
    }
#pragma unroll
    for (int p = 0; p < U; ++p) {
      const int64_t g = g0 + static_cast<int64_t>(p) * gpw;
      const bool valid = g < a.n_groups;
      Codec<MODE> c;
      if (pre) {
        c.from_given(valid ? a.pre_scale[g] : 1.0f, valid ? load_pre_zp(a, g) : 0.0f);
      } else {
        float mn, mx;
        minmax8(raw[p], mn, mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          if (o < L) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          }
        }
        c.from_stats(mn, mx);
      }
      float v[8];
      unpack8(raw[p], v);
      float err = 0.0f;
      if (valid) err = encode_store8<MODE>(a, c, v, g * gs + lig * 8);
      if (a.sqerr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          if (o < L) err += __shfl_xor_sync(0xffffffffu, err, o);
        }
        if (valid && lig == 0) a.sqerr[g] = err;
      }
      if (valid && lig == 0) store_group_params<MODE>(a, g, c);
    }
  }
}

// =====================================================================================================
// Row groups, group_size % 8 == 0 and large (per-channel rows): T = threads_per_group threads of a
// 256-thread block share a group; each thread keeps up to K raw vectors in registers so the row is
// read from HBM once; vectors beyond the cache are read again (from L2).
// =====================================================================================================
template <typename SrcT>
struct WideCache {
  static constexpr int K = sizeof(SrcT) == 4 ? 4 : 8;
};

template <typename SrcT, int MODE>
__global__ void __launch_bounds__(256) quant_wide_kernel(const QArgs a, const int T) {
  constexpr int K = WideCache<SrcT>::K;
  __shared__ float red_mn[8], red_mx[8], red_err[8];
  const int gpb = 256 / T;  // groups per block
  const int tig = threadIdx.x % T;
  const int gib = threadIdx.x / T;
  const int warp_in_block = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int warps_per_group = T >> 5;
  const int first_warp = gib * warps_per_group;
  const SrcT* __restrict__ src = reinterpret_cast<const SrcT*>(a.weight);
  const int64_t gs = a.group_size;
  const int64_t nvec = gs >> 3;
  const int64_t n_blocks = (a.n_groups + gpb - 1) / gpb;
  const bool pre = a.pre_scale != nullptr;

  for (int64_t gb = blockIdx.x; gb < n_blocks; gb += gridDim.x) {
    const int64_t g = gb * gpb + gib;
    const bool valid = g < a.n_groups;
    const SrcT* row = src + (valid ? g : 0) * gs;
    Raw8<SrcT> cache[K];
    float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int64_t j = tig + static_cast<int64_t>(k) * T;
      if (valid && j < nvec) {
        cache[k] = load_raw8<SrcT>(row + j * 8);
      }
    }
    Codec<MODE> c;
    if (pre) {
      c.from_given(valid ? a.pre_scale[g] : 1.0f, valid ? load_pre_zp(a, g) : 0.0f);
    } else {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int64_t j = tig + static_cast<int64_t>(k) * T;
        if (valid && j < nvec) {
          float a0, b0;
          minmax8(cache[k], a0, b0);
          mn = fminf(mn, a0);
          mx = fmaxf(mx, b0);
        }
      }
      for (int64_t j = tig + static_cast<int64_t>(K) * T; valid && j < nvec; j += T) {
        float a0, b0;
        minmax8(load_raw8<SrcT>(row + j * 8), a0, b0);
        mn = fminf(mn, a0);
        mx = fmaxf(mx, b0);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      if (lane == 0) {
        red_mn[warp_in_block] = mn;
        red_mx[warp_in_block] = mx;
      }
      __syncthreads();
      mn = red_mn[first_warp];
      mx = red_mx[first_warp];
      for (int w = 1; w < warps_per_group; ++w) {
        mn = fminf(mn, red_mn[first_warp + w]);
        mx = fmaxf(mx, red_mx[first_warp + w]);
      }
      c.from_stats(mn, mx);
    }
    float err = 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int64_t j = tig + static_cast<int64_t>(k) * T;
      if (valid && j < nvec) {
        float v[8];
        unpack8(cache[k], v);
        err += encode_store8<MODE>(a, c, v, g * gs + j * 8);
      }
    }
    for (int64_t j = tig + static_cast<int64_t>(K) * T; valid && j < nvec; j += T) {
      float v[8];
      unpack8(load_raw8<SrcT>(row + j * 8), v);
      err += encode_store8<MODE>(a, c, v, g * gs + j * 8);
    }
    if (a.sqerr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
      if (lane == 0) red_err[warp_in_block] = err;
      __syncthreads();
      if (valid && tig == 0) {
        float e = 0.0f;
        for (int w = 0; w < warps_per_group; ++w) e += red_err[first_warp + w];
        a.sqerr[g] = e;
      }
    }
    if (valid && tig == 0) store_group_params<MODE>(a, g, c);
    __syncthreads();  // red_* are reused by the next iteration
  }
}

// =====================================================================================================
// Row groups of any size and alignment: one warp per group, scalar loads, two passes (the second
// one hits L1/L2).  Also the path for odd group sizes; nibble output needs an even group size.
// =====================================================================================================
template <typename SrcT, int MODE>
__global__ void __launch_bounds__(256) quant_generic_kernel(const QArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const SrcT* __restrict__ src = reinterpret_cast<const SrcT*>(a.weight);
  const int64_t gs = a.group_size;
  const bool pre = a.pre_scale != nullptr;

  for (int64_t g = warp; g < a.n_groups; g += n_warps) {
    const SrcT* row = src + g * gs;
    Codec<MODE> c;
    if (pre) {
      c.from_given(a.pre_scale[g], load_pre_zp(a, g));
    } else {
      float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
      for (int64_t i = lane; i < gs; i += 32) {
        const float w = to_f32<SrcT>(row[i]);
        mn = fminf(mn, w);
        mx = fmaxf(mx, w);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      c.from_stats(mn, mx);
    }
    float err = 0.0f;
    const int64_t e0 = g * gs;
    if (a.codes_format == NNCFB_CODES_NIBBLE) {
      // pairs (2i, 2i+1) of the group; gs is even (checked on the host)
      for (int64_t i = 2 * lane; i < gs; i += 64) {
        float u0, u1;
        const float w0 = to_f32<SrcT>(row[i]), w1 = to_f32<SrcT>(row[i + 1]);
        const uint32_t c0 = Codec<MODE>::nibble(c.encode(w0, u0));
        const uint32_t c1 = Codec<MODE>::nibble(c.encode(w1, u1));
        a.codes[(e0 + i) >> 1] = static_cast<uint8_t>(c0 | (c1 << 4));
        if (a.values) { a.values[e0 + i] = u0; a.values[e0 + i + 1] = u1; }
        if (a.dq || a.sqerr) {
          const float d0 = __fmul_rn(u0, c.scale), d1 = __fmul_rn(u1, c.scale);
          if (a.dq) { a.dq[e0 + i] = d0; a.dq[e0 + i + 1] = d1; }
          const float t0 = __fsub_rn(d0, w0), t1 = __fsub_rn(d1, w1);
          err = __fmaf_rn(t0, t0, err);
          err = __fmaf_rn(t1, t1, err);
        }
      }
    } else {
      for (int64_t i = lane; i < gs; i += 32) {
        float u;
        const float w = to_f32<SrcT>(row[i]);
        const uint32_t code = c.encode(w, u);
        if (a.codes_format == NNCFB_CODES_BYTE) a.codes[e0 + i] = static_cast<uint8_t>(code);
        if (a.values) a.values[e0 + i] = u;
        if (a.dq || a.sqerr) {
          const float d = __fmul_rn(u, c.scale);
          if (a.dq) a.dq[e0 + i] = d;
          const float t = __fsub_rn(d, w);
          err = __fmaf_rn(t, t, err);
        }
      }
    }
    if (a.sqerr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
      if (lane == 0) a.sqerr[g] = err;
    }
    if (lane == 0) store_group_params<MODE>(a, g, c);
  }
}

// =====================================================================================================
// Column groups (inner > 1; weights stored [in, out] or stacked experts [E, in, out]): thread t owns
// column pair / column c of one (outer, group) tile and walks the group_size rows, so that a warp
// reads 32 consecutive columns of each row (coalesced).  Two passes; the tile (group_size x 32
// columns) stays in L1/L2 between them.  Nibble output pairs neighbouring columns, so it needs an
// even `inner`; the thread then owns two columns.
// =====================================================================================================
template <typename SrcT, int MODE>
__global__ void __launch_bounds__(256) quant_column_kernel(const QArgs a) {
  const SrcT* __restrict__ src = reinterpret_cast<const SrcT*>(a.weight);
  const int64_t gs = a.group_size, inner = a.inner, G = a.groups_per_row;
  const bool nib = a.codes_format == NNCFB_CODES_NIBBLE;
  const int cpt = nib ? 2 : 1;  // columns per thread
  const int64_t col_threads = (inner + cpt - 1) / cpt;
  const int64_t n_tiles = a.n_groups / inner;  // outer * G
  const int64_t total = n_tiles * col_threads;
  const bool pre = a.pre_scale != nullptr;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t tile = t / col_threads;
    const int64_t c0 = (t - tile * col_threads) * cpt;
    const int64_t o = tile / G, gi = tile - o * G;
    const int64_t base = (o * G * gs + gi * gs) * inner;  // element (o, gi*gs, 0)
    Codec<MODE> cd[2];
    const int ncol = (c0 + 1 < inner && cpt == 2) ? 2 : 1;
    for (int k = 0; k < ncol; ++k) {
      const int64_t g = tile * inner + c0 + k;
      if (pre) {
        cd[k].from_given(a.pre_scale[g], load_pre_zp(a, g));
      } else {
        float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
        for (int64_t r = 0; r < gs; ++r) {
          const float w = to_f32<SrcT>(src[base + r * inner + c0 + k]);
          mn = fminf(mn, w);
          mx = fmaxf(mx, w);
        }
        cd[k].from_stats(mn, mx);
      }
    }
    float err[2] = {0.0f, 0.0f};
    for (int64_t r = 0; r < gs; ++r) {
      const int64_t e = base + r * inner + c0;
      uint32_t code[2] = {0u, 0u};
      for (int k = 0; k < ncol; ++k) {
        float u;
        const float w = to_f32<SrcT>(src[e + k]);
        code[k] = cd[k].encode(w, u);
        if (a.values) a.values[e + k] = u;
        if (a.dq || a.sqerr) {
          const float d = __fmul_rn(u, cd[k].scale);
          if (a.dq) a.dq[e + k] = d;
          const float tt = __fsub_rn(d, w);
          err[k] = __fmaf_rn(tt, tt, err[k]);
        }
      }
      if (nib) {
        a.codes[e >> 1] = static_cast<uint8_t>(Codec<MODE>::nibble(code[0]) | (Codec<MODE>::nibble(code[1]) << 4));
      } else if (a.codes_format == NNCFB_CODES_BYTE) {
        a.codes[e] = static_cast<uint8_t>(code[0]);
      }
    }
    for (int k = 0; k < ncol; ++k) {
      const int64_t g = tile * inner + c0 + k;
      if (a.sqerr) a.sqerr[g] = err[k];
      store_group_params<MODE>(a, g, cd[k]);
    }
  }
}

// =====================================================================================================
// Column groups, storage path (codes + parameters, computed from the weight): inner % 8 == 0.
// A 256-thread block owns a tile of 64 columns x one group: 8 column lanes of one 16-byte vector (8 columns)
// by 32 row lanes, so a warp reads four 128-byte row segments per load.  Each thread keeps its first K vectors
// in registers (groups of up to 32 * K rows are read from HBM once; longer ones - per-channel weights stored
// [in, out] - are read a second time for the encoding pass).  Per-column min / max are combined across the row
// lanes in shared memory; the per-column parameters come back through shared memory.
// =====================================================================================================
template <typename SrcT, int MODE>
__global__ void __launch_bounds__(256) quant_column_tile_kernel(const QArgs a) {
  constexpr int K = WideCache<SrcT>::K;
  __shared__ float red_mn[32][64], red_mx[32][64];
  __shared__ float par_scale[64], par_zp[64];
  const SrcT* __restrict__ src = reinterpret_cast<const SrcT*>(a.weight);
  const int64_t gs = a.group_size, inner = a.inner, G = a.groups_per_row;
  const int cl = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int64_t col_blocks = (inner + 63) / 64;
  const int64_t n_tiles = a.n_groups / inner;  // outer * G
  for (int64_t blk = blockIdx.x; blk < n_tiles * col_blocks; blk += gridDim.x) {
    const int64_t tile = blk / col_blocks, cb = blk - tile * col_blocks;
    const int64_t c0 = cb * 64 + cl * 8;
    const bool active = c0 < inner;  // whole vector: inner is a multiple of 8
    const int64_t o = tile / G, gi = tile - o * G;
    const int64_t base = (o * G * gs + gi * gs) * inner + c0;  // element (o, gi * gs, c0)

    float mn[8], mx[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mn[j] = __uint_as_float(0x7f800000u);
      mx[j] = __uint_as_float(0xff800000u);
    }
    auto fold = [&](const Raw8<SrcT>& raw) {
      float v[8];
      unpack8(raw, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mn[j] = fminf(mn[j], v[j]);
        mx[j] = fmaxf(mx[j], v[j]);
      }
    };
    Raw8<SrcT> cache[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int64_t r = rl + 32 * k;
      if (active && r < gs) {
        cache[k] = load_raw8<SrcT>(src + base + r * inner);
        fold(cache[k]);
      }
    }
    for (int64_t r = rl + 32 * K; active && r < gs; r += 32) fold(load_raw8<SrcT>(src + base + r * inner));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      red_mn[rl][cl * 8 + j] = mn[j];
      red_mx[rl][cl * 8 + j] = mx[j];
    }
    __syncthreads();
    if (threadIdx.x < 64) {
      const int col = threadIdx.x;
      float m = red_mn[0][col], M = red_mx[0][col];
#pragma unroll
      for (int q = 1; q < 32; ++q) {
        m = fminf(m, red_mn[q][col]);
        M = fmaxf(M, red_mx[q][col]);
      }
      if (cb * 64 + col < inner) {
        Codec<MODE> c;
        c.from_stats(m, M);
        store_group_params<MODE>(a, tile * inner + cb * 64 + col, c);
        par_scale[col] = c.scale;
        par_zp[col] = c.zp;
      }
    }
    __syncthreads();
    if (active && a.codes_format != NNCFB_CODES_NONE) {
      Codec<MODE> cd[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) cd[j].from_given(par_scale[cl * 8 + j], par_zp[cl * 8 + j]);
      auto encode = [&](const Raw8<SrcT>& raw, int64_t e) {
        float v[8];
        unpack8(raw, v);
        uint32_t code[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float u;
          code[j] = cd[j].encode(v[j], u);
        }
        if (a.codes_format == NNCFB_CODES_NIBBLE) {
          uint32_t w = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) w |= Codec<MODE>::nibble(code[j]) << (4 * j);
          *reinterpret_cast<uint32_t*>(a.codes + (e >> 1)) = w;
        } else {
          uint2 w;
          w.x = (code[0] & 255u) | ((code[1] & 255u) << 8) | ((code[2] & 255u) << 16) | ((code[3] & 255u) << 24);
          w.y = (code[4] & 255u) | ((code[5] & 255u) << 8) | ((code[6] & 255u) << 16) | ((code[7] & 255u) << 24);
          *reinterpret_cast<uint2*>(a.codes + e) = w;
        }
      };
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int64_t r = rl + 32 * k;
        if (r < gs) encode(cache[k], base + r * inner);
      }
      for (int64_t r = rl + 32 * K; r < gs; r += 32) encode(load_raw8<SrcT>(src + base + r * inner), base + r * inner);
    }
    __syncthreads();  // shared arrays are reused by the next tile
  }
}

}  // namespace nncfb
