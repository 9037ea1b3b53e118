// Weight decompression: packed codes + scale (+ zero point) -> fp16 / bf16 / fp32 weight.
//
// The run-time twin of the compression kernels, replacing the eager chain of the reference's
// decompressor modules (src/nncf/torch/quantization/layers.py:1334-1338, 1406-1416, 1453-1460:
// unpack_uint4 -> stack -> reshape -> type cast -> subtract -> multiply -> reshape -> cast) with one
// pass: 0.5 or 1 byte read and one output element written per weight.
//
// Integer modes reproduce the reference bit for bit: the arithmetic is done in fp16 like
// decompress_asymmetric / decompress_symmetric (src/nncf/torch/quantization/quantize_functions.py:389-414:
// (x.f16 - zp.f16) * scale.f16), then cast to the result dtype.  NF4 / E2M1 / E4M3 have no torch decompressor in
// the reference; they decode the format's value and multiply by the fp32 (or E8M0) scale in fp32.
#include <algorithm>

#include "nncfb_common.cuh"

namespace nncfb {

struct DecompressArgs {
  const uint8_t* codes;
  const void* scale;       // fp16 (integer modes), fp32 (NF4 / FP4) or E8M0 bytes (MXFP4) [n_groups]
  const uint8_t* zp;       // asym: u8 per group (INT8) or nibble-packed per group pair (INT4)
  void* out;
  int64_t n;               // elements
  int64_t group_size;
  int64_t vecs_per_group;  // group_size / 8 (vector kernel)
  int vec_shift;           // log2(vecs_per_group) when it is a power of two, else -1
  int mode;
  int out_dtype;
};

template <typename OutT>
__device__ __forceinline__ OutT cast_out(float v);
template <>
__device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 8 consecutive elements per thread and step (one 32-bit word of nibbles or two words of bytes); a group never
// ends inside a vector because group sizes handled here are multiples of 8.  Four steps are in flight per
// thread (their loads are issued before any arithmetic), a warp's loads and 16-byte stores are contiguous.
//
// Integer modes work on pairs of fp16 values: OR-ing a code c < 1024 into the bit pattern of 1024.0 gives the
// half 1024 + c exactly, so one packed subtraction yields (c - 8), (c - 128) or c as halves without a single
// integer-to-float conversion, then (x - zp) * scale as two packed fp16 operations - the reference's arithmetic
// (every intermediate is an integer below 2048, exact in fp16; the product is rounded once).
constexpr int kDecompressUnroll = 4;

__device__ __forceinline__ __half2 as_half2(uint32_t bits) { return *reinterpret_cast<const __half2*>(&bits); }

template <typename OutT>
__device__ __forceinline__ void store_pairs(OutT* dst, const __half2 (&r)[4], bool strided);
// r holds elements (0,1)(2,3)(4,5)(6,7), or (0,4)(1,5)(2,6)(3,7) when `strided` (the order nibbles unpack in)
template <>
__device__ __forceinline__ void store_pairs<__half>(__half* dst, const __half2 (&r)[4], bool strided) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = *reinterpret_cast<const uint32_t*>(&r[i]);
  uint4 o;
  if (strided) {
    o.x = __byte_perm(w[0], w[1], 0x5410);
    o.y = __byte_perm(w[2], w[3], 0x5410);
    o.z = __byte_perm(w[0], w[1], 0x7632);
    o.w = __byte_perm(w[2], w[3], 0x7632);
  } else {
    o = make_uint4(w[0], w[1], w[2], w[3]);
  }
  *reinterpret_cast<uint4*>(dst) = o;
}
template <>
__device__ __forceinline__ void store_pairs<__nv_bfloat16>(__nv_bfloat16* dst, const __half2 (&r)[4], bool strided) {
  float2 f[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = __half22float2(r[i]);
  __nv_bfloat162 o[4];
  if (strided) {
    o[0] = __floats2bfloat162_rn(f[0].x, f[1].x);
    o[1] = __floats2bfloat162_rn(f[2].x, f[3].x);
    o[2] = __floats2bfloat162_rn(f[0].y, f[1].y);
    o[3] = __floats2bfloat162_rn(f[2].y, f[3].y);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(f[i].x, f[i].y);
  }
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
}
template <>
__device__ __forceinline__ void store_pairs<float>(float* dst, const __half2 (&r)[4], bool strided) {
  float2 f[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = __half22float2(r[i]);
  if (strided) {
    *reinterpret_cast<float4*>(dst) = make_float4(f[0].x, f[1].x, f[2].x, f[3].x);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(f[0].y, f[1].y, f[2].y, f[3].y);
  } else {
    *reinterpret_cast<float4*>(dst) = make_float4(f[0].x, f[0].y, f[1].x, f[1].y);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(f[2].x, f[2].y, f[3].x, f[3].y);
  }
}

template <typename OutT, int MODE>
__global__ void __launch_bounds__(256, 8) decompress_kernel(const DecompressArgs a) {
  constexpr bool kFour = mode_bits(MODE) == 4;
  constexpr int U = kDecompressUnroll;
  const int64_t nvec = a.n >> 3;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v0 < nvec; v0 += U * stride) {
    uint2 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = v0 + u * stride;
      raw[u] = make_uint2(0u, 0u);
      if (v < nvec) {
        if constexpr (kFour) raw[u].x = __ldcs(reinterpret_cast<const uint32_t*>(a.codes) + v);
        else raw[u] = __ldcs(reinterpret_cast<const uint2*>(a.codes) + v);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = v0 + u * stride;
      if (v >= nvec) break;
      const int64_t g = a.vec_shift >= 0 ? (v >> a.vec_shift) : (v / a.vecs_per_group);
      OutT* dst = reinterpret_cast<OutT*>(a.out) + (v << 3);
      if constexpr (mode_is_integer(MODE)) {
        const __half s = reinterpret_cast<const __half*>(a.scale)[g];
        const __half2 s2 = __half2half2(s);
        // what is subtracted from 1024 + code: 1024 (+ 8 or + 128 for the symmetric modes' offset binary codes),
        // plus the zero point for the asymmetric modes - every term an integer, so one subtraction is exact
        uint32_t off_bits = MODE == NNCFB_INT4_SYM ? 0x64086408u : MODE == NNCFB_INT8_SYM ? 0x64806480u : 0x64006400u;
        if constexpr (mode_is_asym(MODE)) {
          uint32_t zb;
          if constexpr (MODE == NNCFB_INT8_ASYM) zb = a.zp[g];
          else zb = (a.zp[g >> 1] >> (4 * (g & 1))) & 15u;
          off_bits |= zb | (zb << 16);
        }
        const __half2 off = as_half2(off_bits);
        __half2 x[4];
        if constexpr (kFour) {
          // nibbles i and i + 4 of the word as one pair
#pragma unroll
          for (int i = 0; i < 4; ++i) x[i] = __hsub2(as_half2(((raw[u].x >> (4 * i)) & 0x000f000fu) | 0x64006400u), off);
        } else {
          const uint32_t flip = MODE == NNCFB_INT8_SYM ? 0x80808080u : 0u;    // two's complement byte + 128
          const uint32_t lo = raw[u].x ^ flip, hi = raw[u].y ^ flip;
          x[0] = __hsub2(as_half2(__byte_perm(lo, 0x64646464u, 0x4140)), off);
          x[1] = __hsub2(as_half2(__byte_perm(lo, 0x64646464u, 0x4342)), off);
          x[2] = __hsub2(as_half2(__byte_perm(hi, 0x64646464u, 0x4140)), off);
          x[3] = __hsub2(as_half2(__byte_perm(hi, 0x64646464u, 0x4342)), off);
        }
        __half2 r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = __hmul2(x[i], s2);
        store_pairs<OutT>(dst, r, kFour);
      } else {
        uint32_t code[8];
        if constexpr (kFour) {
#pragma unroll
          for (int i = 0; i < 8; ++i) code[i] = (raw[u].x >> (4 * i)) & 15u;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            code[i] = (raw[u].x >> (8 * i)) & 255u;
            code[4 + i] = (raw[u].y >> (8 * i)) & 255u;
          }
        }
        float s;
        if constexpr (mode_is_mx(MODE)) s = exp2_int(static_cast<int>(reinterpret_cast<const uint8_t*>(a.scale)[g]) - 127);
        else s = reinterpret_cast<const float*>(a.scale)[g];
        alignas(16) OutT o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float uval;
          if constexpr (MODE == NNCFB_NF4) {
            uval = kNf4Levels[code[i]];
          } else if constexpr (mode_bits(MODE) == 8) {
            uval = e4m3_value(code[i]);
          } else {
            const float mag = e2m1_magnitude(static_cast<int>(code[i] & 7u));
            uval = (code[i] & 8u) ? -mag : mag;
          }
          o[i] = cast_out<OutT>(__fmul_rn(uval, s));
        }
        if constexpr (sizeof(OutT) == 2) {
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
        } else {
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
          *reinterpret_cast<uint4*>(dst + 4) = *reinterpret_cast<const uint4*>(o + 4);
        }
      }
    }
  }
}

// One element per thread, group index per element: group sizes that are not a multiple of 8 (a per-channel
// INT8 layer whose inner dimension is, say, 100), where a group may end inside an 8-element vector.  Same
// arithmetic as the vector kernel.
template <typename OutT, int MODE>
__global__ void __launch_bounds__(256) decompress_scalar_kernel(const DecompressArgs a) {
  constexpr bool kFour = mode_bits(MODE) == 4;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < a.n;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t g = e / a.group_size;
    uint32_t code;
    if constexpr (kFour) code = (a.codes[e >> 1] >> (4 * (e & 1))) & 15u;
    else code = a.codes[e];
    float r;
    if constexpr (mode_is_integer(MODE)) {
      const __half s = reinterpret_cast<const __half*>(a.scale)[g];
      int q;
      if constexpr (MODE == NNCFB_INT4_SYM) q = static_cast<int>(code) - 8;
      else if constexpr (MODE == NNCFB_INT8_SYM) q = static_cast<int>(static_cast<int8_t>(code));
      else q = static_cast<int>(code);
      __half x = __int2half_rn(q);
      if constexpr (MODE == NNCFB_INT8_ASYM) x = __hsub(x, __int2half_rn(a.zp[g]));
      if constexpr (MODE == NNCFB_INT4_ASYM) x = __hsub(x, __int2half_rn((a.zp[g >> 1] >> (4 * (g & 1))) & 15));
      r = __half2float(__hmul(x, s));
    } else {
      float s;
      if constexpr (mode_is_mx(MODE)) s = exp2_int(static_cast<int>(reinterpret_cast<const uint8_t*>(a.scale)[g]) - 127);
      else s = reinterpret_cast<const float*>(a.scale)[g];
      float u;
      if constexpr (MODE == NNCFB_NF4) {
        u = kNf4Levels[code];
      } else if constexpr (mode_bits(MODE) == 8) {
        u = e4m3_value(code);
      } else {
        const float mag = e2m1_magnitude(static_cast<int>(code & 7u));
        u = (code & 8u) ? -mag : mag;
      }
      r = __fmul_rn(u, s);
    }
    reinterpret_cast<OutT*>(a.out)[e] = cast_out<OutT>(r);
  }
}

template <typename OutT>
int launch_decompress(const DecompressArgs& a, cudaStream_t st) {
  if (a.group_size % 8 != 0 || !aligned16(a.out) || (reinterpret_cast<uintptr_t>(a.codes) & 7u) != 0) {
    const int sgrid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((a.n + 255) / 256, static_cast<int64_t>(sm_count()) * 32)));
#define NNCFB_DQS(M) decompress_scalar_kernel<OutT, M><<<sgrid, 256, 0, st>>>(a); break
    switch (a.mode) {
      case NNCFB_INT8_SYM: NNCFB_DQS(NNCFB_INT8_SYM);
      case NNCFB_INT8_ASYM: NNCFB_DQS(NNCFB_INT8_ASYM);
      case NNCFB_INT4_SYM: NNCFB_DQS(NNCFB_INT4_SYM);
      case NNCFB_INT4_ASYM: NNCFB_DQS(NNCFB_INT4_ASYM);
      case NNCFB_NF4: NNCFB_DQS(NNCFB_NF4);
      case NNCFB_FP4: NNCFB_DQS(NNCFB_FP4);
      case NNCFB_MXFP4: NNCFB_DQS(NNCFB_MXFP4);
      case NNCFB_FP8_E4M3: NNCFB_DQS(NNCFB_FP8_E4M3);
      case NNCFB_MXFP8_E4M3: NNCFB_DQS(NNCFB_MXFP8_E4M3);
      default:
        set_error("nncfb_decompress: mode %d is not supported", a.mode);
        return NNCFB_E_UNSUPPORTED;
    }
#undef NNCFB_DQS
    NNCFB_CUDA(cudaGetLastError());
    return NNCFB_OK;
  }
  const int64_t nvec = a.n >> 3;
  const int64_t per_cta = 256 * kDecompressUnroll;
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((nvec + per_cta - 1) / per_cta, static_cast<int64_t>(sm_count()) * 16)));
#define NNCFB_DQ(M) decompress_kernel<OutT, M><<<grid, 256, 0, st>>>(a); break
  switch (a.mode) {
    case NNCFB_INT8_SYM: NNCFB_DQ(NNCFB_INT8_SYM);
    case NNCFB_INT8_ASYM: NNCFB_DQ(NNCFB_INT8_ASYM);
    case NNCFB_INT4_SYM: NNCFB_DQ(NNCFB_INT4_SYM);
    case NNCFB_INT4_ASYM: NNCFB_DQ(NNCFB_INT4_ASYM);
    case NNCFB_NF4: NNCFB_DQ(NNCFB_NF4);
    case NNCFB_FP4: NNCFB_DQ(NNCFB_FP4);
    case NNCFB_MXFP4: NNCFB_DQ(NNCFB_MXFP4);
    case NNCFB_FP8_E4M3: NNCFB_DQ(NNCFB_FP8_E4M3);
    case NNCFB_MXFP8_E4M3: NNCFB_DQ(NNCFB_MXFP8_E4M3);
    default:
      set_error("nncfb_decompress: mode %d is not supported", a.mode);
      return NNCFB_E_UNSUPPORTED;
  }
#undef NNCFB_DQ
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

}  // namespace nncfb

using namespace nncfb;

extern "C" int nncfb_decompress(const void* codes, int32_t mode, int64_t n_elements, int64_t group_size, const void* scale,
                                const void* zero_point, void* out, int32_t out_dtype, void* stream) {
  NNCFB_CHECK_ARG(codes && scale && out, NNCFB_E_BAD_ARG, "nncfb_decompress: null pointer");
  NNCFB_CHECK_ARG(n_elements > 0 && group_size > 0 && n_elements % group_size == 0, NNCFB_E_BAD_ARG,
                  "nncfb_decompress: %lld elements are not a whole number of groups of %lld", (long long)n_elements,
                  (long long)group_size);
  NNCFB_CHECK_ARG(!mode_is_asym(mode) || zero_point, NNCFB_E_BAD_ARG, "nncfb_decompress: zero_point is null");
  NNCFB_CHECK_ARG(mode_bits(mode) != 4 || n_elements % 2 == 0, NNCFB_E_BAD_ARG,
                  "nncfb_decompress: %lld 4-bit codes do not fill whole bytes", (long long)n_elements);
  DecompressArgs a;
  a.codes = static_cast<const uint8_t*>(codes);
  a.scale = scale;
  a.zp = static_cast<const uint8_t*>(zero_point);
  a.out = out;
  a.n = n_elements;
  a.group_size = group_size;
  a.vecs_per_group = std::max<int64_t>(1, group_size / 8);
  a.vec_shift = -1;
  if ((a.vecs_per_group & (a.vecs_per_group - 1)) == 0) {
    a.vec_shift = 0;
    while ((int64_t{1} << a.vec_shift) < a.vecs_per_group) ++a.vec_shift;
  }
  a.mode = mode;
  a.out_dtype = out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case NNCFB_F32: return launch_decompress<float>(a, st);
    case NNCFB_F16: return launch_decompress<__half>(a, st);
    case NNCFB_BF16: return launch_decompress<__nv_bfloat16>(a, st);
    default: break;
  }
  set_error("nncfb_decompress: unsupported output dtype %d", out_dtype);
  return NNCFB_E_BAD_ARG;
}
