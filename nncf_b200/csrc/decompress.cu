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

// 8 consecutive elements per thread (one 32-bit word of nibbles or two words of bytes); a group never
// ends inside a vector because group sizes handled here are multiples of 8.
template <typename OutT, int MODE>
__global__ void __launch_bounds__(256) decompress_kernel(const DecompressArgs a) {
  constexpr bool kFour = mode_bits(MODE) == 4;
  const int64_t nvec = a.n >> 3;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e0 = v << 3;
    const int64_t g = e0 / a.group_size;
    uint32_t code[8];
    if constexpr (kFour) {
      const uint32_t w = __ldcs(reinterpret_cast<const uint32_t*>(a.codes + (e0 >> 1)));
#pragma unroll
      for (int i = 0; i < 8; ++i) code[i] = (w >> (4 * i)) & 15u;
    } else {
      const uint2 w = __ldcs(reinterpret_cast<const uint2*>(a.codes + e0));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        code[i] = (w.x >> (8 * i)) & 255u;
        code[4 + i] = (w.y >> (8 * i)) & 255u;
      }
    }
    float r[8];
    if constexpr (mode_is_integer(MODE)) {
      const __half s = reinterpret_cast<const __half*>(a.scale)[g];
      __half z = __float2half_rn(0.0f);
      if constexpr (MODE == NNCFB_INT8_ASYM) z = __int2half_rn(a.zp[g]);
      if constexpr (MODE == NNCFB_INT4_ASYM) z = __int2half_rn((a.zp[g >> 1] >> (4 * (g & 1))) & 15);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int q;
        if constexpr (MODE == NNCFB_INT4_SYM) q = static_cast<int>(code[i]) - 8;             // stored with +8
        else if constexpr (MODE == NNCFB_INT8_SYM) q = static_cast<int>(static_cast<int8_t>(code[i]));
        else q = static_cast<int>(code[i]);
        __half x = __int2half_rn(q);
        if constexpr (mode_is_asym(MODE)) x = __hsub(x, z);
        r[i] = __half2float(__hmul(x, s));
      }
    } else {
      float s;
      if constexpr (mode_is_mx(MODE)) s = exp2_int(static_cast<int>(reinterpret_cast<const uint8_t*>(a.scale)[g]) - 127);
      else s = reinterpret_cast<const float*>(a.scale)[g];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float u;
        if constexpr (MODE == NNCFB_NF4) {
          u = kNf4Levels[code[i]];
        } else if constexpr (mode_bits(MODE) == 8) {
          u = e4m3_value(code[i]);
        } else {
          const float mag = e2m1_magnitude(static_cast<int>(code[i] & 7u));
          u = (code[i] & 8u) ? -mag : mag;
        }
        r[i] = __fmul_rn(u, s);
      }
    }
    alignas(16) OutT o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = cast_out<OutT>(r[i]);
    OutT* dst = reinterpret_cast<OutT*>(a.out) + e0;
    if constexpr (sizeof(OutT) == 2) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
    } else {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
      *(reinterpret_cast<uint4*>(dst) + 1) = *(reinterpret_cast<const uint4*>(o) + 1);
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
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((nvec + 255) / 256, static_cast<int64_t>(sm_count()) * 16)));
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
