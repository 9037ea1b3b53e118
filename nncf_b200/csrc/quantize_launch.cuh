// Host-side kernel selection for nncfb_quantize, instantiated once per source element type
// (one translation unit each, so the three compile in parallel).
#pragma once

#include <algorithm>

#include "quantize_fast.cuh"
#include "quantize_kernels.cuh"

namespace nncfb {

// Which kernel serves a validated request.
enum class QuantPath { kSubwarp, kWide, kGeneric, kColumn, kColumnTile };

inline QuantPath choose_path(int64_t group_size, int64_t inner, bool aligned) {
  if (inner > 1) return QuantPath::kColumn;
  if (aligned && group_size % 8 == 0) {
    if (group_size <= 256 && (group_size & (group_size - 1)) == 0) return QuantPath::kSubwarp;
    if (group_size >= 512) return QuantPath::kWide;
  }
  return QuantPath::kGeneric;
}

template <typename SrcT, int MODE>
int launch_quantize_mode(const QArgs& a, QuantPath path, cudaStream_t stream) {
  const int sms = sm_count();
  constexpr int kThreads = 256;
  switch (path) {
    case QuantPath::kSubwarp: {
      constexpr int U = 4;
      const int L = static_cast<int>(a.group_size / 8);
      const int64_t per_warp_iter = static_cast<int64_t>(32 / L) * U;
      const int64_t iters = (a.n_groups + per_warp_iter - 1) / per_warp_iter;
      const int64_t blocks_needed = (iters + (kThreads / 32) - 1) / (kThreads / 32);
      const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks_needed, static_cast<int64_t>(sms) * 8)));
      if (L == 16) {
        quant_subwarp_kernel<SrcT, MODE, 16, U><<<grid, kThreads, 0, stream>>>(a);
      } else if (L == 4) {
        quant_subwarp_kernel<SrcT, MODE, 4, U><<<grid, kThreads, 0, stream>>>(a);
      } else {
        quant_subwarp_kernel<SrcT, MODE, 0, U><<<grid, kThreads, 0, stream>>>(a);
      }
      break;
    }
    case QuantPath::kWide: {
      const int T = a.group_size <= 2048 ? 64 : (a.group_size <= 4096 ? 128 : 256);
      const int64_t blocks_needed = (a.n_groups + (kThreads / T) - 1) / (kThreads / T);
      const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks_needed, static_cast<int64_t>(sms) * 8)));
      quant_wide_kernel<SrcT, MODE><<<grid, kThreads, 0, stream>>>(a, T);
      break;
    }
    case QuantPath::kGeneric: {
      const int64_t blocks_needed = (a.n_groups + (kThreads / 32) - 1) / (kThreads / 32);
      const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks_needed, static_cast<int64_t>(sms) * 8)));
      quant_generic_kernel<SrcT, MODE><<<grid, kThreads, 0, stream>>>(a);
      break;
    }
    case QuantPath::kColumnTile: {
      const int64_t blocks_needed = (a.n_groups / a.inner) * ((a.inner + 63) / 64);
      const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks_needed, static_cast<int64_t>(sms) * 8)));
      quant_column_tile_kernel<SrcT, MODE><<<grid, kThreads, 0, stream>>>(a);
      break;
    }
    case QuantPath::kColumn: {
      const int cpt = a.codes_format == NNCFB_CODES_NIBBLE ? 2 : 1;
      const int64_t total = (a.n_groups / a.inner) * ((a.inner + cpt - 1) / cpt);
      const int64_t blocks_needed = (total + kThreads - 1) / kThreads;
      const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks_needed, static_cast<int64_t>(sms) * 8)));
      quant_column_kernel<SrcT, MODE><<<grid, kThreads, 0, stream>>>(a);
      break;
    }
  }
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

template <typename SrcT>
int launch_quantize_t(const QArgs& a, int mode, QuantPath path, cudaStream_t stream) {
  switch (mode) {
    case NNCFB_INT8_SYM: return launch_quantize_mode<SrcT, NNCFB_INT8_SYM>(a, path, stream);
    case NNCFB_INT8_ASYM: return launch_quantize_mode<SrcT, NNCFB_INT8_ASYM>(a, path, stream);
    case NNCFB_INT4_SYM: return launch_quantize_mode<SrcT, NNCFB_INT4_SYM>(a, path, stream);
    case NNCFB_INT4_ASYM: return launch_quantize_mode<SrcT, NNCFB_INT4_ASYM>(a, path, stream);
    case NNCFB_NF4: return launch_quantize_mode<SrcT, NNCFB_NF4>(a, path, stream);
    case NNCFB_MXFP4: return launch_quantize_mode<SrcT, NNCFB_MXFP4>(a, path, stream);
    case NNCFB_FP4: return launch_quantize_mode<SrcT, NNCFB_FP4>(a, path, stream);
    case NNCFB_FP8_E4M3: return launch_quantize_mode<SrcT, NNCFB_FP8_E4M3>(a, path, stream);
    case NNCFB_MXFP8_E4M3: return launch_quantize_mode<SrcT, NNCFB_MXFP8_E4M3>(a, path, stream);
    default: break;
  }
  set_error("unknown mode %d", mode);
  return NNCFB_E_BAD_ARG;
}

// ---- fast batched path -----------------------------------------------------------------------------
// Shape class of a batch: every tensor of a batch shares it.
struct FastClass {
  int kind;         // 0: not eligible, 1: row groups, 2: per channel
  int64_t group;    // group size (kind 1) or row length (kind 2)
  bool operator==(const FastClass& o) const { return kind == o.kind && group == o.group; }
};

inline FastClass fast_class(const nncfb_quantize_args& p) {
  FastClass none{0, 0};
  const bool fast_float = mode_is_fast_float(p.mode);
  if (!(mode_is_integer(p.mode) || fast_float) || p.inner != 1 || p.pre_scale || p.pre_zp || p.values_out ||
      p.dq_out || p.sqerr_out || !p.codes_out)
    return none;
  if (p.scale_e8m0_out && !mode_is_mx(p.mode)) return none;
  if (!p.scale_out && !(mode_is_mx(p.mode) && p.scale_e8m0_out)) return none;
  if (mode_is_asym(p.mode) && !p.zp_out && !p.zp_packed_out) return none;
  const bool four = mode_bits(p.mode) == 4;
  if (p.codes_format != (four ? NNCFB_CODES_NIBBLE : NNCFB_CODES_BYTE)) return none;
  if (!aligned16(p.weight) || !aligned16(p.codes_out)) return none;
  if (p.group_size == 128 || p.group_size == 64 || p.group_size == 32) return FastClass{1, p.group_size};
  if (fast_float) return none;  // per-channel float modes use the general kernels
  // the per-channel kernel writes packed zero points one byte per row only: two rows per byte (4-bit) is left
  // to the general kernels
  if (p.zp_packed_out && four) return none;
  if (p.group_size == p.reduce && p.reduce % 8 == 0 && p.reduce >= 512) return FastClass{2, p.reduce};
  return none;
}

// Groups in flight per sub-warp: an fp32 vector of 8 elements takes eight registers instead of four, and four
// groups of them spill under the 64-register budget of four resident blocks per SM.
constexpr int rows_in_flight(size_t elem_size) { return elem_size == 4 ? NNCFB_ROWS_U / 2 : NNCFB_ROWS_U; }

template <typename SrcT, int MODE>
int launch_fast_mode(const FastBatch& b, FastClass cls, cudaStream_t stream) {
  const int sms = sm_count();
  if constexpr (mode_is_fast_float(MODE)) {
    if (cls.kind != 1) {
      set_error("fast path: float modes support group sizes 32, 64 and 128 only");
      return NNCFB_E_UNSUPPORTED;
    }
  }
  if (cls.kind == 1) {
    constexpr int U = rows_in_flight(sizeof(SrcT));
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>((b.iter_start[b.n_tensors] + 7) / 8, static_cast<int64_t>(sms) * NNCFB_ROWS_MINBLOCKS)));
    if (cls.group == 128) {
      quant_rows_batch_kernel<SrcT, MODE, 8, 2, U><<<grid, 256, 0, stream>>>(b);
    } else if (cls.group == 64) {
      quant_rows_batch_kernel<SrcT, MODE, 4, 2, U><<<grid, 256, 0, stream>>>(b);
    } else {
      quant_rows_batch_kernel<SrcT, MODE, 2, 2, U><<<grid, 256, 0, stream>>>(b);
    }
  } else if constexpr (!mode_is_fast_float(MODE)) {
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>(b.iter_start[b.n_tensors], static_cast<int64_t>(sms) * 3)));
    const int64_t nvec = cls.group / 8;
    constexpr int K = WideCache<SrcT>::K;
    if (nvec <= 64 * K) {
      quant_channel_batch_kernel<SrcT, MODE, 64><<<grid, 256, 0, stream>>>(b, cls.group);
    } else if (nvec <= 128 * K) {
      quant_channel_batch_kernel<SrcT, MODE, 128><<<grid, 256, 0, stream>>>(b, cls.group);
    } else {
      quant_channel_batch_kernel<SrcT, MODE, 256><<<grid, 256, 0, stream>>>(b, cls.group);
    }
  }
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

template <typename SrcT>
int launch_fast_t(const FastBatch& b, int mode, FastClass cls, cudaStream_t stream) {
  switch (mode) {
    case NNCFB_INT8_SYM: return launch_fast_mode<SrcT, NNCFB_INT8_SYM>(b, cls, stream);
    case NNCFB_INT8_ASYM: return launch_fast_mode<SrcT, NNCFB_INT8_ASYM>(b, cls, stream);
    case NNCFB_INT4_SYM: return launch_fast_mode<SrcT, NNCFB_INT4_SYM>(b, cls, stream);
    case NNCFB_INT4_ASYM: return launch_fast_mode<SrcT, NNCFB_INT4_ASYM>(b, cls, stream);
    case NNCFB_NF4: return launch_fast_mode<SrcT, NNCFB_NF4>(b, cls, stream);
    case NNCFB_FP4: return launch_fast_mode<SrcT, NNCFB_FP4>(b, cls, stream);
    case NNCFB_MXFP4: return launch_fast_mode<SrcT, NNCFB_MXFP4>(b, cls, stream);
    case NNCFB_FP8_E4M3: return launch_fast_mode<SrcT, NNCFB_FP8_E4M3>(b, cls, stream);
    case NNCFB_MXFP8_E4M3: return launch_fast_mode<SrcT, NNCFB_MXFP8_E4M3>(b, cls, stream);
    default: break;
  }
  set_error("fast path: unsupported mode %d", mode);
  return NNCFB_E_UNSUPPORTED;
}

// iterations one tensor contributes to a batch of class `cls`
inline int64_t fast_iterations(const FastClass& cls, int64_t n_groups, size_t elem_size) {
  if (cls.kind == 1) {
    const int L = cls.group == 128 ? 8 : (cls.group == 64 ? 4 : 2);
    const int64_t per_iter = (32 / L) * rows_in_flight(elem_size);  // GPW * U
    return (n_groups + per_iter - 1) / per_iter;
  }
  const int K = elem_size == 4 ? 4 : 8;
  const int64_t nvec = cls.group / 8;
  const int tpr = nvec <= 64 * K ? 64 : (nvec <= 128 * K ? 128 : 256);
  const int rpb = 256 / tpr;
  return (n_groups + rpb - 1) / rpb;
}

// defined in quantize_f32.cu / quantize_f16.cu / quantize_bf16.cu
int launch_fast_f32(const FastBatch& b, int mode, FastClass cls, cudaStream_t stream);
int launch_fast_f16(const FastBatch& b, int mode, FastClass cls, cudaStream_t stream);
int launch_fast_bf16(const FastBatch& b, int mode, FastClass cls, cudaStream_t stream);
int launch_quantize_f32(const QArgs& a, int mode, QuantPath path, cudaStream_t stream);
int launch_quantize_f16(const QArgs& a, int mode, QuantPath path, cudaStream_t stream);
int launch_quantize_bf16(const QArgs& a, int mode, QuantPath path, cudaStream_t stream);

}  // namespace nncfb
