// GPTQ: blocked column sweep with error feedback, the lazy-batch trailing update and the fp32
// (CUDA-core) Hessian accumulation.
//
// Restates GPTQ._quantize_weights of the reference
// (src/nncf/quantization/algorithms/weight_compression/gptq.py:297-379) after its Hessian
// preparation (dead columns, damping, Cholesky inverse: host-side library calls).  The reference
// walks the columns in Python with ~8 small tensor operations per column; here one C call runs
//   gptq_sweep_fast_kernel  once per full 128-column block: eight lanes share an output row, the block's
//                         weights live in their registers, the matching Hinv block in shared memory;
//                         group parameters are taken at each group start from the tensor-level weight
//                         (updated at block ends only), exactly as the reference indexes it;
//   gptq_sweep_kernel     the same sweep with a thread per row, for ragged or unaligned blocks;
//   gptq_trailing_kernel  W[:, i2:] -= Err_blk @ Hinv[i1:i2, i2:] as a tiled fp32 contraction.
// Rounding follows the reference: quotients are true fp32 divisions, the in-block update is a
// product rounded to fp32 followed by a subtraction (what `w -= outer(err, h)` does).  The trailing
// contraction accumulates in fp32 in ascending k; BLAS libraries use another order, and GPTQ
// amplifies such last-bit differences into occasional flipped codes.
#include <algorithm>
#include <map>
#include <memory>
#include <mutex>
#include <utility>

#include "quantize_kernels.cuh"

namespace nncfb {

constexpr int kGptqMaxBlock = 128;
constexpr int kSweepRows = 32;
constexpr int kSweepLd = kSweepRows + 1;

struct GptqArgs {
  float* w;            // [rows, cols] tensor-level weight, updated in place
  const float* hinv;   // [cols, cols] upper Cholesky factor of H^-1
  float* q;            // [rows, cols] dequantised result
  float* err;          // [rows, kGptqMaxBlock] scratch: error columns of the current block
  const float* err_prev;  // optional: the previous block's error columns, still to be applied to this block's
                          // columns (W[:, block] -= Err_prev @ Hinv[previous block's rows, block]) by the sweep itself
  __nv_bfloat16* err_planes;  // optional [3 * 128, err_ld]: the same errors as three bf16 planes, transposed
  int64_t err_ld;
  float* scale;        // [rows, G]
  int32_t* zp;         // [rows, G] or null
  int64_t rows, cols;
  int64_t gs, G;
  int i1, count;       // current block: columns [i1, i1 + count)
  int given;           // 1: scale / zp of the groups starting in this block are already in the tables
};

// A warp owns 32 output rows (a thread owns a row); kSweepWarps warps share one copy of the block of Hinv.
// The 128-column block is swept in four sub-blocks of 32 columns: the sub-block lives in registers and its
// triangular update is fully unrolled; the error columns of a finished sub-block are then applied to the rest
// of the block, column by column in ascending error order, so every weight sees exactly the sequence of
// rounded multiply / subtract steps that the reference's column loop applies to it (WC/gptq.py:337-358).
// The kernel is a chain of dependent steps, so what matters is the latency of its prologue: Hinv and the
// weight tile are fetched with wide independent loads by all warps, and the parameters of every group that
// starts inside the block are computed from the tile before the sweep (the tensor-level weight the reference
// reads at a group start is this tile as loaded: it is only updated at block ends).
constexpr int kSweepWarps = 4;
constexpr int kSweepMaxGroups = 16;  // groups starting inside one block whose parameters are kept in shared memory

struct SweepSmem {
  static constexpr size_t hs_floats = static_cast<size_t>(kGptqMaxBlock) * kGptqMaxBlock;
  static constexpr size_t per_warp_floats = 2 * static_cast<size_t>(kGptqMaxBlock) * kSweepLd + 2 * kSweepMaxGroups * kSweepRows;
  static constexpr size_t bytes = (hs_floats + kSweepWarps * per_warp_floats) * sizeof(float);
};

template <int MODE>
__global__ void __launch_bounds__(kSweepWarps * kSweepRows) gptq_sweep_kernel(const GptqArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, t = threadIdx.x & 31;
  float* hs = smem;                                                    // [128][128] Hinv block (row i, col j >= i used)
  float* ws = hs + SweepSmem::hs_floats + warp * SweepSmem::per_warp_floats;  // [128][33] weights, column-major per thread
  float* es = ws + kGptqMaxBlock * kSweepLd;                           // [128][33] error columns
  float* ps = es + kGptqMaxBlock * kSweepLd;                           // [16][32] scale of the groups starting here
  float* pz = ps + kSweepMaxGroups * kSweepRows;                       // [16][32] zero point
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * kSweepWarps + warp) * kSweepRows;
  const int64_t row = row0 + t;
  const bool valid = row < a.rows;
  const int count = a.count, i1 = a.i1;
  // 16-byte loads need whole, aligned quads of columns
  const bool vec = count == kGptqMaxBlock && (a.cols & 3) == 0 && (i1 & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(a.hinv) | reinterpret_cast<uintptr_t>(a.w) |
                     reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.err)) & 15u) == 0;

  if (vec) {
    // quads that touch the upper triangle (j + 3 >= i); the rest of hs is never read
#pragma unroll 8
    for (int idx = threadIdx.x; idx < kGptqMaxBlock * (kGptqMaxBlock / 4); idx += kSweepWarps * kSweepRows) {
      const int i = idx >> 5, j = (idx & 31) << 2;
      if (j + 3 >= i) {
        *reinterpret_cast<float4*>(hs + i * kGptqMaxBlock + j) =
            *reinterpret_cast<const float4*>(a.hinv + static_cast<int64_t>(i1 + i) * a.cols + (i1 + j));
      }
    }
#pragma unroll 8
    for (int r = 0; r < kSweepRows; ++r) {
      const int64_t rr = row0 + r;
      if (rr < a.rows) {
        const float4 v = *reinterpret_cast<const float4*>(a.w + rr * a.cols + i1 + 4 * t);
        ws[(4 * t + 0) * kSweepLd + r] = v.x;
        ws[(4 * t + 1) * kSweepLd + r] = v.y;
        ws[(4 * t + 2) * kSweepLd + r] = v.z;
        ws[(4 * t + 3) * kSweepLd + r] = v.w;
      }
    }
  } else {
    for (int idx = threadIdx.x; idx < kGptqMaxBlock * kGptqMaxBlock; idx += kSweepWarps * kSweepRows) {
      const int i = idx / kGptqMaxBlock, j = idx - i * kGptqMaxBlock;
      hs[idx] = (i < count && j < count) ? a.hinv[static_cast<int64_t>(i1 + i) * a.cols + (i1 + j)] : 0.0f;
    }
    for (int r = 0; r < kSweepRows; ++r) {
      const int64_t rr = row0 + r;
      if (rr >= a.rows) break;
      for (int j = t; j < count; j += kSweepRows) ws[j * kSweepLd + r] = a.w[rr * a.cols + i1 + j];
    }
  }
  __syncthreads();

  Codec<MODE> c;
  c.from_given(1.0f, 0.0f);
  if (valid && i1 % a.gs != 0) {
    // the block starts inside a group that an earlier block opened: take its stored parameters
    const int64_t g = i1 / a.gs;
    c.from_given(a.scale[row * a.G + g], a.zp ? static_cast<float>(a.zp[row * a.G + g]) : 0.0f);
  }
  // parameters of the groups that start inside this block, from the tensor-level weight (WC/gptq.py:312-335):
  // the columns inside the block are the tile as loaded, later ones are read from global memory
  const int64_t first_start = ((static_cast<int64_t>(i1) + a.gs - 1) / a.gs) * a.gs;
  if (valid) {
    int gl = 0;
    for (int64_t col = first_start; col < i1 + count; col += a.gs, ++gl) {
      const int64_t end = min(col + a.gs, a.cols);
      const int64_t in_block_end = min(end, static_cast<int64_t>(i1 + count));
      float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
      for (int64_t kk = col; kk < in_block_end && !a.given; ++kk) {
        const float v = ws[(kk - i1) * kSweepLd + t];
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
      const float* wr = a.w + row * a.cols;
      for (int64_t kk = in_block_end; kk < end && !a.given; ++kk) {
        const float v = wr[kk];
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
      Codec<MODE> cg;
      const int64_t g = col / a.gs;
      if (a.given) {
        // refined by ScaleEstimation for this block (WC/gptq.py:319-327)
        cg.from_given(a.scale[row * a.G + g], a.zp ? static_cast<float>(a.zp[row * a.G + g]) : 0.0f);
      } else {
        cg.from_stats(mn, mx);
        a.scale[row * a.G + g] = cg.scale;
        if (a.zp) a.zp[row * a.G + g] = static_cast<int32_t>(cg.zp);
      }
      if (gl < kSweepMaxGroups) {
        ps[gl * kSweepRows + t] = cg.scale;
        pz[gl * kSweepRows + t] = cg.zp;
      }
    }
  }
  // block-relative column of the next group start, advanced in 32-bit arithmetic (no 64-bit modulo per column)
  int next_start = static_cast<int>(min(first_start - i1, static_cast<int64_t>(kGptqMaxBlock)));
  const int gs_step = static_cast<int>(min(a.gs, static_cast<int64_t>(kGptqMaxBlock)));
  int gl_next = 0;
  // Sub-blocks of 8 and 16 columns (less unrolled code, more passes over the rest of the block) were measured at
  // the same speed as 32: the kernel is a chain of dependent steps either way.
  constexpr int SB = 32;
  for (int sb0 = 0; sb0 < count; sb0 += SB) {
    const int cb = min(SB, count - sb0);
    float w[SB], e[SB];
#pragma unroll
    for (int k = 0; k < SB; ++k) {
      w[k] = (k < cb) ? ws[(sb0 + k) * kSweepLd + t] : 0.0f;
      e[k] = 0.0f;
    }
#pragma unroll
    for (int k = 0; k < SB; ++k) {
      if (k < cb) {
        const int i = sb0 + k;
        if (i == next_start) {  // a group starts at this column
          if (valid) {
            if (gl_next < kSweepMaxGroups) {
              c.from_given(ps[gl_next * kSweepRows + t], pz[gl_next * kSweepRows + t]);
            } else {
              const int64_t g = (static_cast<int64_t>(i1) + i) / a.gs;  // written above by this thread
              c.from_given(a.scale[row * a.G + g], a.zp ? static_cast<float>(a.zp[row * a.G + g]) : 0.0f);
            }
          }
          next_start += gs_step;
          ++gl_next;
        }
        const float* hrow = hs + i * kGptqMaxBlock + sb0;
        const float d = hrow[k];
        float u = 0.0f;
        if (valid) c.encode(w[k], u);
        const float dq = __fmul_rn(u, c.scale);
        e[k] = __fdiv_rn(__fsub_rn(w[k], dq), d);
        ws[i * kSweepLd + t] = dq;  // the slot of a finished column carries its result
        es[i * kSweepLd + t] = e[k];
#pragma unroll
        for (int k2 = k + 1; k2 < SB; ++k2) w[k2] = __fsub_rn(w[k2], __fmul_rn(e[k], hrow[k2]));
      }
    }
    // the finished sub-block's errors applied to the remaining columns of the block, four columns at a time
    for (int j = sb0 + SB; j < count; j += 4) {
      float wj[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) wj[q4] = ws[(j + q4) * kSweepLd + t];   // rows beyond `count` are unused padding
#pragma unroll
      for (int k = 0; k < SB; ++k) {
        const float4 h = *reinterpret_cast<const float4*>(hs + (sb0 + k) * kGptqMaxBlock + j);
        wj[0] = __fsub_rn(wj[0], __fmul_rn(e[k], h.x));
        wj[1] = __fsub_rn(wj[1], __fmul_rn(e[k], h.y));
        wj[2] = __fsub_rn(wj[2], __fmul_rn(e[k], h.z));
        wj[3] = __fsub_rn(wj[3], __fmul_rn(e[k], h.w));
      }
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        if (j + q4 < count) ws[(j + q4) * kSweepLd + t] = wj[q4];
      }
    }
  }
  __syncwarp();
  if (a.err_planes != nullptr && valid) {
    // operand of the tensor-core trailing update: plane p, row k, column = this thread's output row
#pragma unroll 4
    for (int j = 0; j < count; ++j) {
      __nv_bfloat16 h, m, l;
      split_bf16x3(es[j * kSweepLd + t], h, m, l);
      a.err_planes[(0 * kGptqMaxBlock + j) * a.err_ld + row] = h;
      a.err_planes[(1 * kGptqMaxBlock + j) * a.err_ld + row] = m;
      a.err_planes[(2 * kGptqMaxBlock + j) * a.err_ld + row] = l;
    }
  }
  if (vec) {
#pragma unroll 4
    for (int r = 0; r < kSweepRows; ++r) {
      const int64_t rr = row0 + r;
      if (rr < a.rows) {
        float4 qv, ev;
        qv.x = ws[(4 * t + 0) * kSweepLd + r]; ev.x = es[(4 * t + 0) * kSweepLd + r];
        qv.y = ws[(4 * t + 1) * kSweepLd + r]; ev.y = es[(4 * t + 1) * kSweepLd + r];
        qv.z = ws[(4 * t + 2) * kSweepLd + r]; ev.z = es[(4 * t + 2) * kSweepLd + r];
        qv.w = ws[(4 * t + 3) * kSweepLd + r]; ev.w = es[(4 * t + 3) * kSweepLd + r];
        *reinterpret_cast<float4*>(a.q + rr * a.cols + i1 + 4 * t) = qv;
        *reinterpret_cast<float4*>(a.err + rr * kGptqMaxBlock + 4 * t) = ev;
      }
    }
  } else {
    for (int r = 0; r < kSweepRows; ++r) {
      const int64_t rr = row0 + r;
      if (rr >= a.rows) break;
      for (int j = t; j < count; j += kSweepRows) {
        a.q[rr * a.cols + i1 + j] = ws[j * kSweepLd + r];
        a.err[rr * kGptqMaxBlock + j] = es[j * kSweepLd + r];
      }
    }
  }
}

// ---- the sweep for full, aligned blocks -------------------------------------------------------------
// Same arithmetic as gptq_sweep_kernel, laid out for latency: the sweep of one block is 128 dependent steps per
// output row, so the time of a launch is the time of one thread's instruction stream.  Here kFsLanes lanes share
// a row.  The block's 32 quads of columns are dealt round-robin to the lanes (lane l owns quads l, l + 8, ...),
// every lane keeps its quads in registers, and a step goes: the owner of the current quad quantises its four
// columns (applying each error to the later columns of the same quad at once), the four errors are broadcast
// to the row's lanes with one shuffle each, and every lane applies them to the quads it still has to process.
// Each weight therefore receives the same rounded multiply / subtract steps in the same (ascending) error
// order as in the reference's column loop (WC/gptq.py:337-358), spread over eight instruction streams.
// The division by Hinv[i, i] uses the reciprocal of the diagonal computed once per block (the same correction
// sequence as the division by the scale); numerators outside a safe exponent range take the IEEE division.
// Warps loop over groups of kFsRows rows, so one copy of the Hinv block in shared memory serves a whole CTA and
// the grid never exceeds one CTA per SM.
constexpr int kFsLanes = 8;
constexpr int kFsRows = 32 / kFsLanes;             // rows per warp
constexpr int kFsQuads = kGptqMaxBlock / 4 / kFsLanes;  // quads per lane
constexpr int kFsMaxWarps = 16;  // 512 threads: the compiler may use 128 registers (fewer made the update loops spill)

// start of quad q of rows in the packed triangle, and the length of its rows
__host__ __device__ constexpr int tri_base(int q) { return 512 * q - 8 * q * (q - 1); }
__host__ __device__ constexpr int tri_len(int q) { return kGptqMaxBlock - 4 * q; }
static_assert(tri_base(32) == 8448, "packed triangle size");

struct FastSweepSmem {
  static constexpr size_t hs_floats = static_cast<size_t>(kGptqMaxBlock) * kGptqMaxBlock;
  static constexpr size_t diag_floats = 2 * kGptqMaxBlock;
  static constexpr size_t per_warp_floats = 3 * kSweepMaxGroups * kFsRows;  // scale, zero point, reciprocal
  // The upper triangle only, rows padded to whole quads of columns: row i keeps columns 4 * (i / 4) .. 127.
  static constexpr size_t tri_floats = 8448;  // sum over the 32 quads of rows of 4 * (128 - 4 q)
  static constexpr size_t bytes(int warps, bool with_previous) {
    return (tri_floats + (with_previous ? hs_floats : 0) + diag_floats + warps * per_warp_floats) * sizeof(float);
  }
};

// Stores that are predicated instead of branched around: a branch costs the lone warp of a scheduler a fetch
// bubble, dozens of times per row.
__device__ __forceinline__ void store_v4_if(float* p, float x, float y, float z, float w, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t@p st.global.v4.f32 [%0], {%1, %2, %3, %4};\n\t}"
               :: "l"(p), "f"(x), "f"(y), "f"(z), "f"(w), "r"(static_cast<int>(pred)) : "memory");
}
__device__ __forceinline__ void store_bf16_if(__nv_bfloat16* p, __nv_bfloat16 v, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p st.global.b16 [%0], %1;\n\t}"
               :: "l"(p), "h"(__bfloat16_as_ushort(v)), "r"(static_cast<int>(pred)) : "memory");
}

// One group of kFsRows rows through the block.  SLOW = false assumes that every division may use the reciprocal
// sequence and returns true when that assumption failed for this lane (a scale or a numerator outside the safe
// exponent range); the caller then repeats the rows with SLOW = true (IEEE divisions), which overwrites every
// output.  QUAD_GROUPS: group starts fall on multiples of four columns, so they are looked for once per quad.
template <int MODE, bool QUAD_GROUPS, bool SLOW>
__device__ __forceinline__ bool sweep_row_group(const GptqArgs& a, const float* hs, const float* hp, const float2* diag,
                                                float* ps, float* pz, float* pr, const int64_t row, const bool valid, const int lane,
                                                const int64_t first_start, const int gs_step) {
  constexpr int L = kFsLanes, M = kFsQuads, B = kGptqMaxBlock;
  const int l = lane & (L - 1), rloc = lane / L;
  const int i1 = a.i1;
  bool bad = false;
  float w[M][4];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (valid) v = *reinterpret_cast<const float4*>(a.w + row * a.cols + i1 + 4 * (l + L * m));
    w[m][0] = v.x; w[m][1] = v.y; w[m][2] = v.z; w[m][3] = v.w;
  }
  if (a.err_prev != nullptr) {
    // The previous block's trailing update for this block's columns, which that block's launch left out so that
    // no kernel stands between two sweeps: fp32 accumulation in ascending k, one subtraction (the arithmetic of
    // gptq_trailing_kernel).  hp is Hinv[previous block's rows, this block's columns].
    float acc[M][4], ep[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;
      // this lane's share of the row's previous errors (the same quads as its weights); the others come by shuffle
      const float4 v = *reinterpret_cast<const float4*>(a.err_prev + (valid ? row : 0) * B + 4 * (l + L * m));
      ep[m][0] = v.x; ep[m][1] = v.y; ep[m][2] = v.z; ep[m][3] = v.w;
    }
    const int src0 = lane & ~(L - 1);
#pragma unroll
    for (int mk = 0; mk < M; ++mk) {
#pragma unroll 2
      for (int lk = 0; lk < L; ++lk) {
        const float* hq = hp + 4 * (lk + L * mk) * B + 4 * l;  // rows k = 4 (lk + L mk) .. + 3, ascending over the loops
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float e = __shfl_sync(0xffffffffu, ep[mk][kk], src0 | lk);
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const float4 h = *reinterpret_cast<const float4*>(hq + kk * B + 4 * L * m);
            acc[m][0] = __fmaf_rn(e, h.x, acc[m][0]);
            acc[m][1] = __fmaf_rn(e, h.y, acc[m][1]);
            acc[m][2] = __fmaf_rn(e, h.z, acc[m][2]);
            acc[m][3] = __fmaf_rn(e, h.w, acc[m][3]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int j = 0; j < 4; ++j) w[m][j] = __fsub_rn(w[m][j], acc[m][j]);
    }
  }
  Codec<MODE> c;
  c.from_given(1.0f, 0.0f);
  if (valid && i1 % a.gs != 0) {
    const int64_t g = i1 / a.gs;  // the block starts inside a group that an earlier block opened
    c.from_given(a.scale[row * a.G + g], a.zp ? static_cast<float>(a.zp[row * a.G + g]) : 0.0f);
  }
  bad = bad || !c.div.fast;
  c.div.fast = !SLOW;
  // parameters of the groups that start inside this block, from the tile as loaded (WC/gptq.py:312-335);
  // the columns of a group that lie beyond the block are read from global memory
  {
    int gl = 0;
    for (int64_t col = first_start; col < i1 + B; col += a.gs, ++gl) {
      const int64_t end = min(col + a.gs, a.cols);
      const int lo_c = static_cast<int>(col - i1);
      const int hi_c = static_cast<int>(min(end, static_cast<int64_t>(i1 + B)) - i1);
      const int64_t g = col / a.gs;
      Codec<MODE> cg;
      if (a.given) {
        // refined by ScaleEstimation for this block (WC/gptq.py:319-327)
        if (valid) cg.from_given(a.scale[row * a.G + g], a.zp ? static_cast<float>(a.zp[row * a.G + g]) : 0.0f);
        else cg.from_given(1.0f, 0.0f);
      } else {
        float mn = __uint_as_float(0x7f800000u), mx = __uint_as_float(0xff800000u);
#pragma unroll
        for (int m = 0; m < M; ++m) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int cidx = 4 * (l + L * m) + k;
            if (cidx >= lo_c && cidx < hi_c) {
              mn = fminf(mn, w[m][k]);
              mx = fmaxf(mx, w[m][k]);
            }
          }
        }
        if (valid) {
          const float* wr = a.w + row * a.cols;
          for (int64_t kk = static_cast<int64_t>(i1) + B + l; kk < end; kk += L) {
            const float v = wr[kk];
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
          }
        }
#pragma unroll
        for (int o = 1; o < L; o <<= 1) {
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        cg.from_stats(mn, mx);
        if (valid && l == 0) {
          a.scale[row * a.G + g] = cg.scale;
          if (a.zp) a.zp[row * a.G + g] = static_cast<int32_t>(cg.zp);
        }
      }
      if (l == 0) {  // at most kSweepMaxGroups groups start inside a block (the launcher checks the group size)
        ps[gl * kFsRows + rloc] = cg.scale;
        pz[gl * kFsRows + rloc] = cg.zp;
        pr[gl * kFsRows + rloc] = cg.div.fast ? cg.div.r : 0.0f;  // 0: this scale needs the IEEE division
      }
    }
  }
  __syncwarp();

  int next_start = static_cast<int>(min(first_start - i1, static_cast<int64_t>(B)));
  int gl_next = 0;
  const int src_base = lane & ~(L - 1);
  const bool planes = a.err_planes != nullptr && valid;
  // running pointers: all of them advance by one quad of columns per step
  float* q_out = a.q + (valid ? row : 0) * a.cols + i1;
  float* e_out = a.err + (valid ? row : 0) * B;
  __nv_bfloat16* pl_out = a.err_planes + (l & 3) * a.err_ld + (valid ? row : 0);
  const int64_t pl_plane = static_cast<int64_t>(B) * a.err_ld;
  int qd = 0;  // the quad of columns being swept; hs is the packed upper triangle (tri_base, tri_len)
#pragma unroll
  for (int mp = 0; mp < M; ++mp) {
#pragma unroll 1
    for (int lo = 0; lo < L; ++lo) {
      const bool own = l == lo;
      const int len = tri_len(qd);
      const float* h_quad = hs + tri_base(qd);           // rows 4 qd .. 4 qd + 3, from column 4 qd
      const float* h_lane = h_quad + 4 * (l - qd);       // the same rows at this lane's columns 4 (l + L m2)
      float e4[4], dq4[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = 4 * qd + k;
        if (!QUAD_GROUPS || k == 0) {
          // a group starts at this column (the same for the whole warp): its parameters replace the current ones
          const bool start = i == next_start;
          const int gi = min(gl_next, kSweepMaxGroups - 1);
          const float ns = ps[gi * kFsRows + rloc], nz = pz[gi * kFsRows + rloc], nr = pr[gi * kFsRows + rloc];
          bad = bad || (start && nr == 0.0f);
          c.scale = start ? ns : c.scale;
          c.zp = start ? nz : c.zp;
          c.div.s = start ? ns : c.div.s;
          c.div.r = start ? nr : c.div.r;
          if constexpr (Codec<MODE>::kMx) {
            Codec<MODE> n;
            n.from_given(ns, nz);
            c.e8m0 = start ? n.e8m0 : c.e8m0;
          }
          next_start += start ? gs_step : 0;
          gl_next += start ? 1 : 0;
        }
        const float wv = w[mp][k];
        float u = 0.0f;
        c.encode(wv, u);
        const float dq = __fmul_rn(u, c.scale);
        const float num = __fsub_rn(wv, dq);
        const float2 d = diag[i];
        float e;
        if (SLOW) {
          e = __fdiv_rn(num, d.x);
        } else {
          // |num| in [2^-60, 2^61): together with the diagonal's range nothing in the sequence under- or overflows
          // (+0 is fine as well: every step of the sequence then yields the quotient's +0 or -0)
          const uint32_t nb = __float_as_uint(num);
          bad = bad || ((nb & 0x7fffffffu) - 0x21800000u >= 0x5e000000u - 0x21800000u && nb != 0u);
          const float q0 = __fmul_rn(num, d.y);
          const float r = __fmaf_rn(-d.x, q0, num);
          e = __fmaf_rn(r, d.y, q0);
        }
        dq4[k] = dq;
        e4[k] = e;
        const float* hrow = h_quad + k * len;
#pragma unroll
        for (int k2 = k + 1; k2 < 4; ++k2) {
          const float nv = __fsub_rn(w[mp][k2], __fmul_rn(e, hrow[k2]));
          w[mp][k2] = own ? nv : w[mp][k2];
        }
      }
      store_v4_if(q_out, dq4[0], dq4[1], dq4[2], dq4[3], own && valid);
      store_v4_if(e_out, e4[0], e4[1], e4[2], e4[3], own && valid);
      const int src = src_base | lo;
#pragma unroll
      for (int k = 0; k < 4; ++k) e4[k] = __shfl_sync(0xffffffffu, e4[k], src);
      {
        // operand of the tensor-core trailing update: plane p, row = error column, column = output row.  Lanes
        // 0..3 of a row write the two upper planes of one error column each, lanes 4..7 the lowest plane.
        const float ek = (l & 1) ? ((l & 2) ? e4[3] : e4[1]) : ((l & 2) ? e4[2] : e4[0]);
        __nv_bfloat16 h, md, lw;
        split_bf16x3(ek, h, md, lw);
        const bool upper = l < 4;
        store_bf16_if(upper ? pl_out : pl_out + 2 * pl_plane, upper ? h : lw, planes);
        store_bf16_if(pl_out + pl_plane, md, planes && upper);
      }
      // the four errors applied to every quad that is still to come, in ascending error order
      const bool later = l > lo;
#pragma unroll
      for (int m2 = mp; m2 < M; ++m2) {
        const bool apply = m2 > mp || later;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 h = *reinterpret_cast<const float4*>(h_lane + k * len + 4 * L * m2);
          const float n0 = __fsub_rn(w[m2][0], __fmul_rn(e4[k], h.x));
          const float n1 = __fsub_rn(w[m2][1], __fmul_rn(e4[k], h.y));
          const float n2 = __fsub_rn(w[m2][2], __fmul_rn(e4[k], h.z));
          const float n3 = __fsub_rn(w[m2][3], __fmul_rn(e4[k], h.w));
          w[m2][0] = apply ? n0 : w[m2][0];
          w[m2][1] = apply ? n1 : w[m2][1];
          w[m2][2] = apply ? n2 : w[m2][2];
          w[m2][3] = apply ? n3 : w[m2][3];
        }
      }
      q_out += 4;
      e_out += 4;
      pl_out += 4 * a.err_ld;
      ++qd;
    }
  }
  __syncwarp();  // ps / pz are rewritten by the next group of rows
  return bad;
}

template <int MODE, bool QUAD_GROUPS>
__global__ void __launch_bounds__(kFsMaxWarps * 32) gptq_sweep_fast_kernel(const GptqArgs a) {
  constexpr int B = kGptqMaxBlock;
  extern __shared__ __align__(16) float smem[];
  float* hs = smem;                                                          // Hinv block, packed upper triangle
  float2* diag = reinterpret_cast<float2*>(hs + FastSweepSmem::tri_floats);  // Hinv[i, i] and its reciprocal
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* ps = reinterpret_cast<float*>(diag + B) + warp * FastSweepSmem::per_warp_floats;  // [16][rows of the warp]
  float* pz = ps + kSweepMaxGroups * kFsRows;
  float* pr = pz + kSweepMaxGroups * kFsRows;
  float* hp = reinterpret_cast<float*>(diag + B) + nwarps * FastSweepSmem::per_warp_floats;  // [128][128], with err_prev
  const int i1 = a.i1;

  // the blocks of Hinv: asynchronous 16-byte copies, all in flight at once
  if (a.err_prev != nullptr) {
    // Hinv[previous block's rows, this block's columns] for the update taken over from the previous block
    for (int idx = threadIdx.x; idx < B * (B / 4); idx += blockDim.x) {
      const int i = idx >> 5, j = (idx & 31) << 2;
      const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(hp + i * B + j));
      const float* src = a.hinv + static_cast<int64_t>(i1 - B + i) * a.cols + (i1 + j);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory");
    }
  }
  for (int idx = threadIdx.x; idx < B * (B / 4); idx += blockDim.x) {
    const int i = idx >> 5, j = (idx & 31) << 2;
    const int q = i >> 2;
    if (j >= 4 * q) {
      const uint32_t dst = static_cast<uint32_t>(
          __cvta_generic_to_shared(hs + tri_base(q) + (i & 3) * tri_len(q) + (j - 4 * q)));
      const float* src = a.hinv + static_cast<int64_t>(i1 + i) * a.cols + (i1 + j);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory");
    }
  }
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  int diag_fast = 1;
  if (threadIdx.x < B) {
    const int q = threadIdx.x >> 2;
    const Divisor dv = make_divisor(hs[tri_base(q) + (threadIdx.x & 3) * tri_len(q) + (threadIdx.x - 4 * q)]);
    diag[threadIdx.x] = make_float2(dv.s, dv.r);
    diag_fast = dv.fast ? 1 : 0;
  }
  const bool all_fast = __syncthreads_and(diag_fast) != 0;

  const int64_t first_start = ((static_cast<int64_t>(i1) + a.gs - 1) / a.gs) * a.gs;
  const int gs_step = static_cast<int>(min(a.gs, static_cast<int64_t>(B)));
  const int64_t n_row_groups = (a.rows + kFsRows - 1) / kFsRows;
  for (int64_t rg = static_cast<int64_t>(blockIdx.x) * nwarps + warp; rg < n_row_groups;
       rg += static_cast<int64_t>(gridDim.x) * nwarps) {
    const int64_t row = rg * kFsRows + lane / kFsLanes;
    const bool valid = row < a.rows;
    bool redo = !all_fast;
    if (all_fast) {
      const bool bad = sweep_row_group<MODE, QUAD_GROUPS, false>(a, hs, hp, diag, ps, pz, pr, row, valid, lane, first_start, gs_step);
      redo = __any_sync(0xffffffffu, bad && valid);
    }
    if (redo) sweep_row_group<MODE, QUAD_GROUPS, true>(a, hs, hp, diag, ps, pz, pr, row, valid, lane, first_start, gs_step);
  }
}

// W[:, c0 + ...] -= Err[rows, count] @ Hinv[i1 : i1+count, c0 : cols]; 64 x 64 tile per block, 4 x 4 per thread.
__global__ void __launch_bounds__(256) gptq_trailing_kernel(const GptqArgs a, const int64_t c0) {
  constexpr int KC = 64;  // k chunk held in shared memory
  __shared__ __align__(16) float e_s[KC][64 + 4];  // [k][row]
  __shared__ __align__(16) float h_s[KC][64 + 4];  // [k][col]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 64, cb = c0 + static_cast<int64_t>(blockIdx.x) * 64;
  const int count = a.count;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < count; k0 += KC) {
    const int kc = min(KC, count - k0);
    for (int idx = threadIdx.x; idx < kc * 64; idx += 256) {
      const int r = idx / kc, k = idx - r * kc;  // Err rows are contiguous along k
      e_s[k][r] = (r0 + r < a.rows) ? a.err[(r0 + r) * kGptqMaxBlock + k0 + k] : 0.0f;
    }
    for (int idx = threadIdx.x; idx < kc * 64; idx += 256) {
      const int k = idx >> 6, cc = idx & 63;
      h_s[k][cc] = (cb + cc < a.cols) ? a.hinv[static_cast<int64_t>(a.i1 + k0 + k) * a.cols + cb + cc] : 0.0f;
    }
    __syncthreads();
    for (int k = 0; k < kc; ++k) {
      const float4 ev = *reinterpret_cast<const float4*>(&e_s[k][ty * 4]);
      const float4 hv = *reinterpret_cast<const float4*>(&h_s[k][tx * 4]);
      const float e4[4] = {ev.x, ev.y, ev.z, ev.w}, h4[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(e4[i], h4[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = r0 + ty * 4 + i;
    if (r >= a.rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t cc = cb + tx * 4 + j;
      if (cc < a.cols) a.w[r * a.cols + cc] = __fsub_rn(a.w[r * a.cols + cc], acc[i][j]);
    }
  }
}

// tensor-core trailing update and its helpers (hessian_tc.cu)
bool gptq_trailing_tc_available();
int gptq_split_slab(const float* hinv, int64_t cols, int i1, int64_t c0, int64_t n, __nv_bfloat16* slab_planes,
                    int64_t slab_ld, cudaStream_t st);
int gptq_trailing_tc(float* w_c, int64_t ld, int64_t rows, int64_t n, const __nv_bfloat16* err_planes, int64_t err_ld,
                     const __nv_bfloat16* slab_c, int64_t slab_ld, cudaStream_t st);

struct GptqTrailingPlan;  // tensor maps of one call's rest updates, encoded once (hessian_tc.cu)
int gptq_trailing_plan_create(GptqTrailingPlan** out, float* w, int64_t ld, int64_t rows, int64_t cols,
                              const __nv_bfloat16* const err_planes[2], int64_t err_ld,
                              const __nv_bfloat16* const slab_planes[2], int64_t slab_ld);
void gptq_trailing_plan_destroy(GptqTrailingPlan* p);
int gptq_trailing_plan_run(const GptqTrailingPlan* p, int which, int64_t c, int64_t slab_col, cudaStream_t st);

struct GptqTcScratch {
  __nv_bfloat16* err_planes[2] = {nullptr, nullptr};   // [3 * 128, err_ld] each, alternating between blocks
  __nv_bfloat16* slab_planes[2] = {nullptr, nullptr};  // [3 * 128, slab_ld] each
  int64_t slab_ld = 0;
  float* err_second = nullptr;  // second buffer of error columns [rows, 128]
};

// Side stream and events of the look-ahead schedule: one set per (device, caller stream), created on first use and
// kept for the life of the process, so that calls enqueued on different streams of one device (the sweeps of layers
// that share a factor) do not queue behind one another on a common side stream.
struct Lookahead {
  cudaStream_t side = nullptr;
  cudaEvent_t panel_done = nullptr, rest_done[2] = {nullptr, nullptr};
  std::mutex in_use;  // held while a call enqueues: two host threads may target the same stream
};
std::mutex g_lookahead_mutex;
std::map<std::pair<int, cudaStream_t>, std::unique_ptr<Lookahead>> g_lookahead;

int lookahead_for(cudaStream_t st, Lookahead** out) {
  int dev = 0;
  NNCFB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_lookahead_mutex);
  auto& slot = g_lookahead[std::make_pair(dev, st)];
  if (!slot) {
    std::unique_ptr<Lookahead> l(new Lookahead());
    // lowest priority: when an SM has room, a waiting CTA of the sweep (the critical path) goes before a tile of the rest
    int least = 0, greatest = 0;
    NNCFB_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    NNCFB_CUDA(cudaStreamCreateWithPriority(&l->side, cudaStreamNonBlocking, least));
    NNCFB_CUDA(cudaEventCreateWithFlags(&l->panel_done, cudaEventDisableTiming));
    NNCFB_CUDA(cudaEventCreateWithFlags(&l->rest_done[0], cudaEventDisableTiming));
    NNCFB_CUDA(cudaEventCreateWithFlags(&l->rest_done[1], cudaEventDisableTiming));
    slot = std::move(l);
  }
  *out = slot.get();
  return NNCFB_OK;
}

// ScaleEstimation inside the sweep (WC/gptq.py:319-327): statistics after process_stats
struct GptqSe {
  const float* importance = nullptr;  // [cols] s = max |X| over samples; null: plain min/max parameters
  const float* x = nullptr;           // [cols, n]
  int n = 0, initial_steps = 0, scale_steps = 0;
  float weight_penalty = -1.0f;
};

int scale_estimation_launch(const void* weight, int32_t weight_dtype, int64_t rows, int64_t cols, int64_t ld,
                            int64_t group_size, int32_t mode, const float* importance, const float* x, int32_t n_samples,
                            int32_t initial_steps, int32_t scale_steps, float weight_penalty, float* scale_out,
                            int32_t* zp_out, int64_t out_ld, cudaStream_t st);

// Schedule with the tensor-core trailing update ("look-ahead"): the update of block b is split into the panel
// that the next block needs (its 128 columns) and the rest.  The rest runs on a side stream, concurrently with
// the sweep of block b + 1 (a latency chain that needs few issue slots while the rest keeps the tensor cores and
// the memory system busy).  The panel is normally not a launch: the sweep of block b + 1 applies block b's
// errors to its own columns in fp32 while it loads them, so one sweep follows the other on the caller's stream;
// where that is not possible (ScaleEstimation, a ragged last block) the panel runs as a tensor-core launch
// between the two sweeps.  Every element of W still receives the updates of blocks 0, 1, 2, ... in that order
// (rest(b - 1) completes before the sweep of block b + 1 or panel(b) starts), so results do not depend on the
// schedule.  Error columns, error planes and slab planes alternate between two buffers: block b + 1 writes one
// set while rest(b) reads the other.
template <int MODE>
int run_gptq(GptqArgs a, int block, const GptqTcScratch& tc, const GptqSe& se, cudaStream_t st) {
  const size_t smem = SweepSmem::bytes;
  auto sweep = gptq_sweep_kernel<MODE>;
  NNCFB_CUDA(cudaFuncSetAttribute(sweep, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const unsigned row_blocks = static_cast<unsigned>((a.rows + kSweepWarps * kSweepRows - 1) / (kSweepWarps * kSweepRows));
  // Full blocks with 16-byte aligned rows take the kernel that spreads a row over several lanes.  Its grid is at
  // most one CTA per SM; the warps per CTA are the fewest that cover all rows in the smallest number of rounds.
  // (group starts on multiples of four columns are looked for once per quad of columns)
  auto sweep_fast = (a.gs & 3) == 0 ? gptq_sweep_fast_kernel<MODE, true> : gptq_sweep_fast_kernel<MODE, false>;
  const bool aligned = (a.cols & 3) == 0 && (block & 3) == 0 && a.gs * kSweepMaxGroups >= kGptqMaxBlock &&
                       ((reinterpret_cast<uintptr_t>(a.hinv) | reinterpret_cast<uintptr_t>(a.w) |
                         reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.err)) & 15u) == 0;
  int fast_warps = 4, fast_ctas = 1;
  if (aligned) {
    int dev = 0, sms = 0;
    NNCFB_CUDA(cudaGetDevice(&dev));
    NNCFB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t row_groups = (a.rows + kFsRows - 1) / kFsRows;
    const int64_t rounds = (row_groups + static_cast<int64_t>(sms) * kFsMaxWarps - 1) / (static_cast<int64_t>(sms) * kFsMaxWarps);
    while (fast_warps < kFsMaxWarps && (row_groups + static_cast<int64_t>(sms) * fast_warps - 1) / (static_cast<int64_t>(sms) * fast_warps) > rounds)
      ++fast_warps;
    fast_ctas = static_cast<int>(std::min<int64_t>(sms, (row_groups + fast_warps - 1) / fast_warps));
    NNCFB_CUDA(cudaFuncSetAttribute(sweep_fast, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(FastSweepSmem::bytes(kFsMaxWarps, true))));
  }
  const bool use_tc = tc.slab_planes[0] != nullptr;
  Lookahead* la = nullptr;
  std::unique_lock<std::mutex> lock;
  if (use_tc) {
    const int rc = lookahead_for(st, &la);
    if (rc != NNCFB_OK) return rc;
    lock = std::unique_lock<std::mutex>(la->in_use);  // the side stream and its events belong to one call at a time
  }
  // A group that reaches beyond its block makes the sweep read columns the previous block's rest update is
  // still writing, so the two may only overlap when every group lies inside one block.
  const bool overlap = use_tc && block % a.gs == 0;
  std::unique_ptr<GptqTrailingPlan, void (*)(GptqTrailingPlan*)> plan(nullptr, gptq_trailing_plan_destroy);
  if (use_tc) {
    GptqTrailingPlan* raw = nullptr;
    const int rc = gptq_trailing_plan_create(&raw, a.w, a.cols, a.rows, a.cols, tc.err_planes, a.err_ld, tc.slab_planes,
                                             tc.slab_ld);
    if (rc != NNCFB_OK) return rc;
    plan.reset(raw);
  }
  // When the next block is a full one for the lane-split kernel, the panel is not a launch at all: that sweep
  // applies the previous block's errors to its own columns while it loads them (GptqArgs::err_prev), the slab
  // split moves to the side stream, and one sweep follows the other on the caller's stream.  The error columns
  // then alternate between two buffers.  ScaleEstimation reads the tensor-level weight before the sweep, so it
  // keeps the panel launch.
  const bool can_fuse = overlap && aligned && se.importance == nullptr && tc.err_second != nullptr;
  float* const err_buf[2] = {a.err, can_fuse ? tc.err_second : a.err};
  bool rest_pending[2] = {false, false};  // rest(b) is recorded in rest_done[b & 1] until somebody waits for it
  auto wait_rest = [&](int which) -> int {
    if (rest_pending[which]) NNCFB_CUDA(cudaStreamWaitEvent(st, la->rest_done[which], 0));
    rest_pending[which] = false;
    return NNCFB_OK;
  };
  bool fused_prev = false;
  int64_t blk = 0;
  for (int64_t i1 = 0; i1 < a.cols; i1 += block, ++blk) {
    const int par = static_cast<int>(blk & 1);
    a.i1 = static_cast<int>(i1);
    a.count = static_cast<int>(std::min<int64_t>(block, a.cols - i1));
    a.given = 0;
    a.err = err_buf[par];
    a.err_prev = fused_prev ? err_buf[par ^ 1] : nullptr;
    if (use_tc) a.err_planes = tc.err_planes[par];
    if (se.importance != nullptr) {
      // The groups that start inside this block are refined now: the tensor-level weight they are computed
      // from has received every earlier block's trailing update and is not touched again before the sweep.
      // One call per block covers them all (groups are independent in ScaleEstimation).
      const int64_t first = ((i1 + a.gs - 1) / a.gs) * a.gs;
      if (first < i1 + a.count) {
        const int64_t n_groups = (i1 + a.count - 1 - first) / a.gs + 1;
        const int rc = scale_estimation_launch(a.w + first, NNCFB_F32, a.rows, n_groups * a.gs, a.cols, a.gs, MODE,
                                               se.importance + first, se.x + first * se.n, se.n, se.initial_steps,
                                               se.scale_steps, se.weight_penalty, a.scale + first / a.gs,
                                               a.zp ? a.zp + first / a.gs : nullptr, a.G, st);
        if (rc != NNCFB_OK) return rc;
      }
      a.given = 1;
    }
    // rest(b - 2) updated this block's columns and read the planes that this sweep is about to overwrite
    if (use_tc) {
      const int rc = wait_rest(par);
      if (rc != NNCFB_OK) return rc;
    }
    if (aligned && a.count == kGptqMaxBlock) {
      sweep_fast<<<fast_ctas, fast_warps * 32, FastSweepSmem::bytes(fast_warps, a.err_prev != nullptr), st>>>(a);
    } else {
      sweep<<<row_blocks, kSweepWarps * kSweepRows, smem, st>>>(a);
    }
    fused_prev = false;
    const int64_t c0 = i1 + a.count;
    if (c0 >= a.cols) continue;
    if (!use_tc) {
      const dim3 grid(static_cast<unsigned>((a.cols - c0 + 63) / 64), static_cast<unsigned>((a.rows + 63) / 64));
      gptq_trailing_kernel<<<grid, 256, 0, st>>>(a, c0);
      continue;
    }
    __nv_bfloat16* slab = tc.slab_planes[par];
    const int64_t panel = std::min<int64_t>(block, a.cols - c0);
    const int64_t rest_n = a.cols - c0 - panel;
    const bool fuse = can_fuse && panel == kGptqMaxBlock;
    int rc = NNCFB_OK;
    if (!fuse) {
      rc = gptq_split_slab(a.hinv, a.cols, a.i1, c0, a.cols - c0, slab, tc.slab_ld, st);
      if (rc != NNCFB_OK) return rc;
      // rest(b - 1) also updates the panel's columns: it has to finish first
      rc = wait_rest(par ^ 1);
      if (rc != NNCFB_OK) return rc;
      rc = gptq_trailing_tc(a.w + c0, a.cols, a.rows, panel, a.err_planes, a.err_ld, slab, tc.slab_ld, st);
      if (rc != NNCFB_OK) return rc;
    }
    fused_prev = fuse;
    if (rest_n > 0) {
      cudaStream_t rest_stream = st;
      if (overlap) {
        NNCFB_CUDA(cudaEventRecord(la->panel_done, st));
        NNCFB_CUDA(cudaStreamWaitEvent(la->side, la->panel_done, 0));
        rest_stream = la->side;
      }
      if (fuse) {
        rc = gptq_split_slab(a.hinv, a.cols, a.i1, c0 + panel, rest_n, slab + panel, tc.slab_ld, rest_stream);
        if (rc != NNCFB_OK) return rc;
      }
      rc = gptq_trailing_plan_run(plan.get(), par, c0 + panel, panel, rest_stream);
      if (rc != NNCFB_OK) return rc;
      if (overlap) {
        NNCFB_CUDA(cudaEventRecord(la->rest_done[par], la->side));
        rest_pending[par] = true;
      }
    }
  }
  if (use_tc) {  // nothing is left running on the side stream
    for (int which = 0; which < 2; ++which) {
      const int rc = wait_rest(which);
      if (rc != NNCFB_OK) return rc;
    }
  }
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

// ---- Hessian, CUDA-core fp32 path --------------------------------------------------------------
// H[i0.., j0..] = alpha * H + beta * X^T X for one 64 x 64 tile with j-tile >= i-tile; the lower
// triangle is mirrored afterwards.  Exact fp32 products and fp32 accumulation in token order.
template <typename SrcT>
__global__ void __launch_bounds__(256) hessian_simt_kernel(float* __restrict__ H, const SrcT* __restrict__ x,
                                                           int64_t tokens, int64_t C, float alpha, float beta) {
  if (blockIdx.x < blockIdx.y) return;  // upper triangle of tiles only
  __shared__ __align__(16) float a_s[32][64 + 4], b_s[32][64 + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t i0 = static_cast<int64_t>(blockIdx.y) * 64, j0 = static_cast<int64_t>(blockIdx.x) * 64;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int64_t t0 = 0; t0 < tokens; t0 += 32) {
    for (int idx = threadIdx.x; idx < 32 * 64; idx += 256) {
      const int k = idx >> 6, cc = idx & 63;
      const bool tk = t0 + k < tokens;
      a_s[k][cc] = (tk && i0 + cc < C) ? to_f32<SrcT>(x[(t0 + k) * C + i0 + cc]) : 0.0f;
      b_s[k][cc] = (tk && j0 + cc < C) ? to_f32<SrcT>(x[(t0 + k) * C + j0 + cc]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&a_s[k][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&b_s[k][tx * 4]);
      const float a4[4] = {av.x, av.y, av.z, av.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(a4[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = i0 + ty * 4 + i;
    if (r >= C) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t cc = j0 + tx * 4 + j;
      if (cc < C) H[r * C + cc] = __fmaf_rn(beta, acc[i][j], __fmul_rn(alpha, H[r * C + cc]));
    }
  }
}

__global__ void __launch_bounds__(256) mirror_upper_kernel(float* __restrict__ H, int64_t C) {
  __shared__ float tile[32][33];
  if (blockIdx.x <= blockIdx.y && !(blockIdx.x == blockIdx.y)) return;  // source tiles: strictly upper + diagonal
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32, c0 = static_cast<int64_t>(blockIdx.x) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8) {
    const int64_t r = r0 + k, cc = c0 + tx;
    tile[k][tx] = (r < C && cc < C) ? H[r * C + cc] : 0.0f;
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int64_t r = c0 + k, cc = r0 + tx;  // transposed position
    if (r < C && cc < C && r > cc) H[r * C + cc] = tile[tx][k];
  }
}

}  // namespace nncfb

using namespace nncfb;

namespace {
constexpr size_t align1k(size_t v) { return (v + 1023) & ~static_cast<size_t>(1023); }
size_t err_bytes(int64_t rows) { return align1k(static_cast<size_t>(rows) * kGptqMaxBlock * sizeof(float)); }
int64_t round8(int64_t v) { return (v + 7) & ~static_cast<int64_t>(7); }
size_t planes_bytes(int64_t extent) { return align1k(static_cast<size_t>(3) * kGptqMaxBlock * round8(extent) * 2); }
}  // namespace

extern "C" size_t nncfb_gptq_workspace_bytes(int64_t rows) {
  return rows > 0 ? static_cast<size_t>(rows) * kGptqMaxBlock * sizeof(float) : 0;
}

extern "C" size_t nncfb_gptq_workspace_bytes_tensor_cores(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return 2 * err_bytes(rows) + 2 * planes_bytes(rows) + 2 * planes_bytes(cols);
}

namespace nncfb {
static int gptq_quantize_impl(float* weight, int64_t rows, int64_t cols, const float* hinv, int32_t mode,
                              int64_t group_size, int32_t block_size, float* q_out, float* scale_out, int32_t* zp_out,
                              void* workspace, size_t workspace_bytes, GptqSe se, void* stream) {
  NNCFB_CHECK_ARG(weight && hinv && q_out && scale_out && workspace, NNCFB_E_BAD_ARG, "nncfb_gptq_quantize: null pointer");
  NNCFB_CHECK_ARG(rows > 0 && cols > 0, NNCFB_E_BAD_ARG, "nncfb_gptq_quantize: bad shape");
  NNCFB_CHECK_ARG(group_size > 0 && cols % group_size == 0, NNCFB_E_GROUP_SIZE,
                  "Channel size %lld should be divisible by size of group %lld.", (long long)cols, (long long)group_size);
  NNCFB_CHECK_ARG(block_size > 0 && block_size <= kGptqMaxBlock, NNCFB_E_TOO_LARGE,
                  "nncfb_gptq_quantize: block size %d is outside (0, %d]", block_size, kGptqMaxBlock);
  NNCFB_CHECK_ARG(!mode_is_asym(mode) || zp_out, NNCFB_E_BAD_ARG, "nncfb_gptq_quantize: zp_out is null");
  NNCFB_CHECK_ARG(workspace_bytes >= nncfb_gptq_workspace_bytes(rows), NNCFB_E_BAD_ARG,
                  "nncfb_gptq_quantize: workspace of %zu bytes is smaller than nncfb_gptq_workspace_bytes() = %zu",
                  workspace_bytes, nncfb_gptq_workspace_bytes(rows));
  GptqArgs a;
  a.w = weight;
  a.hinv = hinv;
  a.q = q_out;
  a.err = static_cast<float*>(workspace);
  a.err_prev = nullptr;
  a.err_planes = nullptr;
  a.err_ld = 0;
  a.scale = scale_out;
  a.zp = mode_is_asym(mode) ? zp_out : nullptr;
  a.rows = rows;
  a.cols = cols;
  a.gs = group_size;
  a.G = cols / group_size;
  a.i1 = 0;
  a.count = 0;
  // The trailing update runs on the tensor cores when the caller's workspace has room for the operand planes
  // (nncfb_gptq_workspace_bytes_tensor_cores) and the shapes allow 16-byte rows: full 128-column blocks, more
  // than one block, rows % 8 == 0, cols % 4 == 0, 16-byte aligned weight.  Otherwise the fp32 CUDA-core kernel.
  GptqTcScratch tc;
  if (workspace_bytes >= nncfb_gptq_workspace_bytes_tensor_cores(rows, cols) && block_size == kGptqMaxBlock &&
      cols > kGptqMaxBlock && rows % 8 == 0 && cols % 4 == 0 && aligned16(weight) && aligned16(workspace) &&
      gptq_trailing_tc_available()) {
    tc.err_second = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + err_bytes(rows));
    uint8_t* base = static_cast<uint8_t*>(workspace) + 2 * err_bytes(rows);
    for (int i = 0; i < 2; ++i) {
      tc.err_planes[i] = reinterpret_cast<__nv_bfloat16*>(base + i * planes_bytes(rows));
      tc.slab_planes[i] = reinterpret_cast<__nv_bfloat16*>(base + 2 * planes_bytes(rows) + i * planes_bytes(cols));
    }
    a.err_planes = tc.err_planes[0];
    a.err_ld = round8(rows);
    tc.slab_ld = round8(cols);
  }
  a.given = 0;
  // the reference refines 4-bit integer groups only (WC/gptq.py:319); other modes keep min/max parameters
  if (mode != NNCFB_INT4_SYM && mode != NNCFB_INT4_ASYM) se = GptqSe();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (mode) {
    case NNCFB_INT4_SYM: return run_gptq<NNCFB_INT4_SYM>(a, block_size, tc, se, st);
    case NNCFB_INT4_ASYM: return run_gptq<NNCFB_INT4_ASYM>(a, block_size, tc, se, st);
    case NNCFB_INT8_SYM: return run_gptq<NNCFB_INT8_SYM>(a, block_size, tc, se, st);
    case NNCFB_INT8_ASYM: return run_gptq<NNCFB_INT8_ASYM>(a, block_size, tc, se, st);
    case NNCFB_NF4: return run_gptq<NNCFB_NF4>(a, block_size, tc, se, st);
    case NNCFB_FP4: return run_gptq<NNCFB_FP4>(a, block_size, tc, se, st);
    case NNCFB_MXFP4: return run_gptq<NNCFB_MXFP4>(a, block_size, tc, se, st);
    default: break;
  }
  set_error("nncfb_gptq_quantize: mode %d is not supported", mode);
  return NNCFB_E_UNSUPPORTED;
}
}  // namespace nncfb

extern "C" int nncfb_gptq_quantize(float* weight, int64_t rows, int64_t cols, const float* hinv, int32_t mode,
                                   int64_t group_size, int32_t block_size, float* q_out, float* scale_out,
                                   int32_t* zp_out, void* workspace, size_t workspace_bytes, void* stream) {
  return gptq_quantize_impl(weight, rows, cols, hinv, mode, group_size, block_size, q_out, scale_out, zp_out, workspace,
                            workspace_bytes, GptqSe(), stream);
}

extern "C" int nncfb_gptq_quantize_se(float* weight, int64_t rows, int64_t cols, const float* hinv, int32_t mode,
                                      int64_t group_size, int32_t block_size, const float* importance, const float* x,
                                      int32_t n_samples, int32_t initial_steps, int32_t scale_steps, float weight_penalty,
                                      float* q_out, float* scale_out, int32_t* zp_out, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  NNCFB_CHECK_ARG(importance && x && n_samples > 0, NNCFB_E_BAD_ARG, "nncfb_gptq_quantize_se: statistics are missing");
  NNCFB_CHECK_ARG(group_size <= 512, NNCFB_E_TOO_LARGE,
                  "nncfb_gptq_quantize_se: group size %lld exceeds the supported maximum of 512 of scale estimation",
                  (long long)group_size);
  GptqSe se;
  se.importance = importance;
  se.x = x;
  se.n = n_samples;
  se.initial_steps = initial_steps;
  se.scale_steps = scale_steps;
  se.weight_penalty = weight_penalty;
  return gptq_quantize_impl(weight, rows, cols, hinv, mode, group_size, block_size, q_out, scale_out, zp_out, workspace,
                            workspace_bytes, se, stream);
}


// ---- GPTQ sweep for callers that cannot hand over scratch memory -----------------------------------
// Some programs that embed this library have no device allocator to offer: a runtime that gave every
// byte of HBM to its own arena at start-up and exposes no allocation hook through a C interface, or a
// service loop in which cudaMalloc (which synchronises the whole device) must never run.  For them the
// error-column scratch of the sweep lives in this fixed array instead of a caller buffer.  It is part of
// the library image: every GPU that loads the library holds these 8 MiB until the process exits.
namespace nncfb {
constexpr int64_t kNoAllocMaxRows = 16384;
static __device__ __align__(256) float g_gptq_noalloc_scratch[kNoAllocMaxRows * kGptqMaxBlock];

namespace {
std::mutex g_noalloc_mutex;
float* g_noalloc_ptr[64] = {};  // device address of the array, per device ordinal
}  // namespace

// Device address of the scratch array on the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, so it is resolved once per device (with that
// device current) through cudaGetSymbolAddress and cached.
static int noalloc_scratch(float** out) {
  int dev = 0;
  NNCFB_CUDA(cudaGetDevice(&dev));
  NNCFB_CHECK_ARG(dev >= 0 && dev < 64, NNCFB_E_UNSUPPORTED, "nncfb_gptq_quantize_noalloc: device ordinal %d >= 64", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    NNCFB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_gptq_noalloc_scratch));
    NNCFB_CHECK_ARG(p != nullptr, NNCFB_E_CUDA, "nncfb_gptq_quantize_noalloc: scratch symbol has no device address");
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return NNCFB_OK;
}
}  // namespace nncfb

extern "C" int nncfb_gptq_quantize_noalloc(float* weight, int64_t rows, int64_t cols, const float* hinv, int32_t mode,
                                           int64_t group_size, int32_t block_size, float* q_out, float* scale_out,
                                           int32_t* zp_out, void* stream) {
  NNCFB_CHECK_ARG(rows <= kNoAllocMaxRows, NNCFB_E_TOO_LARGE,
                  "nncfb_gptq_quantize_noalloc: %lld rows exceed the built-in scratch (maximum %lld rows); use "
                  "nncfb_gptq_quantize with a caller workspace",
                  (long long)rows, (long long)kNoAllocMaxRows);
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != NNCFB_OK) return rc;
  // Nothing in the scratch has to start at zero: each block's sweep writes every error column of every
  // row before the trailing update reads it, so contents left by an earlier call are never observed.
  // The size handed on is the minimum for `rows`, not the size of the array: a larger figure would let mid-size
  // problems qualify for the tensor-core look-ahead schedule, which creates a stream and two events on first
  // use and rounds differently.  With the minimum, the fp32 CUDA-core trailing update always runs.
  return nncfb_gptq_quantize(weight, rows, cols, hinv, mode, group_size, block_size, q_out, scale_out, zp_out, scratch,
                             nncfb_gptq_workspace_bytes(rows), stream);
}

namespace nncfb {
// tensor-core path for 16-bit activations (hessian_tc.cu); returns NNCFB_E_UNSUPPORTED when the
// shape does not fit its tiling, in which case the CUDA-core kernel above runs.
int hessian_tc_accumulate(float* H, int64_t C, const void* x, int dtype, int64_t tokens, float alpha, float beta,
                          void* workspace, size_t workspace_bytes, cudaStream_t st);
}  // namespace nncfb

extern "C" int nncfb_hessian_accumulate(float* hessian, int64_t channels, const void* x, int32_t dtype, int64_t tokens,
                                        float alpha, float beta, int32_t allow_tensor_cores, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  NNCFB_CHECK_ARG(hessian && x, NNCFB_E_BAD_ARG, "nncfb_hessian_accumulate: null pointer");
  NNCFB_CHECK_ARG(channels > 0 && tokens > 0, NNCFB_E_BAD_ARG, "nncfb_hessian_accumulate: bad shape");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (allow_tensor_cores && (dtype == NNCFB_BF16 || dtype == NNCFB_F16)) {
    const int rc = hessian_tc_accumulate(hessian, channels, x, dtype, tokens, alpha, beta, workspace, workspace_bytes, st);
    if (rc != NNCFB_E_UNSUPPORTED) return rc;
  }
  const dim3 grid(static_cast<unsigned>((channels + 63) / 64), static_cast<unsigned>((channels + 63) / 64));
  switch (dtype) {
    case NNCFB_F32:
      hessian_simt_kernel<float><<<grid, 256, 0, st>>>(hessian, static_cast<const float*>(x), tokens, channels, alpha, beta);
      break;
    case NNCFB_F16:
      hessian_simt_kernel<__half><<<grid, 256, 0, st>>>(hessian, static_cast<const __half*>(x), tokens, channels, alpha, beta);
      break;
    case NNCFB_BF16:
      hessian_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(hessian, static_cast<const __nv_bfloat16*>(x), tokens,
                                                               channels, alpha, beta);
      break;
    default:
      set_error("nncfb_hessian_accumulate: unsupported dtype %d", dtype);
      return NNCFB_E_BAD_ARG;
  }
  NNCFB_CUDA(cudaGetLastError());
  const dim3 mgrid(static_cast<unsigned>((channels + 31) / 32), static_cast<unsigned>((channels + 31) / 32));
  mirror_upper_kernel<<<mgrid, 256, 0, st>>>(hessian, channels);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}
