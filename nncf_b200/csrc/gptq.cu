// GPTQ: blocked column sweep with error feedback, the lazy-batch trailing update and the fp32
// (CUDA-core) Hessian accumulation.
//
// Restates GPTQ._quantize_weights of the reference
// (src/nncf/quantization/algorithms/weight_compression/gptq.py:297-379) after its Hessian
// preparation (dead columns, damping, Cholesky inverse: host-side library calls).  The reference
// walks the columns in Python with ~8 small tensor operations per column; here one C call runs
//   gptq_sweep_kernel     once per 128-column block: a thread owns an output row; the block's weights,
//                         the matching Hinv block and the error columns live in shared memory;
//                         group parameters are taken at each group start from the tensor-level weight
//                         (updated at block ends only), exactly as the reference indexes it;
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

struct GptqTcScratch {
  __nv_bfloat16* err_planes[2] = {nullptr, nullptr};   // [3 * 128, err_ld] each, alternating between blocks
  __nv_bfloat16* slab_planes[2] = {nullptr, nullptr};  // [3 * 128, slab_ld] each
  int64_t slab_ld = 0;
};

// Side stream and events of the look-ahead schedule: one set per (device, caller stream), created on first use and
// kept for the life of the process, so that calls enqueued on different streams of one device (the sweeps of layers
// that share a factor) do not queue behind one another on a common side stream.
struct Lookahead {
  cudaStream_t side = nullptr;
  cudaEvent_t panel_done = nullptr, rest_done = nullptr;
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
    NNCFB_CUDA(cudaStreamCreateWithFlags(&l->side, cudaStreamNonBlocking));
    NNCFB_CUDA(cudaEventCreateWithFlags(&l->panel_done, cudaEventDisableTiming));
    NNCFB_CUDA(cudaEventCreateWithFlags(&l->rest_done, cudaEventDisableTiming));
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
// that the next block needs (its 128 columns) and the rest.  The panel runs on the caller's stream right after
// the sweep; the rest runs on a side stream, concurrently with the sweep of block b + 1, which is a latency
// chain on a few SMs while the rest keeps the others busy.  Every element of W still receives the updates of
// blocks 0, 1, 2, ... in that order (rest(b - 1) completes before panel(b) starts), so results do not depend on
// the schedule.  Error planes and slab planes alternate between two buffers: block b + 1 writes one set while
// rest(b) reads the other.
template <int MODE>
int run_gptq(GptqArgs a, int block, const GptqTcScratch& tc, const GptqSe& se, cudaStream_t st) {
  const size_t smem = SweepSmem::bytes;
  auto sweep = gptq_sweep_kernel<MODE>;
  NNCFB_CUDA(cudaFuncSetAttribute(sweep, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const unsigned row_blocks = static_cast<unsigned>((a.rows + kSweepWarps * kSweepRows - 1) / (kSweepWarps * kSweepRows));
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
  bool rest_pending = false;
  int64_t blk = 0;
  for (int64_t i1 = 0; i1 < a.cols; i1 += block, ++blk) {
    a.i1 = static_cast<int>(i1);
    a.count = static_cast<int>(std::min<int64_t>(block, a.cols - i1));
    a.given = 0;
    if (use_tc) a.err_planes = tc.err_planes[blk & 1];
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
    sweep<<<row_blocks, kSweepWarps * kSweepRows, smem, st>>>(a);
    const int64_t c0 = i1 + a.count;
    if (c0 >= a.cols) continue;
    if (!use_tc) {
      const dim3 grid(static_cast<unsigned>((a.cols - c0 + 63) / 64), static_cast<unsigned>((a.rows + 63) / 64));
      gptq_trailing_kernel<<<grid, 256, 0, st>>>(a, c0);
      continue;
    }
    __nv_bfloat16* slab = tc.slab_planes[blk & 1];
    int rc = gptq_split_slab(a.hinv, a.cols, a.i1, c0, a.cols - c0, slab, tc.slab_ld, st);
    if (rc != NNCFB_OK) return rc;
    // rest(b - 1) also updates the panel's columns: it has to finish first
    if (rest_pending) NNCFB_CUDA(cudaStreamWaitEvent(st, la->rest_done, 0));
    const int64_t panel = std::min<int64_t>(block, a.cols - c0);
    rc = gptq_trailing_tc(a.w + c0, a.cols, a.rows, panel, a.err_planes, a.err_ld, slab, tc.slab_ld, st);
    if (rc != NNCFB_OK) return rc;
    rest_pending = false;
    if (c0 + panel < a.cols) {
      cudaStream_t rest_stream = st;
      if (overlap) {
        NNCFB_CUDA(cudaEventRecord(la->panel_done, st));
        NNCFB_CUDA(cudaStreamWaitEvent(la->side, la->panel_done, 0));
        rest_stream = la->side;
      }
      rc = gptq_trailing_tc(a.w + c0 + panel, a.cols, a.rows, a.cols - c0 - panel, a.err_planes, a.err_ld, slab + panel,
                            tc.slab_ld, rest_stream);
      if (rc != NNCFB_OK) return rc;
      if (overlap) {
        NNCFB_CUDA(cudaEventRecord(la->rest_done, la->side));
        rest_pending = true;
      }
    }
  }
  if (rest_pending) NNCFB_CUDA(cudaStreamWaitEvent(st, la->rest_done, 0));  // nothing is left running on the side stream
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
  return err_bytes(rows) + 2 * planes_bytes(rows) + 2 * planes_bytes(cols);
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
    uint8_t* base = static_cast<uint8_t*>(workspace) + err_bytes(rows);
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
