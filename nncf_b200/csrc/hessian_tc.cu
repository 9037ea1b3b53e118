// GPTQ Hessian accumulation H = alpha * H + beta * X^T X on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory, operands staged by TMA).
//
// Restates the contraction of GPTQ._calculate_hessian
// (src/nncf/quantization/algorithms/weight_compression/gptq.py:200-242): X is an activation
// [tokens, C] in bf16 / fp16, H is fp32 [C, C].  Products of 16-bit values are exact in fp32 and the
// accumulation is fp32 in tensor memory, so the result is fp32-faithful without operand splitting;
// the scale factors are applied once in the epilogue instead of to every element of X.
//
// Both operands are the SAME matrix X read "MN-major": A = X^T (M = channels i, K = tokens) and
// B = X (K = tokens, N = channels j) both have the channel index contiguous in memory, so no
// transposed copy of X is ever made.  A TMA box of 64 channels x 64 tokens with 128-byte swizzle is
// exactly one canonical MN-major swizzle-128B operand atom column (8 token rows per 1024-byte atom).
//
// A CTA computes 128 x 256 tiles of the upper triangle of H over all tokens, one after the other (one
// persistent CTA per SM; the accumulator is double-buffered in tensor memory so that a tile's epilogue
// overlaps the next tile's MMAs):
//   warp 0        TMA producer (one elected lane), 4-stage ring running across tiles, mbarrier expect-tx
//   warp 1        tensor-memory allocation, MMA issue (one elected lane), tcgen05.commit
//   warps 2..5    epilogue: tcgen05.ld of the fp32 accumulators, H = alpha*H + beta*acc
// The same kernel, with two tensor maps and twelve K segments, is the lazy-batch trailing update of the
// GPTQ sweep, W[:, i2:] -= Err_blk @ Hinv[i1:i2, i2:] (WC/gptq.py:361-363): both fp32 operands are split into
// three bf16 planes (hi + mid + lo = the fp32 value to 2^-27), stored with the block's 128 rows of K as the
// slow axis, and six plane products (everything down to 2^-24 relative) are accumulated in fp32 in tensor
// memory, smallest terms first.  That update is bound by the read-modify-write of W; it is launched with one
// CTA per tile because it shares the GPU with the next block's sweep kernel.
// Every wait is bounded in time: a role that waited longer than the limit records its code in the launch's
// status word (and in a per-device sticky flag), and leaves; the other roles then see the word or time out
// the same way, tensor memory is released and the kernel returns (the host reports NNCFB_E_TIMEOUT).  Single-CTA TMA loads of this GPU's own memory only.
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <memory>

#include "nncfb_common.cuh"

namespace nncfb {

namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kBoxC = 64;    // channels per TMA box (128 bytes of bf16)
constexpr int kBlockK = 64;  // tokens per pipeline stage
constexpr int kStagesHessian = 4;
// The trailing update runs one tile per CTA (twelve K stages), so a CTA's life is a sequence of phases that do not
// overlap: pipeline ramp-up, MMAs, drain, read-modify-write epilogue.  Two stages (96 KB) and one 256-column
// accumulator let TWO such CTAs live on an SM and fill each other's gaps; four stages and a 512-column
// allocation (what the persistent Hessian kernel wants) would admit one: the second CTA's tensor-memory
// allocation waits until the first one frees its columns.
constexpr int kStagesTrailing = 2;
constexpr int kMaxStages = 4;
constexpr int kBoxBytes = kBoxC * kBlockK * 2;                           // 8192
constexpr int kStageBytes = (kTileM / kBoxC + kTileN / kBoxC) * kBoxBytes;  // 49152
constexpr int kTmemColsPersistent = 512;  // two accumulators of kTileN fp32 columns (tile t + 1 starts while t drains)
constexpr int kTmemColsOneTile = 256;     // one accumulator: a CTA that computes a single tile
constexpr uint64_t kWaitLimitNs = 4000000000ull;  // 4 s per wait: far beyond any legitimate wait of this kernel

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up (returns false) once `limit_ns` nanoseconds have passed without the barrier
// completing the phase.  The clock is read only after a batch of unsuccessful polls, so a wait that is
// satisfied quickly costs what a plain poll loop costs.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i) {
    if (mbar_test(bar, parity)) return true;
  }
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_test(bar, parity)) return true;
    }
    if (global_timer_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// D[y.., x..] += tile: a 2-D bulk tensor reduction from shared memory into global memory (fp32 add done by the
// memory system next to L2, so the tile of D never travels to the SM).  Completion is tracked by the bulk async
// group of the issuing thread.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int x, int y, const void* src) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(smem_u32(src))
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_generic_to_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// MN-major, 128-byte swizzle shared-memory operand descriptor:
//   start address >> 4 | LBO (stride between 64-element atoms along M/N) >> 4 at bit 16 |
//   SBO (stride between groups of 8 K rows) >> 4 at bit 32 | version 1 at bit 46 | layout 2 (SW128) at bit 61
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(kBoxBytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_c),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Order of the upper-triangle tiles of the Hessian.  Tile (mi, nj) (128 rows x 256 columns) is needed when
// nj >= mi / 2.  Tiles are numbered band by band, a band being kBandN tile columns wide, and inside a band
// row by row: the ~148 tiles that are resident together then form a compact patch (about 18 tile rows x 8
// tile columns) that touches ~4.4 K channels of X instead of all of them, so a wave re-reads a third of X
// from HBM rather than the whole matrix (X is 0.9 GB per call at C = 14336, seven times the L2).
constexpr int kBandN = 8;

__host__ __device__ inline int band_tiles(int b, int tiles_m, int tiles_n) {
  const int n_lo = b * kBandN, n_hi = min(n_lo + kBandN, tiles_n);
  int total = 0;
  const int full_rows = min(2 * n_lo, tiles_m);       // rows whose whole band segment is above the diagonal
  const int width = n_hi - n_lo;
  total += full_rows * width;
  if (2 * n_hi <= tiles_m) {
    total += width * (width + 1);  // rows 2 n_lo .. 2 n_hi - 1 hold width, width, width - 1, width - 1, ..., 1, 1 tiles
  } else {
    for (int mi = 2 * n_lo; mi < tiles_m; ++mi) total += n_hi - max(n_lo, mi / 2);
  }
  return total;
}

__host__ __device__ inline int hessian_tile_count(int tiles_m, int tiles_n) {
  int total = 0;
  for (int b = 0; b * kBandN < tiles_n; ++b) total += band_tiles(b, tiles_m, tiles_n);
  return total;
}

__host__ __device__ inline void hessian_tile_decode(int idx, int tiles_m, int tiles_n, int& mi, int& nj) {
  int b = 0;
  for (;; ++b) {
    const int t = band_tiles(b, tiles_m, tiles_n);
    if (idx < t) break;
    idx -= t;
  }
  const int n_lo = b * kBandN, n_hi = min(n_lo + kBandN, tiles_n);
  const int width = n_hi - n_lo;
  const int full_rows = min(2 * n_lo, tiles_m);
  if (idx < full_rows * width) {
    mi = idx / width;
    nj = n_lo + idx - mi * width;
    return;
  }
  idx -= full_rows * width;
  for (mi = 2 * n_lo;; ++mi) {
    const int lo = max(n_lo, mi / 2);
    const int cnt = n_hi - lo;
    if (idx < cnt) {
      nj = lo + idx;
      return;
    }
    idx -= cnt;
  }
}

struct __align__(8) Control {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];   // accumulator buffer b holds a finished tile
  uint64_t acc_empty[2];  // the epilogue has read accumulator buffer b
  uint32_t tmem_base;
  uint32_t pad;
};

// Per-device sticky record of a bounded wait that ran out (static device memory: nothing is allocated).  It is
// raised by any tensor-core launch and cleared only when the host reads it (nncfb_hessian_status), so an
// error in one call of a series is still visible after the last one.
__device__ int g_hessian_status;

__device__ __forceinline__ void give_up(int* status, int role) {
  atomicExch(status, role);           // this launch: the other roles stop at their next check
  atomicMax(&g_hessian_status, role);  // the device: reported by the next nncfb_hessian_status
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent kernel: one CTA per SM walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The operand ring
// runs on across tile boundaries and the accumulator is double-buffered in tensor memory (2 x 256 columns), so
// the producer prefetches the next tile's operands and the MMA warp starts it while the epilogue warps are still
// writing the previous tile back.
// TRAILING = false: D = H [C, C], upper-triangle tiles in banded order, K = tokens, both operands from `amap`.
// TRAILING = true:  D [m_bound, n_bound] += beta * A^T B for fp32 operands given as three bf16 planes each: all tiles,
//                   6 * K / 64 pipeline stages (plane pair (pa, pb) x the K / 64 chunks of the contraction);
//                   A planes in `amap`, B planes in `bmap`, each a 2-D tensor [3 * K, extent] with plane p at rows
//                   [K p, K p + K); `tokens` carries K (128 for the GPTQ block update).  D is updated through `dmap`.
template <int kStages, bool TRAILING>
__global__ void __launch_bounds__(192, TRAILING ? 2 : 1)
tc_tn_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
             const __grid_constant__ CUtensorMap dmap, float* __restrict__ H,
             int64_t ld, int64_t m_bound, int64_t n_bound, int64_t tokens, float alpha, float beta, uint32_t idesc,
             int n_tiles_n, int n_tiles, int* __restrict__ status, uint64_t wait_ns, int producer_short,
             int b_col0, int d_col0) {
  // b_col0 / d_col0: column of `bmap` / `dmap` at which this launch's column 0 lies (maps that cover a whole buffer
  // are encoded once and reused by launches on different column ranges); both multiples of 8
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte aligned operand ring (swizzle-128B atoms must start on 1 KiB), control block behind it
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(ring + kStages * kStageBytes);

  constexpr int kTmemCols = TRAILING ? kTmemColsOneTile : kTmemColsPersistent;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = static_cast<int>((m_bound + kTileM - 1) / kTileM);
  // TRAILING: `tokens` is K, the number of rows of each operand plane (a multiple of 64): six plane pairs x K / 64
  const int k_chunks = static_cast<int>((tokens + kBlockK - 1) / kBlockK);
  const int k_iters = TRAILING ? 6 * k_chunks : k_chunks;
  auto tile_origin = [&](int tile, int& m0, int& n0) {
    int mi, nj;
    if constexpr (TRAILING) {
      mi = tile / n_tiles_n;
      nj = tile - mi * n_tiles_n;
    } else {
      hessian_tile_decode(tile, tiles_m, n_tiles_n, mi, nj);  // nj >= mi / 2: tiles that touch the upper triangle
    }
    m0 = mi * kTileM;
    n0 = nj * kTileN;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int bf = 0; bf < 2; ++bf) {
      mbar_init(&ctl->acc_full[bf], 1);
      mbar_init(&ctl->acc_empty[bf], 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer ------------------------------------------------------------------------
      bool ok = true;
      int g = 0;  // stages issued so far, over all tiles
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int m0, n0;
        tile_origin(tile, m0, n0);
        // producer_short is 0 except in the self test of the bounded waits, where the producer leaves out the last
        // stage(s) of every tile so that the MMA role's wait for them runs out
        for (int it = 0; it < k_iters - producer_short; ++it, ++g) {
          const int s = g % kStages;
          if (!mbar_wait(&ctl->empty[s], ((g / kStages) & 1) ^ 1, wait_ns)) {
            give_up(status, 1);
            ok = false;
            break;
          }
          uint8_t* stage = ring + s * kStageBytes;
          mbar_expect_tx(&ctl->full[s], kStageBytes);
          int ka = it * kBlockK, kb = ka;
          if constexpr (TRAILING) {
            // plane pairs, smallest products first: (lo,hi) (hi,lo) (mid,mid) (mid,hi) (hi,mid) (hi,hi); hi = plane 0;
            // each pair runs over all of K before the next, so the small terms are summed before the large ones
            const int combo = it / k_chunks, chunk = it - combo * k_chunks;
            const int plane_rows = static_cast<int>(tokens);
            ka = static_cast<int>((0x001102u >> (4 * combo)) & 15u) * plane_rows + chunk * kBlockK;
            kb = static_cast<int>((0x010120u >> (4 * combo)) & 15u) * plane_rows + chunk * kBlockK;
          }
#pragma unroll
          for (int b = 0; b < kTileM / kBoxC; ++b)
            tma_load_2d(stage + b * kBoxBytes, &amap, m0 + b * kBoxC, ka, &ctl->full[s]);
#pragma unroll
          for (int b = 0; b < kTileN / kBoxC; ++b)
            tma_load_2d(stage + (kTileM / kBoxC + b) * kBoxBytes, &bmap, b_col0 + n0 + b * kBoxC, kb, &ctl->full[s]);
        }
      }
      // do not leave while a copy into this CTA's shared memory may still be in flight: wait (bounded)
      // for the last copies issued to each stage
      for (int it = max(0, g - kStages); it < g; ++it) {
        if (!mbar_wait(&ctl->full[it % kStages], (it / kStages) & 1, wait_ns)) {
          give_up(status, 4);
          break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----------------------------------------------------------------------------
      bool ok = true;
      int g = 0, t = 0;  // stages consumed, tiles started
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
        const int bf = t & 1;
        // the epilogue must have drained this accumulator buffer (two tiles ago); a fresh barrier passes
        if (!mbar_wait(&ctl->acc_empty[bf], ((t >> 1) & 1) ^ 1, wait_ns)) {
          give_up(status, 5);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(bf * kTileN);
        for (int it = 0; it < k_iters; ++it, ++g) {
          const int s = g % kStages;
          if (!mbar_wait(&ctl->full[s], (g / kStages) & 1, wait_ns)) {
            give_up(status, 2);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(ring + s * kStageBytes);
          const uint32_t b_addr = a_addr + (kTileM / kBoxC) * kBoxBytes;
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            // 16 tokens per instruction = two groups of eight 128-byte rows = 2048 bytes
            const uint64_t adesc = make_desc(a_addr + k * 2048);
            const uint64_t bdesc = make_desc(b_addr + k * 2048);
            umma_f16(tmem_acc, adesc, bdesc, idesc, (it > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&ctl->empty[s]);  // frees the stage when these MMAs have read it
        }
        umma_commit(&ctl->acc_full[bf]);  // accumulator complete (or abandoned: the epilogue checks status)
      }
    }
  } else {
    // ---- epilogue: warps 2..5 own tensor-memory lanes 32 * (warp % 4) ------------------------------
    const int q = warp & 3;
    // Pull this thread's row of a D tile (eight 128-byte lines) into L2 one tile ahead of its read-modify-write,
    // which would otherwise wait for DRAM once per step.
    auto prefetch_tile = [&](int tile) {
      if (tile >= n_tiles) return;
      int pm0, pn0;
      tile_origin(tile, pm0, pn0);
      const int64_t pr = static_cast<int64_t>(pm0) + q * 32 + lane;
      if (pr < m_bound) {
        const float* drow = H + pr * ld + pn0;
#pragma unroll
        for (int c = 0; c < kTileN; c += 32) {
          if (pn0 + c < n_bound) asm volatile("prefetch.global.L2 [%0];" ::"l"(drow + c));
        }
      }
    };
    if constexpr (!TRAILING) prefetch_tile(blockIdx.x);
    int t = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
      const int bf = t & 1;
      int m0, n0;
      tile_origin(tile, m0, n0);
      const int64_t r = static_cast<int64_t>(m0) + q * 32 + lane;
      if constexpr (!TRAILING) prefetch_tile(tile + gridDim.x);
      const bool ok = mbar_wait(&ctl->acc_full[bf], (t >> 1) & 1, wait_ns);
      if (!ok && lane == 0) give_up(status, 3);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!ok || *reinterpret_cast<volatile int*>(status) != 0) break;  // warp-uniform: some role gave up
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(bf * kTileN);
      if constexpr (TRAILING) {
        // D += beta * acc without reading D into the SM: every 32 x 32 piece of the accumulator is written to
        // shared memory (in the 128-byte swizzle the tensor map expects, which also keeps the 16-byte stores of a
        // warp free of bank conflicts) and added to D by a bulk tensor reduction.  Every element of D receives
        // exactly one add per launch, so the result is the correctly rounded D + beta * acc, as before; rows and
        // columns beyond the bounds are clipped by the tensor map.  The staging buffers reuse the operand ring:
        // the accumulator is complete, so every stage has been consumed and nothing else is loaded (one tile per
        // CTA).  Four 4 KB buffers per warp: the reads of the first four reductions are awaited before the fifth.
        uint8_t* stage = ring + static_cast<size_t>(q) * (4 * 4096);
#pragma unroll 1
        for (int c = 0; c < kTileN; c += 32) {
          if (c == 128) {
            if (lane == 0) bulk_wait_read_all();
            __syncwarp();
          }
          uint32_t acc[32];
          tmem_ld32(tmem_acc + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c), acc);
          uint8_t* buf = stage + ((c >> 5) & 3) * 4096;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 v;
            v.x = __fmul_rn(beta, __uint_as_float(acc[4 * j]));
            v.y = __fmul_rn(beta, __uint_as_float(acc[4 * j + 1]));
            v.z = __fmul_rn(beta, __uint_as_float(acc[4 * j + 2]));
            v.w = __fmul_rn(beta, __uint_as_float(acc[4 * j + 3]));
            *reinterpret_cast<float4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
          }
          fence_generic_to_async_smem();
          __syncwarp();
          if (lane == 0 && n0 + c < n_bound && m0 + q * 32 < m_bound) {
            tma_reduce_add_2d(&dmap, d_col0 + n0 + c, m0 + q * 32, buf);
            bulk_commit();
          }
        }
        if (lane == 0) bulk_wait_all();
        __syncwarp();
      } else {
      // tcgen05.ld hands each lane one accumulator row, 32 columns (one 128-byte line of D) per step.  The
      // eight 16-byte loads of a step are issued together, before the first store, so that they overlap.
#pragma unroll 1
      for (int c = 0; c < kTileN; c += 32) {
        uint32_t acc[32];
        tmem_ld32(tmem_acc + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c), acc);
        if (r < m_bound) {
          float* hrow = H + r * ld + n0 + c;
          if (n0 + c + 31 < n_bound) {
            float4 h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = *reinterpret_cast<const float4*>(hrow + 4 * j);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              h[j].x = __fmaf_rn(beta, __uint_as_float(acc[4 * j]), __fmul_rn(alpha, h[j].x));
              h[j].y = __fmaf_rn(beta, __uint_as_float(acc[4 * j + 1]), __fmul_rn(alpha, h[j].y));
              h[j].z = __fmaf_rn(beta, __uint_as_float(acc[4 * j + 2]), __fmul_rn(alpha, h[j].z));
              h[j].w = __fmaf_rn(beta, __uint_as_float(acc[4 * j + 3]), __fmul_rn(alpha, h[j].w));
              *reinterpret_cast<float4*>(hrow + 4 * j) = h[j];
            }
          } else {
            for (int jj = 0; jj < 32; ++jj) {
              if (n0 + c + jj < n_bound) hrow[jj] = __fmaf_rn(beta, __uint_as_float(acc[jj]), __fmul_rn(alpha, hrow[jj]));
            }
          }
        }
      }
      }
      // this warp has read its quarter of the buffer: hand it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[bf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

__global__ void __launch_bounds__(256) mirror_upper_tc_kernel(float* __restrict__ H, int64_t C) {
  __shared__ float tile[32][33];
  if (blockIdx.x < blockIdx.y) return;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32, c0 = static_cast<int64_t>(blockIdx.x) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8) {
    const int64_t r = r0 + k, cc = c0 + tx;
    tile[k][tx] = (r < C && cc < C) ? H[r * C + cc] : 0.0f;
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int64_t r = c0 + k, cc = r0 + tx;
    if (r < C && cc < C && r > cc) H[r * C + cc] = tile[tx][k];
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

}  // namespace

// Status words of individual launches: a ring in static device memory.  Each launch takes the next word and
// clears it on its stream before the kernel starts; the roles of that launch use it to tell one another that
// one of them gave up.  A word is reused after kStatusSlots further launches, by which time its launch has
// long ended in any realistic schedule (a stale non-zero word would only make a launch stop early and report
// a timeout, never compute wrongly in silence).
constexpr int kStatusSlots = 256;
__device__ int g_launch_status[kStatusSlots];

namespace {

// The slot of a launch: a word that is zero unless a role of some launch that used it gave up.  Slots start as
// zeros and are only ever set by give_up(); the host clears the whole ring when it reads a raised status
// (hessian_tc_status), so no launch has to be preceded by a memset.
int next_launch_status(int** status, cudaStream_t /*st*/) {
  static std::atomic<unsigned> counter{0};
  int* base = nullptr;
  NNCFB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_launch_status));
  *status = base + (counter.fetch_add(1) % kStatusSlots);
  return NNCFB_OK;
}

// instruction descriptor: fp32 accumulate, A/B format, both operands MN-major, N >> 3, M >> 4
uint32_t instr_desc(bool bf16) {
  const uint32_t fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | (static_cast<uint32_t>(kTileN >> 3) << 17) |
         (static_cast<uint32_t>(kTileM >> 4) << 24);
}

// 2-D map over a row-major 16-bit matrix [k_rows, extent] with `ld` elements between rows; boxes of
// 64 (extent) x 64 (k) with the 128-byte swizzle the operand descriptors expect.
int encode_map(CUtensorMap* map, const void* base, bool bf16, int64_t extent, int64_t k_rows, int64_t ld) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return NNCFB_E_UNSUPPORTED;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(extent), static_cast<cuuint64_t>(k_rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kBoxC, kBlockK};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d", static_cast<int>(cr));
    return NNCFB_E_CUDA;
  }
  return NNCFB_OK;
}

// 2-D map over a row-major fp32 matrix [rows, extent] with `ld` floats between rows; boxes of 32 x 32 floats (one
// 128-byte line per row) in the 128-byte swizzle the epilogue's staging buffers use.
int encode_map_f32(CUtensorMap* map, const float* base, int64_t extent, int64_t rows, int64_t ld) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return NNCFB_E_UNSUPPORTED;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(extent), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (fp32 output map) failed with code %d", static_cast<int>(cr));
    return NNCFB_E_CUDA;
  }
  return NNCFB_OK;
}

template <int kStages>
constexpr size_t tc_smem_bytes() { return static_cast<size_t>(kStages) * kStageBytes + sizeof(Control) + 1024; }

}  // namespace

static int hessian_tc_launch(float* H, int64_t C, const void* x, int dtype, int64_t tokens, float alpha, float beta,
                             cudaStream_t st, uint64_t wait_ns, int producer_short) {
  if (C % 64 != 0 || C < 256 || !aligned16(x) || !aligned16(H) || tokens <= 0 || tokens > 0x7fffffff ||
      C > 0x7fffffff / 2)
    return NNCFB_E_UNSUPPORTED;
  CUtensorMap map;
  const int rc = encode_map(&map, x, dtype == NNCFB_BF16, C, tokens, C);
  if (rc != NNCFB_OK) return rc;
  const int tiles_m = static_cast<int>((C + kTileM - 1) / kTileM);
  const int tiles_n = static_cast<int>((C + kTileN - 1) / kTileN);
  const int n_tiles = hessian_tile_count(tiles_m, tiles_n);
  constexpr size_t smem = tc_smem_bytes<kStagesHessian>();
  auto kernel = tc_tn_kernel<kStagesHessian, false>;
  NNCFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  int* status = nullptr;
  if (const int sr = next_launch_status(&status, st); sr != NNCFB_OK) return sr;
  kernel<<<std::min(n_tiles, sm_count()), 192, smem, st>>>(map, map, map, H, C, C, C, tokens, alpha, beta,
                                                            instr_desc(dtype == NNCFB_BF16), tiles_n, n_tiles, status,
                                                            wait_ns, producer_short, 0, 0);
  NNCFB_CUDA(cudaGetLastError());
  const dim3 mgrid(static_cast<unsigned>((C + 31) / 32), static_cast<unsigned>((C + 31) / 32));
  mirror_upper_tc_kernel<<<mgrid, 256, 0, st>>>(H, C);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

int hessian_tc_accumulate(float* H, int64_t C, const void* x, int dtype, int64_t tokens, float alpha, float beta,
                          void* /*workspace*/, size_t /*workspace_bytes*/, cudaStream_t st) {
  return hessian_tc_launch(H, C, x, dtype, tokens, alpha, beta, st, kWaitLimitNs, 0);
}

// ---- GPTQ trailing update on the tensor cores -------------------------------------------------------
// Three bf16 planes of one 128-row slab of the upper factor: planes[p][k][j] ~ Hinv[i1 + k][c0 + j].
__global__ void __launch_bounds__(256) gptq_split_slab_kernel(const float* __restrict__ hinv, int64_t cols, int i1,
                                                              int64_t c0, int64_t n, int64_t ld,
                                                              __nv_bfloat16* __restrict__ planes) {
  const int k = blockIdx.y;
  const int64_t j = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (j >= n) return;
  __nv_bfloat16 h, m, l;
  split_bf16x3(hinv[static_cast<int64_t>(i1 + k) * cols + c0 + j], h, m, l);
  planes[(0 * 128 + k) * ld + j] = h;
  planes[(1 * 128 + k) * ld + j] = m;
  planes[(2 * 128 + k) * ld + j] = l;
}

bool gptq_trailing_tc_available() { return encode_tiled_fn() != nullptr; }


// planes[p][k][j] = plane p of Hinv[i1 + k][c0 + j], j < n (bf16 [3 * 128, ld]).
int gptq_split_slab(const float* hinv, int64_t cols, int i1, int64_t c0, int64_t n, __nv_bfloat16* slab_planes,
                    int64_t slab_ld, cudaStream_t st) {
  const dim3 sgrid(static_cast<unsigned>((n + 255) / 256), 128);
  gptq_split_slab_kernel<<<sgrid, 256, 0, st>>>(hinv, cols, i1, c0, n, slab_ld, slab_planes);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

// W[:, c : c + n] -= Err @ Hinv[i1 : i1 + 128, c : c + n].
//   w_c        = W + c (row stride ld floats; 16-byte aligned, ld a multiple of 4)
//   err_planes : bf16 [3 * 128, err_ld], plane p row k column r = plane p of Err[r][k]  (written by the sweep kernel)
//   slab_c     : bf16 [3 * 128, slab_ld] planes of the slab, already offset to column c (16-byte aligned)
int gptq_trailing_tc(float* w_c, int64_t ld, int64_t rows, int64_t n, const __nv_bfloat16* err_planes, int64_t err_ld,
                     const __nv_bfloat16* slab_c, int64_t slab_ld, cudaStream_t st) {
  CUtensorMap amap, bmap, dmap;
  int rc = encode_map(&amap, err_planes, true, rows, 3 * 128, err_ld);
  if (rc != NNCFB_OK) return rc;
  rc = encode_map(&bmap, slab_c, true, n, 3 * 128, slab_ld);
  if (rc != NNCFB_OK) return rc;
  rc = encode_map_f32(&dmap, w_c, n, rows, ld);
  if (rc != NNCFB_OK) return rc;
  const int tiles_m = static_cast<int>((rows + kTileM - 1) / kTileM);
  const int tiles_n = static_cast<int>((n + kTileN - 1) / kTileN);
  constexpr size_t smem = tc_smem_bytes<kStagesTrailing>();
  auto kernel = tc_tn_kernel<kStagesTrailing, true>;
  NNCFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  int* status = nullptr;
  if (const int sr = next_launch_status(&status, st); sr != NNCFB_OK) return sr;
  // One CTA per tile here: this kernel shares the GPU with the next block's sweep (whose CTAs fill the shared
  // memory of the SMs they sit on), so a fixed set of persistent CTAs would leave tiles waiting behind it;
  // with a CTA per tile the hardware hands tiles to whichever SMs are free.
  kernel<<<tiles_m * tiles_n, 192, smem, st>>>(amap, bmap, dmap, w_c, ld, rows, n, 128, 1.0f, -1.0f, instr_desc(true), tiles_n,
                                               tiles_m * tiles_n, status, kWaitLimitNs, 0, 0, 0);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

// The rest updates of one GPTQ call: every block launches the same product on a column range that shrinks by 128,
// so the tensor maps are encoded once for the whole buffers (error planes and slab planes alternate between two
// buffers each) and a launch only passes its column offsets.  The range of a launch must end at the last column
// of W: a tile that reaches beyond the range is clipped by the map of W, not by the launch.
struct GptqTrailingPlan {
  CUtensorMap amap[2], bmap[2], dmap;
  float* w;
  int64_t ld, rows, cols;
  int* status_base;
};

int gptq_trailing_plan_create(GptqTrailingPlan** out, float* w, int64_t ld, int64_t rows, int64_t cols,
                              const __nv_bfloat16* const err_planes[2], int64_t err_ld,
                              const __nv_bfloat16* const slab_planes[2], int64_t slab_ld) {
  std::unique_ptr<GptqTrailingPlan> p(new GptqTrailingPlan());
  for (int i = 0; i < 2; ++i) {
    int rc = encode_map(&p->amap[i], err_planes[i], true, rows, 3 * 128, err_ld);
    if (rc != NNCFB_OK) return rc;
    rc = encode_map(&p->bmap[i], slab_planes[i], true, cols, 3 * 128, slab_ld);
    if (rc != NNCFB_OK) return rc;
  }
  const int rc = encode_map_f32(&p->dmap, w, cols, rows, ld);
  if (rc != NNCFB_OK) return rc;
  p->w = w;
  p->ld = ld;
  p->rows = rows;
  p->cols = cols;
  NNCFB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p->status_base), g_launch_status));
  auto kernel = tc_tn_kernel<kStagesTrailing, true>;
  NNCFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(tc_smem_bytes<kStagesTrailing>())));
  *out = p.release();
  return NNCFB_OK;
}

void gptq_trailing_plan_destroy(GptqTrailingPlan* p) { delete p; }

// W[:, c : cols] -= Err @ Hinv[i1 : i1 + 128, c : cols] with the operands of parity `which`; the slab planes hold
// column c at their column `slab_col`.
int gptq_trailing_plan_run(const GptqTrailingPlan* p, int which, int64_t c, int64_t slab_col, cudaStream_t st) {
  const int64_t n = p->cols - c;
  const int tiles_m = static_cast<int>((p->rows + kTileM - 1) / kTileM);
  const int tiles_n = static_cast<int>((n + kTileN - 1) / kTileN);
  static std::atomic<unsigned> counter{0};
  int* status = p->status_base + (counter.fetch_add(1) % kStatusSlots);
  auto kernel = tc_tn_kernel<kStagesTrailing, true>;
  kernel<<<tiles_m * tiles_n, 192, tc_smem_bytes<kStagesTrailing>(), st>>>(
      p->amap[which], p->bmap[which], p->dmap, p->w + c, p->ld, p->rows, n, 128, 1.0f, -1.0f, instr_desc(true), tiles_n,
      tiles_m * tiles_n, status, kWaitLimitNs, 0, static_cast<int>(slab_col), static_cast<int>(c));
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

// ---- fp32-faithful GEMM on the tensor cores -----------------------------------------------------------
// planes[p][k][j] = plane p of src[k][j] (src row-major [K, extent], `ld` floats between rows): B operands.
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ src, int64_t ld, int64_t K,
                                                         int64_t extent, int64_t plane_ld,
                                                         __nv_bfloat16* __restrict__ planes) {
  const int64_t k = blockIdx.y;
  const int64_t j = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (j >= extent) return;
  __nv_bfloat16 h, m, l;
  split_bf16x3(src[k * ld + j], h, m, l);
  planes[(0 * K + k) * plane_ld + j] = h;
  planes[(1 * K + k) * plane_ld + j] = m;
  planes[(2 * K + k) * plane_ld + j] = l;
}

// planes[p][k][i] = plane p of src[i][k] (src row-major [extent, K]): A operands, transposed through a 32 x 32 tile.
__global__ void __launch_bounds__(256) split_transposed_kernel(const float* __restrict__ src, int64_t ld, int64_t K,
                                                               int64_t extent, int64_t plane_ld,
                                                               __nv_bfloat16* __restrict__ planes) {
  __shared__ float tile[32][33];
  const int64_t i0 = static_cast<int64_t>(blockIdx.y) * 32, k0 = static_cast<int64_t>(blockIdx.x) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int64_t i = i0 + r, k = k0 + tx;
    tile[r][tx] = (i < extent && k < K) ? src[i * ld + k] : 0.0f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int64_t k = k0 + r, i = i0 + tx;
    if (k < K && i < extent) {
      __nv_bfloat16 h, m, l;
      split_bf16x3(tile[tx][r], h, m, l);
      planes[(0 * K + k) * plane_ld + i] = h;
      planes[(1 * K + k) * plane_ld + i] = m;
      planes[(2 * K + k) * plane_ld + i] = l;
    }
  }
}

namespace {
int64_t round8_i64(int64_t v) { return (v + 7) & ~static_cast<int64_t>(7); }
size_t planes_bytes_gemm(int64_t K, int64_t extent) {
  return (static_cast<size_t>(3) * K * round8_i64(extent) * 2 + 1023) & ~static_cast<size_t>(1023);
}
}  // namespace

size_t gemm_f32_workspace(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return planes_bytes_gemm(K, M) + planes_bytes_gemm(K, N);
}

// C[M, N] (row stride ldc) = C * (accumulate ? 1 : 0) + alpha * A[M, K] @ B, with B given as [K, N] (row stride ldb)
// or, with transpose_b, as [N, K] (C = A B^T)
int gemm_f32(const float* A, int64_t lda, const float* B, int64_t ldb, bool transpose_b, float* C, int64_t ldc, int64_t M,
             int64_t N, int64_t K, float alpha, bool accumulate, void* workspace, size_t workspace_bytes,
             cudaStream_t st) {
  if (K % kBlockK != 0 || ldc % 4 != 0 || !aligned16(C) || !aligned16(workspace) || M > 0x7fffffff || N > 0x7fffffff ||
      K > 0x7fffffff / 3 || encode_tiled_fn() == nullptr)
    return NNCFB_E_UNSUPPORTED;
  if (workspace_bytes < gemm_f32_workspace(M, N, K)) {
    set_error("nncfb_gemm_f32: workspace of %zu bytes is smaller than nncfb_gemm_f32_workspace_bytes() = %zu",
              workspace_bytes, gemm_f32_workspace(M, N, K));
    return NNCFB_E_BAD_ARG;
  }
  __nv_bfloat16* a_planes = static_cast<__nv_bfloat16*>(workspace);
  __nv_bfloat16* b_planes = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(workspace) + planes_bytes_gemm(K, M));
  const int64_t a_ld = round8_i64(M), b_ld = round8_i64(N);
  const dim3 ga(static_cast<unsigned>((K + 31) / 32), static_cast<unsigned>((M + 31) / 32));
  split_transposed_kernel<<<ga, 256, 0, st>>>(A, lda, K, M, a_ld, a_planes);
  if (transpose_b) {
    const dim3 gb(static_cast<unsigned>((K + 31) / 32), static_cast<unsigned>((N + 31) / 32));
    split_transposed_kernel<<<gb, 256, 0, st>>>(B, ldb, K, N, b_ld, b_planes);
  } else {
    const dim3 gb(static_cast<unsigned>((N + 255) / 256), static_cast<unsigned>(K));
    split_rows_kernel<<<gb, 256, 0, st>>>(B, ldb, K, N, b_ld, b_planes);
  }
  NNCFB_CUDA(cudaGetLastError());
  if (!accumulate) NNCFB_CUDA(cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(N) * 4, M, st));
  CUtensorMap amap, bmap, dmap;
  int rc = encode_map(&amap, a_planes, true, M, 3 * K, a_ld);
  if (rc != NNCFB_OK) return rc;
  rc = encode_map(&bmap, b_planes, true, N, 3 * K, b_ld);
  if (rc != NNCFB_OK) return rc;
  rc = encode_map_f32(&dmap, C, N, M, ldc);
  if (rc != NNCFB_OK) return rc;
  const int tiles_m = static_cast<int>((M + kTileM - 1) / kTileM);
  const int tiles_n = static_cast<int>((N + kTileN - 1) / kTileN);
  constexpr size_t smem = tc_smem_bytes<kStagesTrailing>();
  auto kernel = tc_tn_kernel<kStagesTrailing, true>;
  NNCFB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  int* status = nullptr;
  if (const int sr = next_launch_status(&status, st); sr != NNCFB_OK) return sr;
  kernel<<<tiles_m * tiles_n, 192, smem, st>>>(amap, bmap, dmap, C, ldc, M, N, K, 1.0f, alpha, instr_desc(true), tiles_n,
                                               tiles_m * tiles_n, status, kWaitLimitNs, 0, 0, 0);
  NNCFB_CUDA(cudaGetLastError());
  return NNCFB_OK;
}

// Reads the device's sticky flag after everything enqueued on `st` has run, and clears it when it was set.
int hessian_tc_status(cudaStream_t st) {
  int* status = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_hessian_status) != cudaSuccess) return -1;
  int h = 0;
  if (cudaMemcpyAsync(&h, status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
  if (h != 0) {
    int* ring = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ring), g_launch_status) != cudaSuccess) return -1;
    if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) return -1;
    if (cudaMemsetAsync(ring, 0, sizeof(int) * kStatusSlots, st) != cudaSuccess) return -1;  // the launches' own words
    if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
  }
  return h;
}

}  // namespace nncfb

extern "C" int nncfb_hessian_status(void* stream) {
  const int s = nncfb::hessian_tc_status(static_cast<cudaStream_t>(stream));
  if (s < 0) {
    nncfb::set_error("nncfb_hessian_status: could not read the status flag");
    return NNCFB_E_CUDA;
  }
  if (s != 0) {
    nncfb::set_error("a tensor-core kernel gave up a bounded wait (role %d: 1 = producer, 2 = MMA, 3 = epilogue, "
                     "4 = producer drain, 5 = MMA waiting for the epilogue)", s);
    return NNCFB_E_TIMEOUT;
  }
  return NNCFB_OK;
}

extern "C" size_t nncfb_gemm_f32_workspace_bytes(int64_t m, int64_t n, int64_t k) { return nncfb::gemm_f32_workspace(m, n, k); }

extern "C" int nncfb_gemm_f32(const float* a, int64_t lda, const float* b, int64_t ldb, int32_t transpose_b, float* c,
                              int64_t ldc, int64_t m, int64_t n, int64_t k, float alpha, int32_t accumulate,
                              void* workspace, size_t workspace_bytes, void* stream) {
  NNCFB_CHECK_ARG(a && b && c && workspace, NNCFB_E_BAD_ARG, "nncfb_gemm_f32: null pointer");
  NNCFB_CHECK_ARG(m > 0 && n > 0 && k > 0 && lda >= k && ldb >= (transpose_b ? k : n) && ldc >= n, NNCFB_E_BAD_ARG,
                  "nncfb_gemm_f32: bad shape");
  const int rc = nncfb::gemm_f32(a, lda, b, ldb, transpose_b != 0, c, ldc, m, n, k, alpha, accumulate != 0, workspace,
                                 workspace_bytes, static_cast<cudaStream_t>(stream));
  if (rc == NNCFB_E_UNSUPPORTED)
    nncfb::set_error("nncfb_gemm_f32: needs k %% 64 == 0, ldc %% 4 == 0, 16-byte aligned c and workspace, and a driver "
                     "with tensor-map support");
  return rc;
}

// Self test of the bounded waits: the Hessian kernel with a 1 ms limit per wait and a producer that leaves out the
// last pipeline stage of every tile.  The MMA role's wait for that stage runs out, it records its code, the
// other roles stop, tensor memory is freed and the kernel returns; H is left partly written.  Nothing traps and
// no wait is unbounded.  The caller then reads NNCFB_E_TIMEOUT from nncfb_hessian_status.
extern "C" int nncfb_selftest_bounded_wait(float* hessian, int64_t channels, const void* x_bf16, int64_t tokens,
                                           void* stream) {
  NNCFB_CHECK_ARG(hessian && x_bf16, NNCFB_E_BAD_ARG, "nncfb_selftest_bounded_wait: null pointer");
  NNCFB_CHECK_ARG(channels >= 256 && channels <= 1024 && channels % 64 == 0 && tokens >= 64 && tokens <= 4096,
                  NNCFB_E_BAD_ARG, "nncfb_selftest_bounded_wait: 256 <= channels <= 1024 (multiple of 64), 64 <= tokens <= 4096");
  const int rc = nncfb::hessian_tc_launch(hessian, channels, x_bf16, NNCFB_BF16, tokens, 0.0f, 1.0f,
                                          static_cast<cudaStream_t>(stream), 1000000ull, 1);
  if (rc == NNCFB_E_UNSUPPORTED) nncfb::set_error("nncfb_selftest_bounded_wait: the tensor-core path is unavailable");
  return rc;
}
