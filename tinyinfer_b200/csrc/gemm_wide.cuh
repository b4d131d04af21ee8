// Many-row GEMM (prefill) on the sm_100a tensor cores:  out[M,N] = A[M,K] . W[K,N] + bias  (+ GELU, + residual, K/V placement)
//
// For passes of hundreds to thousands of rows the decode-shaped kernel (gemm_tc.cuh) spends most of a CTA's life in its
// prologue and epilogue: K is short (768 .. 4096), a 64-row tile is 12 .. 64 stages of work wrapped in fixed costs, and
// every weight is dequantised again for every 64-row tile.  This kernel is built for that regime:
//   * the weights are read from an "operand image": the fp16 values the INT8 matrix dequantises to (or the fp16 weights
//     of an fp16 artifact), stored once at load time in exactly the shared-memory layout tcgen05.mma wants
//     ([slab of 128 channels][64-row stage][16 KB of MN-major core matrices]).  A stage is one contiguous 16 KB block:
//     warp 0 fetches it with a single bulk copy, no thread ever touches a weight;
//   * the rows of A arrive the same way: one TMA box of 128 rows x 64 columns per stage, written with the 128-byte
//     swizzle that tcgen05.mma reads as a K-major operand (no thread copies a row either);
//   * tiles of 128 channels x 128 rows, six operand stages in flight, CTAs persistent over the tiles of the problem, so
//     the epilogue of one tile overlaps the main loop of the next;
//   * the K ranges of gemm()'s K split still get separate TMEM accumulators (three, in rotation) and are added in range
//     order -- by sixteen dedicated warps that keep the running sums in registers while the tensor cores work on the next
//     range -- so a row's result carries the same bits as in the decode-shaped kernel, whatever the row count.
// Warp roles (576 threads): 0 producer (bulk copy of the weights, TMA of the rows), 1 MMA issuer, 2-17 fold the K ranges
// and finish the tile (bias, GELU, residual, K/V placement, store) -- the finishing of a tile is cut into pieces of
// eight rows that run between the folds of the next tile, so it never holds the tensor cores up.  Every wait is bounded.
#pragma once
#include <cuda.h>

#include "attention.cuh"
#include "common.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"

namespace tib {

constexpr int kWideRows = 128;                     // rows of A per tile = MMA N
constexpr int kWideStages = 6;                     // operand stages (weights 16 KB + rows 16 KB each): 192 KB in flight per SM
constexpr int kWideFolders = 512;                  // warps 2..17: four per TMEM lane quarter, each with a quarter of the tile's rows
constexpr int kWideGroups = kWideFolders / 128;    // groups of four warps that share rows of the tile
constexpr int kWideOwn = kWideRows / kWideGroups;  // rows of a tile one folder thread owns (for its channel)
constexpr int kWidePieces = kWideOwn / 8;          // pieces of eight rows a finished tile leaves in
constexpr int kWideBuffers = 3;                    // TMEM accumulators of one K range each: the MMAs run up to two ranges ahead of the folders
constexpr int kWideThreads = 64 + kWideFolders;
constexpr int kWideImageStage = 128 * kTcStageK * 2;        // bytes of one weight stage in the operand image

struct WideSmem {
  static constexpr int kOpAOff = 0;
  static constexpr int kOpBBytes = kWideRows * kTcStageK * 2;
  static constexpr int kOpBOff = kOpAOff + kWideStages * kWideImageStage;
  static constexpr int kBarOff = kOpBOff + kWideStages * kOpBBytes;
  static constexpr int kBytes = kBarOff + 256 + 1024;     // the swizzled operand stages sit on 1024-byte boundaries
};

// Byte offset of element (k, c) of a [K,N] matrix inside its operand image (stages_per_slab = ceil(K / 64)).
__host__ __device__ __forceinline__ size_t wide_image_offset(int k, int c, int stages_per_slab) {
  const int slab = c >> 7, stage = k >> 6, kg = (k & 63) >> 3, ng = (c & 127) >> 3;
  return (size_t(slab) * stages_per_slab + stage) * kWideImageStage + size_t(kg * 16 + ng) * 128 + (k & 7) * 16 + (c & 7) * 2;
}

// Image of an INT8 matrix (its dequantised values) or of an fp16 matrix; channels >= n and rows >= k are zero.
// One thread per 16 bytes of the image (8 channels of one k row).
__global__ void wide_image_kernel(const int8_t* q, const __half* w16, long long ld, const float* scales, uint8_t* image, int k, int n,
                                  int stages_per_slab, long long chunks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= chunks) return;
  // chunk i of the image: (slab, stage, kg, ng, k8)
  const int k8 = int(i & 7), ng = int((i >> 3) & 15), kg = int((i >> 7) & 7);
  const long long block = i >> 10;
  const int stage = int(block % stages_per_slab), slab = int(block / stages_per_slab);
  const int row = stage * 64 + kg * 8 + k8, col0 = slab * 128 + ng * 8;
  __half h[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int col = col0 + e;
    h[e] = f2h(0.f);
    if (row < k && col < n) h[e] = q ? f2h(float(q[(long long)row * ld + col]) * scales[col]) : w16[(long long)row * ld + col];
  }
  *reinterpret_cast<uint4*>(image + i * 16) = *reinterpret_cast<const uint4*>(h);
}

// Shared-memory descriptor of a K-major operand written by TMA with the 128-byte swizzle: rows of 128 bytes, groups of
// eight rows 1024 bytes apart; a 16-element K step moves the start address by 32 bytes inside the swizzled row.
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t smem_addr) {
  return uint64_t((smem_addr >> 4) & 0x3fffu) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}

// grid = min(tiles, SMs) persistent CTAs, block = kWideThreads.  p.w = operand image; p.k_chunk = rows per K range;
// a_map = [M, K] fp16 rows of A, box 64 x 128, 128-byte swizzle.
__global__ void __launch_bounds__(kWideThreads, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap a_map, const GemvArgs p) {
  using L = WideSmem;
  extern __shared__ uint8_t wide_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(wide_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* op_a = smem + L::kOpAOff;
  uint8_t* op_b = smem + L::kOpBOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t *op_full = bars, *op_empty = op_full + kWideStages, *range_done = op_empty + kWideStages, *range_free = range_done + kWideBuffers;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(range_free + kWideBuffers);
  static_assert((2 * kWideStages + 2 * kWideBuffers) * 8 + 8 <= 256, "barrier block");
  __shared__ int s_failed;
  __shared__ __align__(16) __half s_piece[2][kWideGroups][8 * 128];   // a piece of a finished tile on its way out: [parity][row group][row][channel]
  __shared__ long long s_row_base[3][kWideRows];               // K/V pool offset of each row of a tile (QKV projection); three tiles in rotation

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slabs = (p.n + 127) / 128, row_tiles = (p.m + kWideRows - 1) / kWideRows, tiles = slabs * row_tiles;
  const int stages = (p.k + kTcStageK - 1) / kTcStageK;        // per tile
  const int chunk_stages = p.k_chunk / kTcStageK;
  const int ranges = (stages + chunk_stages - 1) / chunk_stages;

  pdl_launch_dependents();
  if (tid == 0) {
    s_failed = 0;
    for (int s = 0; s < kWideStages; ++s) { mbar_init(&op_full[s], 2); mbar_init(&op_empty[s], 1); }   // weights and rows are announced separately
    for (int b = 0; b < kWideBuffers; ++b) { mbar_init(&range_done[b], 1); mbar_init(&range_free[b], kWideFolders / 32); }
    mbar_fence_init();
  }
  constexpr uint32_t kTmemCols = 512;                           // three accumulators of 128 columns; allocations are powers of two
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  volatile int* failed = &s_failed;
  auto wait = [&](uint64_t* bar, uint32_t parity, unsigned int code) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
      if (mbar_try(bar, parity)) return true;
      if ((spin & 1023u) == 1023u && *failed) return false;
    }
    report(code);
    *failed = 1;
    return false;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer: per stage one 16 KB bulk copy (weights) and
    // one TMA box (rows of A).  The weights of the first stages do not depend on the previous kernel and go out ahead of
    // the dependency wait; the two halves of a stage are announced to its barrier separately (two arrivals).
    if (lane == 0 && int(blockIdx.x) < tiles) {
      const uint8_t* image = static_cast<const uint8_t*>(p.w);
      const int my_tiles = (tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
      const int total = my_tiles * stages, lead = min(total, kWideStages);
      auto weights = [&](int idx) {
        const int slot = idx % kWideStages, tile = int(blockIdx.x) + (idx / stages) * int(gridDim.x), i = idx % stages;
        mbar_expect_tx(&op_full[slot], kWideImageStage);
        bulk_load(op_a + slot * kWideImageStage, image + (size_t(tile % slabs) * stages + i) * kWideImageStage, kWideImageStage, &op_full[slot]);
      };
      auto rows = [&](int idx) {
        const int slot = idx % kWideStages, tile = int(blockIdx.x) + (idx / stages) * int(gridDim.x), i = idx % stages;
        mbar_expect_tx(&op_full[slot], L::kOpBBytes);
        tma_load_2d(op_b + slot * L::kOpBBytes, &a_map, i * kTcStageK, (tile / slabs) * kWideRows, &op_full[slot]);
      };
      for (int idx = 0; idx < lead; ++idx) weights(idx);
      pdl_wait();                                              // A comes from the previous kernel
      for (int idx = 0; idx < lead; ++idx) rows(idx);
      bool ok = true;
      for (int idx = lead; idx < total && ok; ++idx) {
        ok = wait(&op_empty[idx % kWideStages], (uint32_t(idx / kWideStages) & 1u) ^ 1u, kStatusPipeTimeout);
        if (!ok) break;
        weights(idx);
        rows(idx);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 15) | (uint32_t(kWideRows >> 3) << 17) | (uint32_t(128 >> 4) << 24);
      int it = 0, g = 0;                                       // running stage / range numbers over all tiles of this CTA
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        for (int r = 0; r < ranges && ok; ++r, ++g) {
          const int buffer = g % kWideBuffers;
          if (g >= kWideBuffers) ok = wait(&range_free[buffer], uint32_t(g / kWideBuffers - 1) & 1u, kStatusPipeTimeout);   // the folders have read it
          if (!ok) break;
          tc_fence_after();
          const int first = r * chunk_stages, last = min(stages, first + chunk_stages);
          for (int i = first; i < last && ok; ++i, ++it) {
            const int slot = it % kWideStages;
            ok = wait(&op_full[slot], uint32_t(it / kWideStages) & 1u, kStatusPipeTimeout);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_addr = smem_u32(op_a + slot * kWideImageStage), b_addr = smem_u32(op_b + slot * L::kOpBBytes);
#pragma unroll
            for (int kk = 0; kk < kTcStageK / 16; ++kk) {
              const uint64_t da = tc_desc(a_addr + kk * 2 * 2048, 2048u, 128u);
              const uint64_t db = tc_desc_sw128(b_addr + kk * 32);
              tc_mma_f16(tmem_base + uint32_t(buffer * kWideRows), da, db, idesc, (i > first || kk > 0) ? 1u : 0u);
            }
            tc_commit(&op_empty[slot]);
          }
          if (ok) tc_commit(&range_done[buffer]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ fold the K ranges, finish the tile
    const int f = warp - 2;                                    // 0..15
    const int quarter = warp & 3, group = f >> 2;               // TMEM lanes 32 * quarter .., columns kWideOwn * group ..
    const uint32_t taddr = tmem_base + (uint32_t(32 * quarter) << 16) + uint32_t(kWideOwn * group);
    const int ft = tid - 64;                                   // 0..255
    int g = 0, tile_no = 0;
    bool ok = true;
    // The tile whose sums are complete and waiting to be finished (eight pieces of eight rows per thread).
    __half2 done[kWideOwn / 2];                                // already rounded to fp16 after the bias: rows 2i, 2i + 1
    bool have_done = false;
    int done_m0 = 0, done_n0 = 0, done_col = 0;
    const long long* done_base = nullptr;
    // Piece `piece` (rows 8 * piece .. + 7 of this thread's kWideOwn) of the finished tile: the rounding points of gemv_store
    // (bias -> fp16 -> GELU -> fp16 -> + residual -> fp16, or K/V to their cache pages).  A thread owns one channel (its
    // TMEM lane) but the output rows run along the channels, so the four warps that share a group of rows pass the
    // piece through shared memory ([8 rows][128 channels]) and every thread writes 16 bytes of one row: a warp stores two
    // runs of 256 bytes instead of thirty-two 2-byte values.  All folder warps execute the same sequence of named
    // barriers whatever happened to their waits.
    const int tg = ((f & 3) << 5) | lane;                      // 0..127 within the group
    const int out_row = tg >> 4, out_c8 = (tg & 15) * 8;       // this thread's 16 bytes of a piece
    const bool wide_stores = (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
                             (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0 && (p.kv_hidden & 7) == 0 &&
                             (reinterpret_cast<uintptr_t>(p.k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.v_pool) & 15) == 0;
    auto residual_of = [&](int piece) {
      uint4 res = make_uint4(0u, 0u, 0u, 0u);
      const int row = done_m0 + kWideOwn * group + piece * 8 + out_row, c0 = done_n0 + out_c8;
      if (have_done && wide_stores && p.residual && row < p.m && c0 + 8 <= p.n && !(p.k_pool && c0 >= p.kv_hidden))
        res = *reinterpret_cast<const uint4*>(p.residual + size_t(row) * p.ldo + c0);
      return res;
    };
    auto finish_piece = [&](int piece, uint4 res) {
      if (!have_done) return;                                   // uniform over all folder warps
      __half2 mine[4] = {};
#pragma unroll
      for (int c = 0; c < kWidePieces; ++c)                     // unrolled: done[] is only ever indexed by constants
        if (c == piece) {
#pragma unroll
          for (int e = 0; e < 4; ++e) mine[e] = done[c * 4 + e];
        }
      __half* stage = s_piece[piece & 1][group];
      const bool plain = !(p.k_pool && done_col >= p.kv_hidden);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        __half h = (e & 1) ? __high2half(mine[e >> 1]) : __low2half(mine[e >> 1]);
        if (p.gelu && plain) h = f2h(gelu_tanh(h2f(h)));
        stage[e * 128 + 32 * quarter + lane] = h;
      }
      asm volatile("bar.sync %0, 128;" ::"r"(5 + group) : "memory");
      const int j = piece * 8 + out_row, row = done_m0 + kWideOwn * group + j, c0 = done_n0 + out_c8;
      if (!ok || row >= p.m || c0 >= p.n) return;
      if (wide_stores && c0 + 8 <= p.n) {
        uint4 packed = *reinterpret_cast<const uint4*>(stage + out_row * 128 + out_c8);
        __half* h = reinterpret_cast<__half*>(&packed);
        if (p.k_pool && c0 >= p.kv_hidden) {
          const int cc = c0 - p.kv_hidden, which = cc >= p.kv_hidden, e = which ? cc - p.kv_hidden : cc;
          *reinterpret_cast<uint4*>((which ? p.v_pool : p.k_pool) + (e >> 6) * 2048 + (e & 63) + done_base[kWideOwn * group + j]) = packed;
        } else {
          if (p.residual) {
            const __half* r = reinterpret_cast<const __half*>(&res);
#pragma unroll
            for (int e = 0; e < 8; ++e) h[e] = f2h(h2f(r[e]) + h2f(h[e]));
          }
          *reinterpret_cast<uint4*>(static_cast<__half*>(p.out) + size_t(row) * p.ldo + c0) = packed;
        }
      } else {
#pragma unroll 1
        for (int e = 0; e < 8 && c0 + e < p.n; ++e) {           // ragged edge or unaligned buffers: value by value
          const int c = c0 + e;
          if (p.k_pool && c >= p.kv_hidden) {
            const int cc = c - p.kv_hidden, which = cc >= p.kv_hidden, x = which ? cc - p.kv_hidden : cc;
            ((which ? p.v_pool : p.k_pool) + (x >> 6) * 2048 + (x & 63))[done_base[kWideOwn * group + j]] = stage[out_row * 128 + out_c8 + e];
          } else {
            __half v = stage[out_row * 128 + out_c8 + e];
            if (p.residual) v = f2h(h2f(p.residual[size_t(row) * p.ldo + c]) + h2f(v));
            static_cast<__half*>(p.out)[size_t(row) * p.ldo + c] = v;
          }
        }
      }
    };
    pdl_wait();                                                // the residual comes from an earlier kernel
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++tile_no) {
      const int slab = tile % slabs, m0 = (tile / slabs) * kWideRows, n0 = slab * 128;
      long long* row_base = s_row_base[tile_no % 3];
      if (p.k_pool) {
        for (int i = ft; i < kWideRows; i += kWideFolders) row_base[i] = m0 + i < p.m ? kv_row_base(p, m0 + i) : 0;
        asm volatile("bar.sync 4, %0;" ::"n"(kWideFolders) : "memory");
      }
      const int col = n0 + 32 * quarter + lane;
      const float bias = p.bias && col < p.n ? h2f(p.bias[col]) : 0.f;
      static_assert(kWideOwn == 32, "one tcgen05.ld of 32 columns per range and folder warp");
      float sum[kWideOwn];
#pragma unroll
      for (int j = 0; j < kWideOwn; ++j) sum[j] = 0.f;
      for (int r = 0; r < ranges; ++r, ++g) {
        const int buffer = g % kWideBuffers;
        uint4 res = make_uint4(0u, 0u, 0u, 0u);
        if (r < kWidePieces) res = residual_of(r);            // requested before the wait: in flight while the range completes
        if (ok) ok = wait(&range_done[buffer], uint32_t(g / kWideBuffers) & 1u, kStatusMmaTimeout);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (ok) {
          float part[32];
          tmem_load32(taddr + uint32_t(buffer * kWideRows), part);
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[j] += part[j];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&range_free[buffer]);
        if (r < kWidePieces) finish_piece(r, res);            // one piece of the previous tile between two folds
      }
      for (int piece = ranges; piece < kWidePieces; ++piece) finish_piece(piece, residual_of(piece));   // fewer ranges than pieces: the rest of the previous tile
#pragma unroll
      for (int j = 0; j < kWideOwn / 2; ++j) done[j] = __halves2half2(f2h(sum[2 * j] + bias), f2h(sum[2 * j + 1] + bias));
      have_done = true; done_m0 = m0; done_n0 = n0; done_col = col; done_base = row_base;
    }
    for (int piece = 0; piece < kWidePieces; ++piece) finish_piece(piece, residual_of(piece));   // the last tile of this CTA
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

}  // namespace tib
