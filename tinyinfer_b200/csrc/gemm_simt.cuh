// Skinny weight-streaming GEMM ("GEMV" at decode batch sizes) for sm_100a.
//
//   out[M,N] = A[M,K] (fp16) . W[K,N] + bias[N],  W = int8 with per-column fp32 scales
//   (dequantised as fp16_rn(float(q)*scale), the reference's rounding, gemm.cu:21-24) or fp16.
//
// HBM-bound: every weight byte is read once per M-tile.  A CTA owns a 128-byte-wide column
// slab of W and a contiguous K range; a thread-block cluster of up to 8 CTAs splits K for one
// slab and reduces its partial sums through distributed shared memory in rank order, so the
// result does not depend on timing.  Weight tiles (64 rows x 128 bytes) are staged by TMA
// (cp.async.bulk.tensor.2d, zero fill out of range) into a ring of shared-memory stages guarded
// by full/empty mbarriers; a thread reads 16 bytes of one row (ld.shared.v4), dequantises
// them once and issues mixed-precision FMAs (fp16 x fp16 + fp32) against up to 4 rows of A
// held in shared memory.  Rows are reduced with warp shuffles (4 row-lanes per warp) and a
// fixed-order pass over the 8 warps.
//
// Epilogue (fused): + bias -> fp16 round -> optional tanh-GELU (+ fp16 round) -> optional
// residual add (+ fp16 round), or fp32 store for the vocabulary projection.  These are the
// rounding points of the reference's separate kernels (gemm.cu:76-78, elementwise.cu:30-31,
// llm/src/runtime.cu:31-33).
//
// When W cannot be described by a tensor map (row pitch or base not a multiple of 16 bytes,
// e.g. N = 50257) the same compute runs on tiles filled by guarded byte loads.
#pragma once
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"

namespace tib {
namespace cg = cooperative_groups;

constexpr int kGemvThreads = 256;
constexpr int kGemvRowBytes = 128;        // bytes of one weight row per CTA slab
constexpr int kGemvStageRows = 64;
constexpr int kGemvStages = 4;
constexpr int kGemvMaxMT = 4;             // rows of A per pass
constexpr int kGemvAChunk = 4096;         // K values of A resident in shared memory at a time

struct GemvArgs {
  const __half* a;            // [M,K], row pitch lda
  const void* w;              // int8 or fp16 [K,N], row pitch ldw elements
  const float* scales;        // fp32[N] for int8 weights
  const __half* bias;         // fp16[N] or null
  void* out;                  // fp16 or fp32 [M,N], row pitch ldo
  const __half* residual;     // fp16 [M,N] (pitch ldo) or null; fp16 output only
  int lda, ldo;
  long long ldw;
  int m, n, k;
  int k_chunk;                // K rows per CTA, multiple of kGemvStageRows
  int early_trigger;          // release the dependent launch at once: the next kernel has work that does not need this one's output
  int serial_chunks;          // tensor-core kernel, one CTA over the whole K: the K ranges of a `serial_chunks`-way split get one
                              // accumulator each and are added in range order (same sums as the split launch); 0 = off
  int w_slab_rows;            // tensor-core kernel: 0 = weights are [K][ldw]; else slab-major [N/128][w_slab_rows][128]
  int out_fp32, gelu;
  // K/V placement (QKV projection of the model runtime; k_pool null elsewhere): columns at or past
  // kv_hidden are the K then V thirds and go straight to their position in the paged pool
  // ([page][layer][head][32][64], see attention.cuh) instead of `out`.
  __half* k_pool; __half* v_pool;
  const int32_t* kv_table; const int32_t* kv_slots; const int32_t* kv_row_req; const int32_t* kv_row_pos;
  int kv_table_pitch, kv_layers, kv_layer, kv_heads, kv_hidden;
  // LayerNorm prologue (tensor-core kernel, at most 32 rows, K = row width <= 768): `a` holds the rows before
  // normalisation; the kernel computes each row's statistics and normalises while staging the operand.
  const __half* ln_gamma; const __half* ln_beta; float ln_eps;
  // Greedy argmax as an epilogue (tensor-core kernel, fp32 output without a K split, i.e. the vocabulary projection):
  // every CTA merges the best (value, lowest index) of its 128 columns into argmax_best[row] (argmax_pack words, zero
  // between steps) with atomicMax; skip_store: the logits themselves are not wanted.
  unsigned long long* argmax_best; int skip_store;
};

// Offset (in halves) of head 0, element 0 of row `row`'s position inside the K / V pool.
__device__ __forceinline__ long long kv_row_base(const GemvArgs& p, int row) {
  const int pos = p.kv_row_pos[row];
  const int page = p.kv_table[size_t(p.kv_slots[p.kv_row_req[row]]) * p.kv_table_pitch + (pos >> 5)];
  return ((long long)(page) * p.kv_layers + p.kv_layer) * p.kv_heads * 2048 + (pos & 31) * 64;
}

template <typename WT> struct WeightTraits;
template <> struct WeightTraits<int8_t> { static constexpr int kCols = 16; };   // columns per 16-byte read
template <> struct WeightTraits<__half> { static constexpr int kCols = 8; };

struct GemvSmem {
  static constexpr int kStageBytes = kGemvStageRows * kGemvRowBytes;
  static constexpr int kStagesOff = 0;
  static constexpr int kAOff = kStagesOff + kGemvStages * kStageBytes;                       // fp16 [MT][kGemvAChunk]
  static constexpr int kRedOff = kAOff + kGemvMaxMT * kGemvAChunk * 2;                       // fp32 [8 warps][MT][128]
  static constexpr int kPartOff = kRedOff + 8 * kGemvMaxMT * 128 * 4;                        // fp32 [MT][128]
  static constexpr int kBarOff = kPartOff + kGemvMaxMT * 128 * 4;
  static constexpr int kBytes = kBarOff + 2 * kGemvStages * 8 + 64;
};

template <typename WT, int MT>
__device__ __forceinline__ void gemv_consume_stage(const uint8_t* stage, const __half* a_smem, int a_pitch, int kk0,
                                                   const float* s, float (&acc)[MT][WeightTraits<WT>::kCols]) {
  constexpr int C = WeightTraits<WT>::kCols;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int it = 0; it < kGemvStageRows / 32; ++it) {
    const int r = it * 32 + warp * 4 + (lane >> 3);
    const uint4 raw = *reinterpret_cast<const uint4*>(stage + r * kGemvRowBytes + (lane & 7) * 16);
    __half2 w2[C / 2];
    if constexpr (sizeof(WT) == 1) {
      const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) dequant4(words[j], s[4 * j], s[4 * j + 1], s[4 * j + 2], s[4 * j + 3], w2[2 * j], w2[2 * j + 1]);
    } else {
      const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) w2[j] = *reinterpret_cast<const __half2*>(&words[j]);
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const __half av = a_smem[m * a_pitch + kk0 + r];
#pragma unroll
      for (int j = 0; j < C / 2; ++j) {
        acc[m][2 * j] = fma_f16(acc[m][2 * j], av, __low2half(w2[j]));
        acc[m][2 * j + 1] = fma_f16(acc[m][2 * j + 1], av, __high2half(w2[j]));
      }
    }
  }
}

// row_base: kv_row_base(p, row) when the caller has it at hand, else -1 (looked up here).
// fetched: the element's bias and residual were read ahead of time (raw halves) and are passed in.
__device__ __forceinline__ void gemv_store(const GemvArgs& p, int row, int col, float acc, long long row_base = -1,
                                           bool fetched = false, __half bias = __half(), __half residual = __half()) {
  const float v = acc + (fetched ? h2f(bias) : (p.bias ? h2f(p.bias[col]) : 0.f));
  if (p.k_pool && col >= p.kv_hidden) {
    const int c = col - p.kv_hidden, which = c >= p.kv_hidden, e = which ? c - p.kv_hidden : c;
    if (row_base < 0) row_base = kv_row_base(p, row);
    (which ? p.v_pool : p.k_pool)[row_base + (e >> 6) * 2048 + (e & 63)] = f2h(v);
    return;
  }
  if (p.out_fp32) { static_cast<float*>(p.out)[size_t(row) * p.ldo + col] = v; return; }
  __half h = f2h(v);
  if (p.gelu) h = f2h(gelu_tanh(h2f(h)));
  if (p.residual) h = f2h(h2f(fetched ? residual : p.residual[size_t(row) * p.ldo + col]) + h2f(h));
  static_cast<__half*>(p.out)[size_t(row) * p.ldo + col] = h;
}

// grid = (column slabs, k splits [cluster dimension], M tiles); block = 256.
template <typename WT, int MT, bool TMA>
__global__ void __launch_bounds__(kGemvThreads, 2)
gemv_kernel(const __grid_constant__ CUtensorMap w_map, const GemvArgs p) {
  constexpr int C = WeightTraits<WT>::kCols;
  constexpr int BN = 8 * C;                                   // columns per slab: 128 (int8) or 64 (fp16)
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* stages = smem + GemvSmem::kStagesOff;
  __half* a_smem = reinterpret_cast<__half*>(smem + GemvSmem::kAOff);
  float* red = reinterpret_cast<float*>(smem + GemvSmem::kRedOff);
  float* part = reinterpret_cast<float*>(smem + GemvSmem::kPartOff);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + GemvSmem::kBarOff);
  uint64_t* empty = full + kGemvStages;

  cg::cluster_group cluster = cg::this_cluster();
  const int splits = int(gridDim.y), rank = int(blockIdx.y);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.z * MT;
  const int k_begin = rank * p.k_chunk, k_end = min(p.k, k_begin + p.k_chunk);
  const int n_stages_total = k_end > k_begin ? (k_end - k_begin + kGemvStageRows - 1) / kGemvStageRows : 0;

  if (TMA && tid == 0) {
    tma_prefetch_desc(&w_map);
    for (int s = 0; s < kGemvStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kGemvThreads / 32); }
    mbar_fence_init();
  }
  __syncthreads();
  // Weights do not depend on the producer of A: start streaming before anything else.
  int issued = 0;
  if (TMA && tid == 0) {
    for (; issued < min(kGemvStages, n_stages_total); ++issued) {
      mbar_expect_tx(&full[issued], GemvSmem::kStageBytes);
      tma_load_2d(stages + issued * GemvSmem::kStageBytes, &w_map, n0, k_begin + issued * kGemvStageRows, &full[issued]);
    }
  }

  float s[C];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    const int col = n0 + (lane & 7) * C + j;
    s[j] = (sizeof(WT) == 1 && col < p.n) ? p.scales[col] : 1.f;
  }
  float acc[MT][C];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < C; ++j) acc[m][j] = 0.f;

  pdl_wait();   // A (and the residual) come from the previous kernel in the stream

  bool healthy = true;
  int stage_index = 0;   // global stage counter of this CTA
  for (int kc0 = k_begin; kc0 < k_end; kc0 += kGemvAChunk) {
    const int kc1 = min(k_end, kc0 + kGemvAChunk);
    const int padded = ((kc1 - kc0 + kGemvStageRows - 1) / kGemvStageRows) * kGemvStageRows;
    __syncthreads();                                          // previous chunk of A fully consumed
    for (int i = tid; i < MT * padded; i += kGemvThreads) {
      const int m = i / padded, kk = i - m * padded;
      const int row = m0 + m, kidx = kc0 + kk;
      a_smem[m * kGemvAChunk + kk] = (row < p.m && kidx < kc1) ? p.a[size_t(row) * p.lda + kidx] : __float2half(0.f);
    }
    __syncthreads();
    for (int kk0 = 0; kk0 < padded; kk0 += kGemvStageRows, ++stage_index) {
      const int slot = stage_index % kGemvStages;
      uint8_t* stage = stages + slot * GemvSmem::kStageBytes;
      if constexpr (TMA) {
        const uint32_t phase = uint32_t(stage_index / kGemvStages) & 1u;
        if (healthy) healthy = mbar_wait(&full[slot], phase, kStatusTmaTimeout);
        if (healthy) gemv_consume_stage<WT, MT>(stage, a_smem, kGemvAChunk, kk0, s, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
        if (tid == 0 && issued < n_stages_total && healthy) {
          // refill this slot with the tile kGemvStages ahead once every warp has released it
          healthy = mbar_wait(&empty[slot], phase, kStatusPipeTimeout);
          if (healthy) {
            mbar_expect_tx(&full[slot], GemvSmem::kStageBytes);
            tma_load_2d(stage, &w_map, n0, k_begin + issued * kGemvStageRows, &full[slot]);
            ++issued;
          }
        }
      } else {
        // Tiles filled by guarded loads (any alignment, any pitch); zero outside the matrix.  A 16-byte piece of a row
        // that lies wholly inside the matrix is assembled from the five aligned 32-bit words that cover it (funnel
        // shifts); pieces at the edges, and the last bytes of the buffer, go byte by byte.
        __syncthreads();
        const uint8_t* wb = static_cast<const uint8_t*>(p.w);
        const size_t w_bytes = (size_t(p.k - 1) * p.ldw + p.n) * sizeof(WT);      // one past the last byte of the matrix
        for (int i = tid; i < kGemvStageRows * 8; i += kGemvThreads) {
          const int r = i >> 3, piece = i & 7;
          const int kidx = kc0 + kk0 + r, col = n0 + piece * (16 / int(sizeof(WT)));
          uint4 v = make_uint4(0, 0, 0, 0);
          if (kidx < kc1 && col < p.n) {
            const size_t off = (size_t(kidx) * p.ldw + col) * sizeof(WT);
            const uintptr_t addr = reinterpret_cast<uintptr_t>(wb) + off;
            if (col + 16 / int(sizeof(WT)) <= p.n && off + 20 <= w_bytes && (off >= 3 || (addr & 3) == 0)) {
              const uint32_t* words = reinterpret_cast<const uint32_t*>(addr & ~uintptr_t(3));
              const uint32_t shift = uint32_t(addr & 3) * 8;
              const uint32_t w0 = words[0], w1 = words[1], w2 = words[2], w3 = words[3], w4 = shift ? words[4] : 0u;
              v.x = __funnelshift_r(w0, w1, shift); v.y = __funnelshift_r(w1, w2, shift);
              v.z = __funnelshift_r(w2, w3, shift); v.w = __funnelshift_r(w3, w4, shift);
            } else {
              uint8_t* bytes = reinterpret_cast<uint8_t*>(&v);
              const int valid = min(16, (p.n - col) * int(sizeof(WT)));
              for (int e = 0; e < valid; ++e) bytes[e] = wb[off + e];
            }
          }
          *reinterpret_cast<uint4*>(stages + r * 128 + piece * 16) = v;
        }
        __syncthreads();
        gemv_consume_stage<WT, MT>(stages, a_smem, kGemvAChunk, kk0, s, acc);
      }
    }
  }
  pdl_launch_dependents();

  // 4 row-lanes of a warp -> lanes 0..7, then the 8 warps in fixed order.
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < C; ++j) {
      float v = acc[m][j];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      acc[m][j] = v;
    }
  if (lane < 8) {
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int j = 0; j < C; ++j) red[(warp * MT + m) * 128 + lane * C + j] = acc[m][j];
  }
  __syncthreads();
  for (int i = tid; i < MT * BN; i += kGemvThreads) {
    const int m = i / BN, c = i - m * BN;
    float v = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) v += red[(w8 * MT + m) * 128 + c];
    part[m * 128 + c] = v;
  }
  if (splits > 1) cluster.sync(); else __syncthreads();
  const int cols_per_rank = BN / splits;                       // splits is 1, 2, 4 or 8
  for (int i = tid; i < MT * cols_per_rank; i += kGemvThreads) {
    const int m = i / cols_per_rank, c = rank * cols_per_rank + (i - m * cols_per_rank);
    float v = 0.f;
    if (splits > 1) {
      for (int r = 0; r < splits; ++r) v += cluster.map_shared_rank(part, r)[m * 128 + c];
    } else v = part[m * 128 + c];
    const int row = m0 + m, col = n0 + c;
    if (row < p.m && col < p.n && healthy) gemv_store(p, row, col, v);
  }
  if (splits > 1) cluster.sync();                              // peers may still be reading `part`
}

}  // namespace tib
