// INT8-weight GEMM on the sm_100a tensor cores (tcgen05.mma, accumulators in tensor memory).
//
//   out[M,N] = A[M,K] (fp16) . fp16_rn(float(W[K,N]) * scale[N]) + bias[N]      (fp32 accumulate)
//
// Used by the operator ABI from 5 rows of A upwards and by the model runtime for every row count
// (so that a request's logits do not depend on its batch): at decode batch sizes it keeps the kernel HBM-bound where SIMT
// FMAs would not (32 FMAs per weight byte), at prefill sizes it is the dense contraction.
//
// The problem is run transposed so that the 128 output channels of a CTA are the 128 TMEM lanes:
//   D[n, m] += Wt[n, k] * At[k, m]      MMA shape M=128 (channels) x N=NMMA (rows of A) x K=16
//   * A-operand: the weight tile, dequantised by CUDA cores into fp16 in shared memory, MN-major
//     (channel-contiguous, exactly how W is stored), no swizzle: 8(k) x 8(n) core matrices of 128 B;
//   * B-operand: NMMA rows of A, K-major, no swizzle;
//   * D: fp32, NMMA columns of tensor memory, read back with tcgen05.ld by 4 warps.
//
// Pipeline of one CTA (320 threads, 2 CTAs per SM at NMMA = 32):
//   warp 0      TMA producer: int8 tiles 64(k) x 128(n) -> ring of 3 raw stages (128-byte swizzle so the
//               dequantisers' 16-byte column reads are bank-conflict free);
//   warps 2-9   dequantise raw stage -> fp16 operand stage (ring of 3), copy the matching 64 columns of
//               A next to it (normalised on the way when the LayerNorm prologue is on), fence.proxy.async,
//               signal; the first stages are dequantised ahead of the dependency wait;
//   warp 1      owns the TMEM allocation; one lane issues 4 tcgen05.mma per stage and commits to the
//               barrier that releases the operand stage; a last commit publishes the accumulator;
//   warps 2-5   move the accumulators out of TMEM; then every thread finishes output elements.
// K can be split over a cluster of up to 8 CTAs.  One 32-row tile: each CTA pushes its partial sums into
// the shared memory of the CTA that finishes the column (one cluster barrier, local reads); larger tiles:
// partial tiles stay put and are read through distributed shared memory (two barriers).  Either way the
// sum runs in rank order.  Every wait is bounded.
#pragma once
#include <cooperative_groups.h>
#include <cuda.h>

#include <math_constants.h>

#include "common.cuh"
#include "elementwise.cuh"
#include "gemm_simt.cuh"

namespace tib {

constexpr int kTcDequantThreads = 256;                 // warps 2..9
#ifndef TIB_SLOT_GRID
#define TIB_SLOT_GRID (gridDim.x > 300)       // development builds: which launch records pipeline marks
#endif
constexpr int kTcThreads = 64 + kTcDequantThreads;
constexpr int kTcStageK = 64;
#ifndef TIB_TC_RAW_STAGES
#define TIB_TC_RAW_STAGES 3
#endif
#ifndef TIB_TC_OP_STAGES
#define TIB_TC_OP_STAGES 3
#endif
#ifndef TIB_TC_AHEAD
#define TIB_TC_AHEAD 3
#endif
constexpr int kTcRawStages = TIB_TC_RAW_STAGES;
constexpr int kTcOpStages = TIB_TC_OP_STAGES;
constexpr int kTcRawBytes = kTcStageK * 128;          // int8 tile
constexpr int kTcOpABytes = 128 * kTcStageK * 2;      // fp16 weight tile

// OPS: operand stages.  LEAN (one 32-row tile without K split or LayerNorm, i.e. the vocabulary projection): two operand
// stages and no receive region -- 65 KB, so that three CTAs share an SM and 393 column slabs run as one wave.
// WB: bytes per weight element (1 = int8 with scales, 2 = fp16): a raw stage is 64 rows x 128 channels of them.
template <int NMMA, bool LEAN = false, int WB = 1> struct TcSmem {
  static constexpr int kOps = LEAN || NMMA == 64 ? 2 : kTcOpStages;      // 64-row tiles: two stages keep two CTAs per SM
  static constexpr int kOpBBytes = NMMA * kTcStageK * 2;
  static constexpr int kRawStage = kTcRawBytes * WB;
  static constexpr int kRawOff = 0;                                        // 1024-aligned (TMA swizzle)
  static constexpr int kOpAOff = kRawOff + kTcRawStages * kRawStage;
  static constexpr int kOpBOff = kOpAOff + kOps * kTcOpABytes;
  // NMMA == 32 (decode): 16 KB where the other CTAs of a K-split cluster deposit their partial sums of the 128 / splits
  // columns this CTA finishes, [source rank][32 rows][128 / splits] fp32.  It aliases nothing: peers write it while this
  // CTA may still be in its main loop.
  static constexpr int kRecvOff = kOpBOff + kOps * kOpBBytes;
  static constexpr int kBarOff = kRecvOff + (NMMA <= 64 && !LEAN ? NMMA * 128 * 4 : 0);
  static constexpr int kBytes = kBarOff + 128 + 1024;                      // barriers + slack for manual 1024 alignment
};

// ---- tcgen05 wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
// Shared-memory matrix descriptor, no swizzle: start address, leading / stride byte offsets (16-byte
// units), descriptor version 1.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return uint64_t((smem_addr >> 4) & 0x3fffu) | (uint64_t((lbo_bytes >> 4) & 0x3fffu) << 16) |
         (uint64_t((sbo_bytes >> 4) & 0x3fffu) << 32) | (uint64_t(1) << 46);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread i of the warp = lane base + i).
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// grid = (N / 128 slabs, k splits [cluster y], M / NMMA tiles), block = 320.
// LN: LayerNorm prologue compiled in (0 = none, 1 = every CTA prepares the rows itself, 2 = rows shared out over the
// K-split cluster); separate instantiations keep the plain GEMM free of that code.
// DIRECT: the weight matrix cannot be described by a tensor map (row pitch not a multiple of 16 bytes); warp 0 then
// fills the raw stages itself with realigned loads instead of issuing TMA copies.
// WT: int8_t (weights dequantised on the way into the operand stage) or __half (fp16 weights, [K,N] row-major: the tiles
// arrive as two 64-channel boxes per stage and are only rearranged into the operand layout -- no arithmetic).
template <int NMMA, int LN = 0, bool LEAN = false, bool DIRECT = false, typename WT = int8_t>
__global__ void __launch_bounds__(kTcThreads, LEAN && sizeof(WT) == 1 ? 3 : NMMA <= 64 ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap w_map, const GemvArgs p) {
  trace_event(kTrGemmTc, 0);
  if (TIB_SLOT_GRID && threadIdx.x == 0) trace_slot(1);
  constexpr bool kHalfW = sizeof(WT) == 2;
  static_assert(!kHalfW || (LN == 0 && !DIRECT), "fp16 weights: plain tensor-map path");
  using L = TcSmem<NMMA, LEAN, int(sizeof(WT))>;
  constexpr int kRawStage = L::kRawStage;
  constexpr int kOps = L::kOps;
  static_assert(!LEAN || (NMMA == 32 && LN == 0), "lean layout: plain 32-row tiles");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw = smem + L::kRawOff;
  uint8_t* op_a = smem + L::kOpAOff;
  uint8_t* op_b = smem + L::kOpBOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t *raw_full = bars, *raw_empty = raw_full + kTcRawStages, *op_full = raw_empty + kTcRawStages, *op_empty = op_full + kOps,
           *acc_ready = op_empty + kOps;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  static_assert((2 * kTcRawStages + 2 * kOps + 2) * 8 <= 128, "barrier block");
  static_assert(LN == 0 || LN == 3 || kOps * L::kOpBBytes >= 8 * 768 * 2, "LayerNorm row strips live in the B-operand ring");
  __shared__ int s_failed;

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int splits = int(gridDim.y), rank = int(blockIdx.y);
  const int n0 = blockIdx.x * 128, m0 = blockIdx.z * NMMA;
  const bool serial_mode = NMMA >= 64 && p.serial_chunks > 1;   // many-row tiles only: the 32-row kernel carries none of it
  const int k_begin = serial_mode ? 0 : rank * p.k_chunk, k_end = serial_mode ? p.k : min(p.k, k_begin + p.k_chunk);
  const int stages = k_end > k_begin ? (k_end - k_begin + kTcStageK - 1) / kTcStageK : 0;
  // One accumulator of NMMA columns, or `serial_chunks` of them side by side (power of two, at most 512 columns).
  const int serial = serial_mode ? p.serial_chunks : 1;
  const uint32_t tmem_cols = uint32_t(max(32, NMMA * serial));

  if (p.early_trigger) pdl_launch_dependents();
  if (tid == 0) {
    s_failed = 0;
    if (!DIRECT) tma_prefetch_desc(&w_map);
    for (int s = 0; s < kTcRawStages; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], kTcDequantThreads / 32); }
    for (int s = 0; s < kOps; ++s) { mbar_init(&op_full[s], kTcDequantThreads / 32); mbar_init(&op_empty[s], 1); }
    mbar_init(acc_ready, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before();
  // LayerNorm prologue of more than 8 rows: the rows are shared out over the K-split cluster and the CTAs write each
  // other's statistics slots, which must be initialised first.  (Written as PTX: with cooperative_groups' cluster
  // sync in this place every launch of the kernel, also those that skip it, measured half a microsecond slower.)
  static_assert(LN == 0 || NMMA <= 64, "LayerNorm prologue: tiles of 32 or 64 rows");
  // LN == 3: shared mode for rows of up to 1024 values (the dispatcher checks that the strips of the rows one CTA
  // prepares fit the B-operand ring); a separate instantiation, so that the 768-wide kernels stay as they are.
  constexpr bool fuse_ln = LN != 0, ln_shared = LN >= 2;
  constexpr int kLnCols = LN == 3 ? 1024 : 768, kLnHeld = kLnCols / 256;
  // (mean, 1/sigma) of every row of the tile.  Shared mode: written by the CTA that prepares the row as one 8-byte store
  // through distributed shared memory and awaited by polling 1/sigma, whose initial bit pattern (a NaN that rsqrtf never
  // returns) means "not here yet": one remote store per row and CTA, no separate signal.
  __shared__ __align__(8) float2 s_stats[LN != 0 ? 64 : 1];
  constexpr uint32_t kStatPending = 0xffffffffu;
  if (ln_shared) {
    if (tid < NMMA) s_stats[tid] = make_float2(0.f, __uint_as_float(kStatPending));
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  } else {
    __syncthreads();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && DIRECT) {
    // ------------------------------------------------------------ producer without TMA: the whole warp copies a stage
    // (64 rows x 128 bytes = 512 pieces of 16 bytes, 16 per lane) from wherever the rows start; a piece wholly inside
    // the matrix is assembled from the five aligned words that cover it, edge pieces go byte by byte; zero outside.
    const uint8_t* wb = static_cast<const uint8_t*>(p.w);
    const size_t w_bytes = size_t(p.k - 1) * p.ldw + p.n;       // one past the last byte of the matrix
    bool ok = true;
    for (int i = 0; i < stages && ok; ++i) {
      const int slot = i % kTcRawStages;
      const uint32_t phase = uint32_t(i / kTcRawStages) & 1u;
      ok = mbar_wait(&raw_empty[slot], phase ^ 1u, kStatusPipeTimeout);
      if (!ok) break;
      uint8_t* tile = raw + slot * kRawStage;
#pragma unroll 1
      for (int batch = 0; batch < 2; ++batch) {
        uint4 v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int piece = lane + 32 * (batch * 8 + q), r = piece >> 3, ch = piece & 7;
          const int kidx = k_begin + i * kTcStageK + r, col = n0 + ch * 16;
          v[q] = make_uint4(0, 0, 0, 0);
          if (kidx < k_end && col < p.n) {
            const size_t off = size_t(kidx) * p.ldw + col;
            const uintptr_t addr = reinterpret_cast<uintptr_t>(wb) + off;
            if (col + 16 <= p.n && off + 20 <= w_bytes && (off >= 3 || (addr & 3) == 0)) {
              const uint32_t* words = reinterpret_cast<const uint32_t*>(addr & ~uintptr_t(3));
              const uint32_t shift = uint32_t(addr & 3) * 8;
              const uint32_t w0 = words[0], w1 = words[1], w2 = words[2], w3 = words[3], w4 = shift ? words[4] : 0u;
              v[q].x = __funnelshift_r(w0, w1, shift); v[q].y = __funnelshift_r(w1, w2, shift);
              v[q].z = __funnelshift_r(w2, w3, shift); v[q].w = __funnelshift_r(w3, w4, shift);
            } else {
              const int valid = min(16, p.n - col);
              uint32_t wd[4] = {0u, 0u, 0u, 0u};
#pragma unroll
              for (int e = 0; e < 16; ++e) if (e < valid) wd[e >> 2] |= uint32_t(wb[off + e]) << ((e & 3) * 8);
              v[q] = make_uint4(wd[0], wd[1], wd[2], wd[3]);
            }
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int piece = lane + 32 * (batch * 8 + q), r = piece >> 3, ch = piece & 7;
          *reinterpret_cast<uint4*>(tile + r * 128 + ((ch ^ (r & 7)) << 4)) = v[q];      // the layout TMA's 128-byte swizzle gives
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_full[slot]);
    }
    if (!ok && lane == 0) s_failed = 1;
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (weights only: no dependency wait)
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < stages && ok; ++i) {
        const int slot = i % kTcRawStages;
        const uint32_t phase = uint32_t(i / kTcRawStages) & 1u;
        ok = mbar_wait(&raw_empty[slot], phase ^ 1u, kStatusPipeTimeout);     // first round passes immediately
        if (!ok) break;
        mbar_expect_tx(&raw_full[slot], kRawStage);
        if (kHalfW) {
          // two boxes of 64 channels (128 bytes of fp16 per row, the widest a 128-byte swizzle takes)
          tma_load_2d(raw + slot * kRawStage, &w_map, n0, k_begin + i * kTcStageK, &raw_full[slot]);
          tma_load_2d(raw + slot * kRawStage + kTcRawBytes, &w_map, n0 + 64, k_begin + i * kTcStageK, &raw_full[slot]);
        } else if (p.w_slab_rows) tma_load_2d(raw + slot * kRawStage, &w_map, 0, int(blockIdx.x) * p.w_slab_rows + k_begin + i * kTcStageK, &raw_full[slot]);
        else tma_load_2d(raw + slot * kRawStage, &w_map, n0, k_begin + i * kTcStageK, &raw_full[slot]);
        if (TIB_SLOT_GRID) trace_slot(10 + i);
      }
      if (!ok) s_failed = 1;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 15) | (uint32_t(NMMA >> 3) << 17) | (uint32_t(128 >> 4) << 24);
      // weight tile, MN-major: 8-channel groups are 128 B apart (stride offset), 8-k groups 2048 B apart (leading offset)
      constexpr uint32_t a_lbo = 2048u, a_sbo = 128u;
      bool ok = true;
      for (int i = 0; i < stages && ok; ++i) {
        const int slot = i % kOps;
        ok = mbar_wait(&op_full[slot], uint32_t(i / kOps) & 1u, kStatusPipeTimeout);
        if (!ok) break;
        if (TIB_SLOT_GRID) trace_slot(70 + i);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(op_a + slot * kTcOpABytes), b_addr = smem_u32(op_b + slot * L::kOpBBytes);
        // serial mode: K range number (i * 64) / k_chunk has its own accumulator, started afresh at the range's first stage
        const int k_off = i * kTcStageK, chunk_id = (NMMA >= 64 && serial > 1) ? k_off / p.k_chunk : 0;
        const bool fresh = (NMMA >= 64 && serial > 1) ? k_off == chunk_id * p.k_chunk : i == 0;
        const uint32_t acc_col = uint32_t(chunk_id * NMMA);
#pragma unroll
        for (int kk = 0; kk < kTcStageK / 16; ++kk) {
          const uint64_t da = tc_desc(a_addr + kk * 2 * 2048, a_lbo, a_sbo);
          const uint64_t db = tc_desc(b_addr + kk * 2 * (NMMA / 8) * 128, (NMMA / 8) * 128, 128);
          tc_mma_f16(tmem_base + acc_col, da, db, idesc, (!fresh || kk > 0) ? 1u : 0u);
        }
        tc_commit(&op_empty[slot]);                 // frees the operand stage when these MMAs have read it
      }
      if (ok) tc_commit(acc_ready); else s_failed = 1;
    }
  } else {
    // ------------------------------------------------------------ dequantise + stage A rows (warps 2..5)
    const int t = tid - 64;                                   // 0..255
    const int r8 = t & 7, cc = (t >> 3) & 7, kg0 = t >> 6;     // k within 8-group, 16-byte chunk (16 channels), first k-group
    float sc[16];
    if (!kHalfW) {
#pragma unroll
      for (int j = 0; j < 16; ++j) { const int col = n0 + cc * 16 + j; sc[j] = col < p.n ? p.scales[col] : 1.f; }
    }
    // Weight tile of raw stage -> fp16 A-operand stage (independent of any earlier kernel).
    auto dequantise = [&](int rslot, int oslot) {
      const uint8_t* src = raw + rslot * kRawStage;
      uint8_t* dst = op_a + oslot * kTcOpABytes;
      if constexpr (kHalfW) {
        // 64 rows x 16 chunks of 8 channels, four per thread: out of the swizzled box, into core matrix (k group, channel group)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int id = t + kTcDequantThreads * j, k8 = id & 7, ch = (id >> 3) & 15, kg = id >> 7, krow = kg * 8 + k8;
          const uint4 w8 = *reinterpret_cast<const uint4*>(src + (ch >> 3) * kTcRawBytes + krow * 128 + (((ch & 7) ^ k8) << 4));
          *reinterpret_cast<uint4*>(dst + (kg * 16 + ch) * 128 + k8 * 16) = w8;
        }
      } else {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kg = kg0 + 4 * j, krow = kg * 8 + r8;
        const uint4 q = *reinterpret_cast<const uint4*>(src + krow * 128 + ((cc ^ r8) << 4));
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        __half2 h[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) dequant4(words[w], sc[4 * w], sc[4 * w + 1], sc[4 * w + 2], sc[4 * w + 3], h[2 * w], h[2 * w + 1]);
        uint8_t* core = dst + (kg * 16 + 2 * cc) * 128 + r8 * 16;      // core matrix (k-group, channel-group), row k%8
        *reinterpret_cast<uint4*>(core) = *reinterpret_cast<const uint4*>(&h[0]);
        *reinterpret_cast<uint4*>(core + 128) = *reinterpret_cast<const uint4*>(&h[4]);
      }
      }
    };
    // The matching 64 columns of A: NMMA rows x 8 chunks of 8 halves, as K-major core matrices.  The
    // global loads run kAhead stages ahead of their use (register ring), so their latency is covered by
    // the dequantisation of the stages in between instead of sitting on every stage's critical path.
    constexpr int kAhead = NMMA <= 64 ? TIB_TC_AHEAD : 1;
    constexpr int kPer = NMMA * 8 / kTcDequantThreads;
    uint4 a_ring[kAhead][kPer];
    auto fetch_a = [&](uint4 (&dst)[kPer], int i) {
      const int k0 = k_begin + i * kTcStageK;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int id = t + kTcDequantThreads * j, m8 = id & 7, kc = (id >> 3) & 7, mg = id >> 6;
        const int row = m0 + mg * 8 + m8, kcol = k0 + kc * 8;
        dst[j] = make_uint4(0, 0, 0, 0);
        if (i < stages && row < p.m && kcol < k_end) dst[j] = *reinterpret_cast<const uint4*>(p.a + size_t(row) * p.lda + kcol);
      }
    };
    // Optional LayerNorm of the rows (decode: NMMA == 32, K <= 768): statistics per row are computed once per CTA
    // right after the dependency resolves, with the same summation order as layernorm_kernel, and applied here.
    __shared__ __half s_gamma[LN != 0 && NMMA <= 64 ? kLnCols : 1], s_beta[LN != 0 && NMMA <= 64 ? kLnCols : 1];
    if (fuse_ln)
      for (int c = k_begin + t; c < k_end; c += kTcDequantThreads) { s_gamma[c - k_begin] = p.ln_gamma[c]; s_beta[c - k_begin] = p.ln_beta[c]; }
    auto store_a = [&](const uint4 (&src)[kPer], int oslot, int i) {
      uint8_t* bdst = op_b + oslot * L::kOpBBytes;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int id = t + kTcDequantThreads * j, m8 = id & 7, kc = (id >> 3) & 7, mg = id >> 6;
        uint4 v = src[j];
        if (fuse_ln) {
          const int m = mg * 8 + m8, kk = i * kTcStageK + kc * 8;      // row of the tile, k offset inside this CTA's range
          if (k_begin + kk < k_end) {
            __half* h = reinterpret_cast<__half*>(&v);
            const float2 st = s_stats[m & 63];
            const float mean = st.x, inv = st.y;
#pragma unroll
            for (int e = 0; e < 8; ++e) h[e] = f2h((h2f(h[e]) - mean) * inv * h2f(s_gamma[kk + e]) + h2f(s_beta[kk + e]));
          }
        }
        *reinterpret_cast<uint4*>(bdst + (kc * (NMMA / 8) + mg) * 128 + m8 * 16) = v;
      }
    };
    auto rotate = [&] {
#pragma unroll
      for (int d = 0; d + 1 < kAhead; ++d)
#pragma unroll
        for (int j = 0; j < kPer; ++j) a_ring[d][j] = a_ring[d + 1][j];
    };
    bool ok = true;
    // Lead-in: the first operand stages need no release; their weights are dequantised before the
    // dependency on the previous kernel is resolved, so under programmatic dependent launch this
    // overlaps the tail of that kernel.
    const int lead = min(stages, kOps);
    for (int i = 0; i < lead; ++i) {
      if (ok) ok = mbar_wait(&raw_full[i], 0, kStatusTmaTimeout);
      if (ok) dequantise(i, i);
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty[i]);
    }
    pdl_wait();                                               // A (and the residual) come from the previous kernel
    if (TIB_SLOT_GRID && t == 0) trace_slot(2);
    // The first stages' rows are requested together (one round trip instead of one per stage).  With the shared
    // LayerNorm prologue they go out before it (its barrier wait covers their latency); with the local one after
    // it (measured: ahead of it they delay the row loads the statistics wait for).
    constexpr bool kFetchFirst = LN >= 2;
    if constexpr (kAhead > 1 && kFetchFirst) {
#pragma unroll
      for (int d = 0; d < kAhead; ++d) fetch_a(a_ring[d], d);
    }
    if constexpr (LN != 0 && NMMA <= 64) {
      if (fuse_ln) {
        // Up to 8 rows: every CTA prepares them all itself, one warp per row.  More: the 32 rows of the tile are shared
        // out over the K-split cluster, rank r prepares rows r*R .. r*R+R-1 (R = 32 / splits), one warp per row
        // (w, w+8, ... of them), and sends each row's mean and 1/sigma to every CTA of the cluster, followed by an
        // arrival on that CTA's barrier (32 arrivals complete it).  Each row passes through a per-warp strip of the
        // still-empty B-operand ring.
        __half* strip = reinterpret_cast<__half*>(op_b) + size_t(warp - 2) * p.k;
        const int chunks = p.k / 8, share = ln_shared ? NMMA / splits : NMMA, first = ln_shared ? rank * share : 0;
#pragma unroll 1
        for (int local = warp - 2; local < share; local += 8) {   // one row per warp in the usual cases (<= 8 rows per CTA)
          float mean = 0.f, inv = 0.f;
          const int row = m0 + first + local;
          if (row < p.m) {                                    // warp-uniform
            uint4 held[kLnHeld];
#pragma unroll
            for (int u = 0; u < kLnHeld; ++u) {
              const int c = lane + 32 * u;
              held[u] = make_uint4(0, 0, 0, 0);
              if (c < chunks) held[u] = *reinterpret_cast<const uint4*>(p.a + size_t(row) * p.lda + c * 8);
            }
#pragma unroll
            for (int u = 0; u < kLnHeld; ++u) { const int c = lane + 32 * u; if (c < chunks) *reinterpret_cast<uint4*>(strip + c * 8) = held[u]; }
            __syncwarp();
            if (TIB_SLOT_GRID && t == 0) trace_slot(5);
            row_stats(strip, p.k, p.ln_eps, mean, inv);
            __syncwarp();
            if (TIB_SLOT_GRID && t == 0) trace_slot(6);
          }
          if (!ln_shared) {
            if (lane == 0) s_stats[local] = make_float2(mean, inv);
          } else if (lane < splits) {
            st_cluster_b64(cluster_addr(&s_stats[first + local], lane),
                           (unsigned long long)__float_as_uint(inv) << 32 | __float_as_uint(mean));
          }
        }
        if (!ln_shared) asm volatile("bar.sync 2, 256;" ::: "memory");      // the eight dequantising warps
        else {
          // every row of the tile is here once its 1/sigma has left the pending pattern (thread t polls rows t, t+256, ..)
          for (int r = t; r < NMMA; r += kTcDequantThreads) {
            bool here = false;
            for (uint32_t spin = 0; spin < kSpinLimit && !here; ++spin)
              here = uint32_t(reinterpret_cast<volatile unsigned long long*>(s_stats)[r] >> 32) != kStatPending;
            if (!here) { report(kStatusPipeTimeout); ok = false; }
          }
          if (TIB_SLOT_GRID && t == 0) trace_slot(7);
          asm volatile("bar.sync 2, 256;" ::: "memory");
          if (TIB_SLOT_GRID && t == 0) trace_slot(8);
        }
      }
    }
    if constexpr (kAhead > 1) {
      if constexpr (!kFetchFirst) {
#pragma unroll
        for (int d = 0; d < kAhead; ++d) fetch_a(a_ring[d], d);
      }
      for (int i = 0; i < lead; ++i) {
        store_a(a_ring[0], i, i);
        rotate();
        fetch_a(a_ring[kAhead - 1], i + kAhead);
        fence_async_smem();                                   // generic-proxy stores -> visible to tcgen05.mma
        __syncwarp();
        if (lane == 0) mbar_arrive(&op_full[i]);
        if (TIB_SLOT_GRID && t == 0) trace_slot(3 + i);
      }
    } else {
      for (int i = 0; i < lead; ++i) {
        fetch_a(a_ring[0], i);
        store_a(a_ring[0], i, i);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&op_full[i]);
      }
      fetch_a(a_ring[0], lead);
    }
    // From here a_ring[0] holds stage i's rows, a_ring[1..] the following stages'.
    for (int i = lead; i < stages; ++i) {
      const int rslot = i % kTcRawStages, oslot = i % kOps;
      if (ok) ok = mbar_wait(&raw_full[rslot], uint32_t(i / kTcRawStages) & 1u, kStatusTmaTimeout);
      if (ok) ok = mbar_wait(&op_empty[oslot], (uint32_t(i / kOps) & 1u) ^ 1u, kStatusMmaTimeout);
      if (TIB_SLOT_GRID && t == 0) trace_slot(30 + i);
      if (ok) {
        dequantise(rslot, oslot);
        store_a(a_ring[0], oslot, i);
        fence_async_smem();
      }
      rotate();
      fetch_a(a_ring[kAhead - 1], i + kAhead);
      __syncwarp();
      if (lane == 0) { mbar_arrive(&raw_empty[rslot]); mbar_arrive(&op_full[oslot]); }
      if (TIB_SLOT_GRID && t == 0) trace_slot(50 + i);
    }
    if (!ok) s_failed = 1;
  }
  pdl_wait();                 // every thread is past the dependency before the epilogue reads or writes global memory
  trace_event(kTrGemmTc, 1);
  pdl_launch_dependents();

  // ---------------------------------------------------------------- epilogue
  // Two steps, both written as short rolled loops (a decode GEMM runs for microseconds: the instructions it has to
  // fetch count as much as the ones it executes).  1. Warps 2..5 (TMEM lanes 32 * (warp % 4) ..) move the accumulators
  // out: into the shared memory of the CTA that finishes the column (K split, one 32-row tile: "push"), else into this
  // CTA's own.  2. After a barrier every thread finishes elements (row, column) of the columns this CTA owns: sum over
  // the K ranks in rank order, bias, activation, residual, store -- one copy of that code.
  float* part = reinterpret_cast<float*>(smem);                // [NMMA][128] fp32, aliases the drained pipeline stages
  float* recv = reinterpret_cast<float*>(smem + L::kRecvOff);  // NMMA == 32 only: [rank][32][128 / splits]
  constexpr bool kPush = NMMA <= 64 && !LEAN;
  const bool push = kPush && splits > 1;
  __shared__ long long s_row_base[NMMA];                       // K/V pool offset of each row of the tile (QKV projection only)
  bool acc_ok = true;
  const int cpr = 128 / splits;                                // columns this CTA finishes: [rank * cpr, rank * cpr + cpr)
  if (warp >= 2 && warp < 6) {
    if (p.k_pool)
      for (int i = tid - 64; i < NMMA; i += 128) s_row_base[i] = m0 + i < p.m ? kv_row_base(p, m0 + i) : 0;
    acc_ok = stages == 0 || mbar_wait(acc_ready, 0, kStatusMmaTimeout);
    if (TIB_SLOT_GRID && tid == 64) trace_slot(90);
    tc_fence_after();
    const int lane_base = 32 * (warp & 3), n_local = lane_base + lane;
    const int owner = n_local / cpr;
    float* dst = push ? cluster.map_shared_rank(recv, owner) + (rank * NMMA) * cpr + (n_local - owner * cpr) : part + n_local;
    const int pitch = push ? cpr : 128;
#pragma unroll 1
    for (int c0 = 0; c0 < NMMA; c0 += 32) {
      float v[32];
      if (acc_ok && stages > 0) tmem_load32(tmem_base + (uint32_t(lane_base) << 16) + uint32_t(c0), v);
      else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      if (NMMA >= 64 && serial > 1 && acc_ok && stages > 0) {
        // add the other K ranges' accumulators in range order: the fp32 sums of the K-split launch
#pragma unroll 1
        for (int r = 1; r < serial; ++r) {
          if (r * p.k_chunk >= p.k) break;
          float w[32];
          tmem_load32(tmem_base + (uint32_t(lane_base) << 16) + uint32_t(r * NMMA + c0), w);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += w[i];
        }
      }
      if (TIB_SLOT_GRID && tid == 64) trace_slot(91);
#pragma unroll
      for (int i = 0; i < 32; ++i) dst[(c0 + i) * pitch] = v[i];
    }
    if (TIB_SLOT_GRID && tid == 64) trace_slot(92);
    tc_fence_before();
  }
  // Finishing works on runs of 8 columns (16-byte loads and stores of fp16) when the tile is large and the layout
  // allows, else element by element.  The bias and residual of a thread's first run are requested now and arrive while the barrier is pending
  // (both are complete: every thread is past the dependency wait); inside the loop the next run's are requested
  // before the current one is finished, so a 64..256-row tile does not pay one round trip per run.
  const int total = NMMA * cpr;
  // (compiled for tiles of 64 rows and more only: the 32-row decode kernel stays small)
  const bool vec8 = NMMA >= 64 && NMMA * cpr >= 8 * kTcThreads &&    // small tiles: one element per thread keeps every thread busy
                    !p.out_fp32 && cpr % 8 == 0 && p.n % 8 == 0 && p.ldo % 8 == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0 &&
                    (!p.bias || reinterpret_cast<uintptr_t>(p.bias) % 16 == 0) && (!p.residual || reinterpret_cast<uintptr_t>(p.residual) % 16 == 0) &&
                    (!p.k_pool || p.kv_hidden % 64 == 0);
  const int runs_per_row = cpr / 8, runs = NMMA * runs_per_row;
  uint4 bias8 = make_uint4(0, 0, 0, 0), res8 = bias8;
  auto request = [&](int i, uint4& b8, uint4& r8) {              // inputs of run i (vec8)
    const int m = i / runs_per_row, row = m0 + m, col = n0 + rank * cpr + (i - m * runs_per_row) * 8;
    b8 = make_uint4(0, 0, 0, 0); r8 = b8;
    if (i < runs && row < p.m && col < p.n) {
      if (p.bias) b8 = *reinterpret_cast<const uint4*>(p.bias + col);
      if (p.residual && !(p.k_pool && col >= p.kv_hidden)) r8 = *reinterpret_cast<const uint4*>(p.residual + size_t(row) * p.ldo + col);
    }
  };
  constexpr int kPre = NMMA <= 32 ? 2 : 4;                      // elements per thread of a split 32 / 64-row tile
  __half pre_bias[kPre], pre_res[kPre];
#pragma unroll
  for (int s = 0; s < kPre; ++s) pre_bias[s] = pre_res[s] = f2h(0.f);
  // 64-row tiles of a K split: a thread finishes four neighbouring columns of one row (their partial sums are read as
  // float4, one per rank), so the 1024 elements of the tile take one round of 256 threads instead of four.
  const bool quad = NMMA == 64 && push && cpr % 4 == 0 && p.n % 4 == 0 && p.ldo % 4 == 0 && !p.out_fp32 &&
                    (!p.bias || reinterpret_cast<uintptr_t>(p.bias) % 8 == 0) && (!p.residual || reinterpret_cast<uintptr_t>(p.residual) % 8 == 0);
  const int quads_per_row = cpr / 4, quads = NMMA * quads_per_row;
  uint2 quad_bias = make_uint2(0, 0), quad_res = make_uint2(0, 0);
  if (NMMA >= 64 && vec8) request(tid, bias8, res8);
  else if (NMMA == 64 && quad) {
    const int m = tid / quads_per_row, row = m0 + m, col = n0 + rank * cpr + (tid - m * quads_per_row) * 4;
    if (tid < quads && row < p.m && col < p.n) {
      if (p.bias) quad_bias = *reinterpret_cast<const uint2*>(p.bias + col);
      if (p.residual && !(p.k_pool && col >= p.kv_hidden)) quad_res = *reinterpret_cast<const uint2*>(p.residual + size_t(row) * p.ldo + col);
    }
  } else {
#pragma unroll
    for (int s = 0; s < kPre; ++s) {
      const int i = tid + s * kTcThreads, m = i / cpr, row = m0 + m, col = n0 + rank * cpr + (i - m * cpr);
      if (i < total && row < p.m && col < p.n) {
        if (p.bias) pre_bias[s] = p.bias[col];
        if (p.residual && !p.out_fp32 && !(p.k_pool && col >= p.kv_hidden)) pre_res[s] = p.residual[size_t(row) * p.ldo + col];
      }
    }
  }
  if (splits > 1) cluster.sync(); else __syncthreads();         // all partial sums are where they will be read
  if (TIB_SLOT_GRID && tid == 64) trace_slot(93);
  const bool good = !s_failed;
  const bool wide_rows = splits == 1 && p.out_fp32 && !p.k_pool && p.ldo % 4 == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0;
  if (wide_rows) {
    // fp32 rows without a K split (vocabulary projection) leave as float4: 512-byte runs per warp
    for (int i = tid; i < NMMA * 32; i += kTcThreads) {
      const int m = i >> 5, c = (i & 31) * 4, row = m0 + m, col = n0 + c;
      if (row >= p.m || !good) continue;
      float4 f = *reinterpret_cast<const float4*>(part + m * 128 + c);
      if (p.bias) {
        if (col < p.n) f.x += h2f(p.bias[col]);
        if (col + 1 < p.n) f.y += h2f(p.bias[col + 1]);
        if (col + 2 < p.n) f.z += h2f(p.bias[col + 2]);
        if (col + 3 < p.n) f.w += h2f(p.bias[col + 3]);
      }
      if (p.argmax_best) {
        // a warp holds one row's 128 columns (the loop bounds are multiples of 32 and `row` is the same for the 32 lanes):
        // largest value, lowest column among equals, columns past N and NaN never win (reference argmax, llm/src/runtime.cu:59-66)
        float bv = -CUDART_INF_F; int bi = 0x7fffffff;
        const float vals[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (col + e < p.n && (vals[e] > bv || (vals[e] == bv && col + e < bi))) { bv = vals[e]; bi = col + e; }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((tid & 31) == 0 && bi != 0x7fffffff) atomicMax(p.argmax_best + row, argmax_pack(bv, bi));
        if (p.skip_store) continue;
      }
      float* out = static_cast<float*>(p.out) + size_t(row) * p.ldo + col;
      if (col + 3 < p.n) *reinterpret_cast<float4*>(out) = f;
      else {
        if (col < p.n) out[0] = f.x;
        if (col + 1 < p.n) out[1] = f.y;
        if (col + 2 < p.n) out[2] = f.z;
      }
    }
  } else if (NMMA >= 64 && vec8) {
#pragma unroll 1
    for (int i = tid; i < runs; i += kTcThreads) {
      uint4 next_b, next_r;
      request(i + kTcThreads, next_b, next_r);
      const int m = i / runs_per_row, c = (i - m * runs_per_row) * 8;
      const int row = m0 + m, col = n0 + rank * cpr + c;
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
      if (push) {
        for (int r = 0; r < splits; ++r) {
          const float4 lo = *reinterpret_cast<const float4*>(recv + (r * NMMA + m) * cpr + c), hi = *reinterpret_cast<const float4*>(recv + (r * NMMA + m) * cpr + c + 4);
          v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w; v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
        }
      } else if (splits > 1) {
        for (int r = 0; r < splits; ++r) {
          const float* src = cluster.map_shared_rank(part, r) + m * 128 + rank * cpr + c;
          const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
          v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w; v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
        }
      } else {
        const float4 lo = *reinterpret_cast<const float4*>(part + m * 128 + c), hi = *reinterpret_cast<const float4*>(part + m * 128 + c + 4);
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      }
      if (row < p.m && col < p.n && good) {
        const __half* b = reinterpret_cast<const __half*>(&bias8);
        const __half* rr = reinterpret_cast<const __half*>(&res8);
        const bool to_cache = p.k_pool && col >= p.kv_hidden;
        uint4 packed;
        __half* h = reinterpret_cast<__half*>(&packed);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          __half t = f2h(v[e] + h2f(b[e]));                    // the rounding points of gemv_store
          if (!to_cache) {
            if (p.gelu) t = f2h(gelu_tanh(h2f(t)));
            if (p.residual) t = f2h(h2f(rr[e]) + h2f(t));
          }
          h[e] = t;
        }
        if (to_cache) {
          const int cc = col - p.kv_hidden, which = cc >= p.kv_hidden, e0 = which ? cc - p.kv_hidden : cc;
          *reinterpret_cast<uint4*>((which ? p.v_pool : p.k_pool) + s_row_base[m] + (e0 >> 6) * 2048 + (e0 & 63)) = packed;
        } else {
          *reinterpret_cast<uint4*>(static_cast<__half*>(p.out) + size_t(row) * p.ldo + col) = packed;
        }
      }
      bias8 = next_b; res8 = next_r;
    }
  } else if (NMMA == 64 && quad) {
#pragma unroll 1
    for (int i = tid, round = 0; i < quads; i += kTcThreads, ++round) {
      const int m = i / quads_per_row, c = (i - m * quads_per_row) * 4, row = m0 + m;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < splits; ++r) {
        const float4 part4 = *reinterpret_cast<const float4*>(recv + (r * NMMA + m) * cpr + c);
        acc.x += part4.x; acc.y += part4.y; acc.z += part4.z; acc.w += part4.w;
      }
#pragma unroll 1
      for (int e = 0; e < 4; ++e) {
        const int col = n0 + rank * cpr + c + e;
        const float v = e == 0 ? acc.x : e == 1 ? acc.y : e == 2 ? acc.z : acc.w;
        const uint32_t wb = e < 2 ? quad_bias.x : quad_bias.y, wr = e < 2 ? quad_res.x : quad_res.y;
        const __half b = __ushort_as_half(static_cast<unsigned short>((e & 1) ? wb >> 16 : wb & 0xffffu));
        const __half rr = __ushort_as_half(static_cast<unsigned short>((e & 1) ? wr >> 16 : wr & 0xffffu));
        if (row < p.m && col < p.n && good) gemv_store(p, row, col, v, p.k_pool ? s_row_base[m] : -1, round == 0, b, rr);
      }
    }
  } else {
#pragma unroll 1
    for (int i = tid, s = 0; i < total; i += kTcThreads, ++s) {
      const int m = i / cpr, c = i - m * cpr;
      float v = 0.f;
      if (push) {
        for (int r = 0; r < splits; ++r) v += recv[(r * NMMA + m) * cpr + c];
      } else if (splits > 1) {
        for (int r = 0; r < splits; ++r) v += cluster.map_shared_rank(part, r)[m * 128 + rank * cpr + c];
      } else {
        v = part[m * 128 + c];
      }
      const int row = m0 + m, col = n0 + rank * cpr + c;
      if (row < p.m && col < p.n && good) {
        __half b = pre_bias[0], r = pre_res[0];
#pragma unroll
        for (int q = 1; q < kPre; ++q) if (s == q) { b = pre_bias[q]; r = pre_res[q]; }
        gemv_store(p, row, col, v, p.k_pool ? s_row_base[m] : -1, s < kPre, b, r);
      }
    }
  }
  if (TIB_SLOT_GRID && tid == 64) trace_slot(94);
  // Pull mode: peers may still be reading this CTA's partial sums.  Push mode: nobody reads remotely after the barrier.
  if (splits > 1 && !push) cluster.sync(); else __syncthreads();
  trace_event(kTrGemmTc, 2);
  if (TIB_SLOT_GRID && threadIdx.x == 0) trace_slot(99);
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, tmem_cols); }
}

}  // namespace tib
