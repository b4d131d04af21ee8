// One whole greedy decode step of the INT8-weight GPT-2 runtime as ONE persistent kernel (up to 32 requests).
//
// The layer loop of the reference (llm/src/runtime.cu:135-168: embed, then per layer ln -> c_attn -> scatter ->
// gather -> attention -> merge -> c_proj -> add -> ln -> c_fc -> gelu -> c_proj -> add, ln_f, lm_head, argmax) costs
// one kernel launch per operation; at decode sizes every one of them is a few microseconds of latency around a few
// hundred kilobytes of weights.  Here the step is a single launch of one CTA per SM and the SMs hand activations to
// each other through global memory (L2) without ever leaving the kernel:
//
//   * Static roles.  CTA c owns the same piece of every layer: one 128-channel slab of c_attn, of attn.c_proj or of
//     c_fc over the whole K, or one (slab, K range) of mlp.c_proj.  The remaining CTAs prepare the embedding rows.
//     Decode attention items (request, head) and the slabs of the vocabulary projection are dealt round robin over
//     all CTAs.  A CTA walks its items in layer order; an item only ever waits for items of earlier phases, so with
//     every CTA resident (cooperative launch) the schedule cannot deadlock.
//   * Weights never wait for activations.  Warp 0 streams the CTA's weight tiles (slab-major int8, 64 x 128 bytes per
//     stage) by TMA into a ring of kStepRaw stages in the fixed order of its items, layers ahead of their use: the
//     ring is refilled as soon as a stage is released, whatever phase the rest of the CTA is in.  The first
//     kStepOps stages of the next item are also dequantised ahead of time.
//   * Hand-over without barriers.  Every activation that crosses CTAs travels as 64-bit words {payload, tag}: two
//     fp16 values (or one fp32 partial sum) and a 32-bit tag that names (step, layer).  A 64-bit store is single-copy
//     atomic, so a consumer that reads a word with the tag it expects has the payload; it polls the words it needs
//     and nothing else -- no fence, no flag, no grid-wide barrier.  Tags grow from step to step, so a buffer needs
//     no clearing.  Every poll is bounded; on expiry the CTA records a status, stops waiting and leaves.
//   * Same arithmetic as the separate kernels.  Tiles run on tcgen05.mma with the operand layouts of gemm_tc.cuh;
//     the K ranges of the launch-per-GEMM path keep one TMEM accumulator each and are added in range order, LayerNorm
//     uses row_stats, the attention replays attn_decode_staged_kernel: logits and tokens are bit-identical to the
//     65-launch step.
//
// One launch = one step; state (ids, positions, lengths, step counter, tag epoch) lives in device memory and is
// advanced by the CTA that finishes last, so launches can follow each other without the host.
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include "attention.cuh"
#include "common.cuh"
#include "elementwise.cuh"
#include "gemm_tc.cuh"
#include "model_glue.cuh"
#include "step_plan.hpp"

namespace tib {

constexpr int kStepThreads = kTcThreads;        // warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 workers
constexpr int kStepWorkers = kTcDequantThreads;
constexpr int kStepRaw = 4;                     // int8 weight stages in flight / resident ahead of use
constexpr int kStepOps = 6;                     // fp16 operand stages: this many stages of the next item are dequantised ahead of its input
constexpr uint32_t kFlagSpinLimit = 1u << 20;   // polls of an L2 round trip each: about a second

struct StepSmem {
  static constexpr int kRawOff = 0;                                           // 1024-aligned (TMA 128-byte swizzle)
  static constexpr int kOpAOff = kRawOff + kStepRaw * kTcRawBytes;
  static constexpr int kOpBBytes = kStepRows * kTcStageK * 2;
  static constexpr int kOpBOff = kOpAOff + kStepOps * kTcOpABytes;
  // Input rows of the current GEMM item as plain fp16 (row pitch kRowPitch halves: 16 bytes more than a power of two, so
  // that the 16-byte row reads of eight rows fall into different banks); the decode attention's K/V tiles between items.
  static constexpr int kRowPitch = kStepMaxHidden + 8;
  static constexpr int kScratchOff = kOpBOff + kStepOps * kOpBBytes;
  static constexpr int kScratchBytes = kStepRows * kRowPitch * 2;
  static constexpr int kBarOff = kScratchOff + kScratchBytes;
  static constexpr int kBarBytes = 512;
  static constexpr int kBytes = kBarOff + kBarBytes + 1024;                   // + slack for manual 1024 alignment
};
static_assert(StepSmem::kScratchBytes >= kStagedWarps * 2 * kPageTokens * 64 * 2, "attention tiles live in the row scratch");
static_assert(StepSmem::kBarOff % 8 == 0, "barrier alignment");

// ---- tagged words ---------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long flag_word(uint32_t payload, uint32_t tag) {
  return (unsigned long long)tag << 32 | payload;
}
__device__ __forceinline__ void st_flag(unsigned long long* p, uint32_t payload, uint32_t tag) {
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(flag_word(payload, tag)) : "memory");
}
__device__ __forceinline__ void st_flag2(unsigned long long* p, uint32_t a, uint32_t b, uint32_t tag) {   // p 16-byte aligned
  asm volatile("st.relaxed.gpu.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(flag_word(a, tag)), "l"(flag_word(b, tag)) : "memory");
}
__device__ __forceinline__ unsigned long long ld_flag(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ld_flag2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {   // p 16-byte aligned
  asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ bool step_aborted(volatile int* failed) {
  return *failed != 0 || *reinterpret_cast<volatile unsigned int*>(&g_device_status) != 0;
}
// Polls until both words carry `tag`.  False after kFlagSpinLimit polls, or when this CTA or any other kernel of the
// library has recorded a failure meanwhile.
__device__ __forceinline__ bool poll_flag2(const unsigned long long* p, uint32_t tag, unsigned long long& a, unsigned long long& b,
                                           volatile int* failed) {
  for (uint32_t spin = 0; spin < kFlagSpinLimit; ++spin) {
    if (uint32_t(a >> 32) == tag && uint32_t(b >> 32) == tag) return true;
    if ((spin & 255u) == 255u && step_aborted(failed)) return false;
    ld_flag2(p, a, b);
  }
  if (uint32_t(a >> 32) == tag && uint32_t(b >> 32) == tag) return true;
  report(kStatusFlagTimeout);
  *failed = 1;
  return false;
}
__device__ __forceinline__ bool poll_flag(const unsigned long long* p, uint32_t tag, unsigned long long& a, volatile int* failed) {
  for (uint32_t spin = 0; spin < kFlagSpinLimit; ++spin) {
    if (uint32_t(a >> 32) == tag) return true;
    if ((spin & 255u) == 255u && step_aborted(failed)) return false;
    a = ld_flag(p);
  }
  if (uint32_t(a >> 32) == tag) return true;
  report(kStatusFlagTimeout);
  *failed = 1;
  return false;
}
// mbarrier wait that also gives up when the CTA has failed elsewhere.
__device__ __forceinline__ bool step_wait(uint64_t* bar, uint32_t parity, unsigned int code, volatile int* failed) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *failed) return false;
  }
  report(code);
  *failed = 1;
  return false;
}

__device__ __forceinline__ uint32_t pack_halves(__half lo, __half hi) {
  return uint32_t(__half_as_ushort(lo)) | uint32_t(__half_as_ushort(hi)) << 16;
}
__device__ __forceinline__ __half low_half(uint32_t w) { return __ushort_as_half(static_cast<unsigned short>(w & 0xffffu)); }
__device__ __forceinline__ __half high_half(uint32_t w) { return __ushort_as_half(static_cast<unsigned short>(w >> 16)); }

// ---- items ------------------------------------------------------------------------------------------
enum StepKind : int { kItemQkv = 0, kItemProj = 1, kItemFc = 2, kItemProj2 = 3, kItemHead = 4 };
struct StepItem {
  int kind, layer, slab, rank;     // rank: K range of mlp.c_proj, else 0
  int y0;                          // first tile row of the item's weights in the arena
  int stages;                      // 64-row stages
  int chunk_stages;                // stages per K range (one TMEM accumulator each)
  int n0;                          // first output channel
  const float* scales; const __half* bias;
};

// Item number j of CTA `cta` (role from step_role): its layer items in layer order, then its vocabulary slabs.
__device__ __forceinline__ int step_item_count(const StepPlan& p, const StepRole& role, int cta, int grid) {
  const int head_slabs = p.head_slabs > cta ? (p.head_slabs - cta + grid - 1) / grid : 0;
  return (role.kind >= 0 ? p.layers : 0) + head_slabs;
}
__device__ __forceinline__ StepItem step_item(const StepPlan& p, const StepRole& role, int cta, int grid, int j) {
  StepItem it{};
  const int layer_items = role.kind >= 0 ? p.layers : 0;
  if (j < layer_items) {
    const StepLayer& L = p.layer[j];
    const StepLinear& lin = role.kind == kItemQkv ? L.qkv : role.kind == kItemProj ? L.proj : role.kind == kItemFc ? L.fc : L.proj2;
    it.kind = role.kind; it.layer = j; it.slab = role.slab; it.rank = role.rank;
    const int k_item = role.kind == kItemProj2 ? p.chunk_proj2 : p.hidden;
    const int chunk = role.kind == kItemQkv ? p.chunk_qkv : role.kind == kItemProj ? p.chunk_proj : role.kind == kItemFc ? p.chunk_fc : p.chunk_proj2;
    it.y0 = lin.tile_row0 + role.slab * lin.slab_rows + (role.kind == kItemProj2 ? role.rank * p.chunk_proj2 : 0);
    it.stages = k_item / kTcStageK; it.chunk_stages = chunk / kTcStageK;
    it.scales = lin.scales; it.bias = lin.bias;
  } else {
    it.kind = kItemHead; it.layer = p.layers; it.slab = cta + (j - layer_items) * grid; it.rank = 0;
    it.y0 = p.head.tile_row0 + it.slab * p.head.slab_rows;
    it.stages = p.hidden / kTcStageK; it.chunk_stages = p.chunk_head / kTcStageK;
    it.scales = p.head.scales; it.bias = nullptr;
  }
  it.n0 = it.slab * 128;
  return it;
}

// grid = one CTA per SM (cooperative launch: every CTA resident), block = kStepThreads.
__global__ void __launch_bounds__(kStepThreads, 1)
decode_step_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ StepPlan p) {
  using S = StepSmem;
  extern __shared__ uint8_t step_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(step_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw = smem + S::kRawOff;
  uint8_t* op_a = smem + S::kOpAOff;
  uint8_t* op_b = smem + S::kOpBOff;
  uint8_t* scratch = smem + S::kScratchOff;
  __half* arow = reinterpret_cast<__half*>(scratch);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
  uint64_t *raw_full = bars, *raw_empty = raw_full + kStepRaw, *op_full = raw_empty + kStepRaw, *op_empty = op_full + kStepOps,
           *acc_ready = op_empty + kStepOps, *acc_free = acc_ready + 1, *att_bar = acc_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(att_bar + kStagedWarps);
  static_assert((2 * kStepRaw + 2 * kStepOps + 2 + kStagedWarps) * 8 + 8 <= S::kBarBytes, "barrier block");

  __shared__ int s_failed_store;
  __shared__ int s_issued, s_consumed;                       // weight stages requested / taken over, for the exit path
  __shared__ __align__(8) float2 s_stats[kStepRows];         // (mean, 1/sigma) of the rows of a LayerNorm item
  __shared__ __half s_gamma[kStepMaxHidden], s_beta[kStepMaxHidden];
  __shared__ long long s_row_base[kStepRows];                // K/V pool offset of row r's position in layer 0, head 0
  __shared__ int s_len[kStepRows];                           // visible keys of each request
  __shared__ float s_acc[kStagedWarps][64];
  __shared__ float s_ml[kStagedWarps][2];
  __shared__ float s_top_v[4][kStepRows];                    // argmax: per epilogue warp and row
  __shared__ int s_top_i[4][kStepRows];
  __shared__ unsigned long long s_best[kStepRows];           // best (value, index) of this CTA's vocabulary slabs
  volatile int* failed = &s_failed_store;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = int(blockIdx.x), grid = int(gridDim.x);
  const int M = p.batch;
  const StepRole role = step_role(p, cta);
  const int n_items = step_item_count(p, role, cta, grid);
  const int hidden_words = p.hidden / 2;
  // ranks of the widest item: K ranges of one hidden-wide GEMM
  const uint32_t tmem_cols = 256;

  if (tid == 0) {
    s_failed_store = 0; s_issued = 0; s_consumed = 0;
    tma_prefetch_desc(&w_map);
    for (int s = 0; s < kStepRaw; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], kStepWorkers / 32); }
    for (int s = 0; s < kStepOps; ++s) { mbar_init(&op_full[s], kStepWorkers / 32); mbar_init(&op_empty[s], 1); }
    mbar_init(acc_ready, 1); mbar_init(acc_free, 4);
    for (int w = 0; w < kStagedWarps; ++w) mbar_init(&att_bar[w], 1);
    mbar_fence_init();
  }
  if (tid < kStepRows) s_best[tid] = 0ull;
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Tags of this step: base + 1 + index, index = layer for what a layer produces, `layers` for the final hidden state.
  const uint32_t epoch = *reinterpret_cast<volatile unsigned int*>(p.sync);
  const uint32_t tag_base = epoch * 64u;
  const int step_now = *reinterpret_cast<volatile int32_t*>(p.step);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: the CTA's weight stages in item order
    if (lane == 0) {
      int raw_i = 0;
      bool ok = true;
      for (int j = 0; j < n_items && ok; ++j) {
        const StepItem it = step_item(p, role, cta, grid, j);
        for (int i = 0; i < it.stages && ok; ++i, ++raw_i) {
          const int slot = raw_i % kStepRaw;
          ok = step_wait(&raw_empty[slot], (uint32_t(raw_i / kStepRaw) & 1u) ^ 1u, kStatusPipeTimeout, failed);
          if (!ok) break;
          mbar_expect_tx(&raw_full[slot], kTcRawBytes);
          tma_load_2d(raw + slot * kTcRawBytes, &w_map, 0, it.y0 + i * kTcStageK, &raw_full[slot]);
        }
      }
      s_issued = raw_i;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 15) | (uint32_t(kStepRows >> 3) << 17) | (uint32_t(128 >> 4) << 24);
      constexpr uint32_t a_lbo = 2048u, a_sbo = 128u;
      int op_i = 0;
      bool ok = true;
      for (int j = 0; j < n_items && ok; ++j) {
        const StepItem it = step_item(p, role, cta, grid, j);
        if (j > 0) ok = step_wait(acc_free, uint32_t(j - 1) & 1u, kStatusPipeTimeout, failed);   // the accumulators have been read out
        if (!ok) break;
        tc_fence_after();
        for (int i = 0; i < it.stages && ok; ++i, ++op_i) {
          const int slot = op_i % kStepOps;
          ok = step_wait(&op_full[slot], uint32_t(op_i / kStepOps) & 1u, kStatusPipeTimeout, failed);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(op_a + slot * kTcOpABytes), b_addr = smem_u32(op_b + slot * S::kOpBBytes);
          const int range = i / it.chunk_stages;                 // K range = accumulator, started afresh at its first stage
          const bool fresh = i == range * it.chunk_stages;
#pragma unroll
          for (int kk = 0; kk < kTcStageK / 16; ++kk) {
            const uint64_t da = tc_desc(a_addr + kk * 2 * 2048, a_lbo, a_sbo);
            const uint64_t db = tc_desc(b_addr + kk * 2 * (kStepRows / 8) * 128, (kStepRows / 8) * 128, 128);
            tc_mma_f16(tmem_base + uint32_t(range * kStepRows), da, db, idesc, (!fresh || kk > 0) ? 1u : 0u);
          }
          tc_commit(&op_empty[slot]);
        }
        if (ok) tc_commit(acc_ready);
      }
    }
  } else {
    // ------------------------------------------------------------ workers (warps 2..9)
    const int t = tid - 64, ww = warp - 2;                     // 0..255, 0..7
    const int r8 = t & 7, cc = (t >> 3) & 7, kg0 = t >> 6;      // dequantiser: k within 8-group, 16-channel chunk, first k-group
    int raw_i = 0, op_i = 0, att_i = 0;
    bool ok = true;
    float sc[16];
#ifdef TIB_STEP_TIMELINE
    int tl_n = 0;
    auto step_mark = [&](int code) {
      if (t == 0 && p.timeline && tl_n < 1024) {
        unsigned long long tm;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
        p.timeline[size_t(cta) * 1024 + tl_n++] = (unsigned long long)code << 48 | (tm & 0xffffffffffffull);
      }
    };
#define STEP_MARK(layer, event) step_mark((layer) * 32 + (event))
#else
#define STEP_MARK(layer, event) ((void)0)
#endif
    STEP_MARK(63, 0);

    // Per-request constants of this step: visible keys and where the new K/V row goes.
    if (t < kStepRows) {
      long long base = 0; int len = 0;
      if (t < M) {
        const int pos = p.row_pos[t];
        const int page = p.table[size_t(p.slots[t]) * p.table_pitch + (pos >> 5)];
        base = (long long)page * p.layers * p.heads * 2048 + (pos & 31) * 64;
        len = max(0, min(p.kv_len[t], p.table_pitch * kPageTokens));
      }
      s_row_base[t] = base; s_len[t] = len;
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");

    // Weight tile of raw stage -> fp16 A-operand stage: the layout and the arithmetic of gemm_tc_kernel.
    auto dequantise = [&](int rslot, int oslot) {
      const uint8_t* src = raw + rslot * kTcRawBytes;
      uint8_t* dst = op_a + oslot * kTcOpABytes;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kg = kg0 + 4 * j, krow = kg * 8 + r8;
        const uint4 q = *reinterpret_cast<const uint4*>(src + krow * 128 + ((cc ^ r8) << 4));
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        __half2 h[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) dequant4(words[w], sc[4 * w], sc[4 * w + 1], sc[4 * w + 2], sc[4 * w + 3], h[2 * w], h[2 * w + 1]);
        uint8_t* core = dst + (kg * 16 + 2 * cc) * 128 + r8 * 16;
        *reinterpret_cast<uint4*>(core) = *reinterpret_cast<const uint4*>(&h[0]);
        *reinterpret_cast<uint4*>(core + 128) = *reinterpret_cast<const uint4*>(&h[4]);
      }
    };
    // What an item can do before its input exists: scales, LayerNorm parameters, and its first operand stages.
    int lead_done = 0;
    bool head_params = false;                                  // ln_f gamma / beta are in place (they serve every vocabulary slab)
    auto prepare = [&](const StepItem& it) {
#pragma unroll
      for (int j = 0; j < 16; ++j) { const int col = it.n0 + cc * 16 + j; sc[j] = (it.kind != kItemHead || col < p.vocab) ? it.scales[col] : 1.f; }
      if (it.kind == kItemQkv || it.kind == kItemFc || (it.kind == kItemHead && !head_params)) {
        head_params = it.kind == kItemHead;
        const __half* g = it.kind == kItemHead ? p.lnf_g : it.kind == kItemQkv ? p.layer[it.layer].ln1_g : p.layer[it.layer].ln2_g;
        const __half* b = it.kind == kItemHead ? p.lnf_b : it.kind == kItemQkv ? p.layer[it.layer].ln1_b : p.layer[it.layer].ln2_b;
        for (int c = t; c < p.hidden; c += kStepWorkers) { s_gamma[c] = g[c]; s_beta[c] = b[c]; }
      }
      lead_done = min(it.stages, kStepOps);
      for (int i = 0; i < lead_done; ++i) {
        const int rslot = (raw_i + i) % kStepRaw, oslot = (op_i + i) % kStepOps;
        if (ok) ok = step_wait(&raw_full[rslot], uint32_t((raw_i + i) / kStepRaw) & 1u, kStatusTmaTimeout, failed);
        if (ok) ok = step_wait(&op_empty[oslot], (uint32_t((op_i + i) / kStepOps) & 1u) ^ 1u, kStatusMmaTimeout, failed);
        if (ok) dequantise(rslot, oslot);
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&raw_empty[rslot]);
      }
    };

    // rows x cols halves of a tagged buffer (row pitch src_pitch words, first column col0) -> arow.
    auto gather = [&](const unsigned long long* src, int src_pitch, int col0, int cols, uint32_t tag) {
      const int per_row = cols / 4, total = M * per_row;       // 16-byte pieces: two words, four values
#pragma unroll 1
      for (int base = t; base < total; base += kStepWorkers * 4) {
        unsigned long long a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + kStepWorkers * u;
          a[u] = b[u] = 0ull;
          if (idx < total && ok) { const int r = idx / per_row, c = idx - r * per_row; ld_flag2(src + size_t(r) * src_pitch + col0 / 2 + 2 * c, a[u], b[u]); }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + kStepWorkers * u;
          if (idx < total && ok) {
            const int r = idx / per_row, c = idx - r * per_row;
            ok = poll_flag2(src + size_t(r) * src_pitch + col0 / 2 + 2 * c, tag, a[u], b[u], failed);
            *reinterpret_cast<uint2*>(arow + r * S::kRowPitch + 4 * c) = make_uint2(uint32_t(a[u]), uint32_t(b[u]));
          }
        }
      }
    };
    // Row statistics of the gathered rows (reference summation order, elementwise.cuh), one warp per row.
    auto row_statistics = [&]() {
#pragma unroll 1
      for (int row = ww; row < M; row += kStepWorkers / 32) {
        float mean, inv;
        row_stats(arow + row * S::kRowPitch, p.hidden, p.ln_eps, mean, inv);
        if (lane == 0) s_stats[row] = make_float2(mean, inv);
      }
    };
    // Stage i of the item's rows -> K-major core matrices of the B operand, normalised on the way when `ln`.
    auto store_a = [&](int i, int oslot, bool ln) {
      const int m8 = t & 7, kc = (t >> 3) & 7, mg = t >> 6;
      const int row = mg * 8 + m8, kk = i * kTcStageK + kc * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < M) {
        v = *reinterpret_cast<const uint4*>(arow + row * S::kRowPitch + kk);
        if (ln) {
          __half* h = reinterpret_cast<__half*>(&v);
          const float2 st = s_stats[row];
          const float mean = st.x, inv = st.y;
#pragma unroll
          for (int e = 0; e < 8; ++e) h[e] = f2h((h2f(h[e]) - mean) * inv * h2f(s_gamma[kk + e]) + h2f(s_beta[kk + e]));
        }
      }
      *reinterpret_cast<uint4*>(op_b + oslot * S::kOpBBytes + (kc * (kStepRows / 8) + mg) * 128 + m8 * 16) = v;
    };
    // The main loop of an item whose rows are in arow; `ln`: normalise them.
    auto run_stages = [&](const StepItem& it, bool ln) {
      for (int i = 0; i < it.stages; ++i, ++raw_i, ++op_i) {
        const int rslot = raw_i % kStepRaw, oslot = op_i % kStepOps;
        if (i >= lead_done) {
          if (ok) ok = step_wait(&raw_full[rslot], uint32_t(raw_i / kStepRaw) & 1u, kStatusTmaTimeout, failed);
          if (ok) ok = step_wait(&op_empty[oslot], (uint32_t(op_i / kStepOps) & 1u) ^ 1u, kStatusMmaTimeout, failed);
          if (ok) dequantise(rslot, oslot);
        }
        if (ok) { store_a(i, oslot, ln); fence_async_smem(); }
        __syncwarp();
        if (lane == 0 && ok) { if (i >= lead_done) mbar_arrive(&raw_empty[rslot]); mbar_arrive(&op_full[oslot]); }
      }
      if (t == 0) s_consumed = raw_i;
      // every worker is done with the rows, the statistics and the LayerNorm parameters of this item: what follows
      // (the next item's parameters, the attention's K/V tiles) may overwrite them
      asm volatile("bar.sync 2, 256;" ::: "memory");
    };

    // Accumulators of an item -> registers: v[i] = sum over the K ranges, in range order, of D[channel][row i].
    const int lane_base = 32 * (warp & 3), n_local = lane_base + lane;
    auto read_acc = [&](float (&v)[32], int ranges, int item_index) {
      if (ok) ok = step_wait(acc_ready, uint32_t(item_index) & 1u, kStatusMmaTimeout, failed);
      ok = __all_sync(0xffffffffu, ok);                      // tcgen05.ld is warp-collective
      tc_fence_after();
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.f;
#pragma unroll 1
      for (int r = 0; r < ranges && ok; ++r) {
        float w[32];
        tmem_load32(tmem_base + (uint32_t(lane_base) << 16) + uint32_t(r * kStepRows), w);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += w[i];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(acc_free);
    };
    // Rows 2k / 2k+1 of a column pair leave as one tagged word each: even lanes write even rows, odd lanes odd rows.
    auto store_pairs = [&](const __half (&h)[32], unsigned long long* dst, int pitch_words, int col, uint32_t tag) {
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        if (i < M) {
          const uint32_t mine = (lane & 1) ? __half_as_ushort(h[i]) : __half_as_ushort(h[i + 1]);
          const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, 1);
          const int row = i + (lane & 1);
          const uint32_t word = (lane & 1) ? (theirs | uint32_t(__half_as_ushort(h[i + 1])) << 16)
                                           : (uint32_t(__half_as_ushort(h[i])) | theirs << 16);
          if (row < M && ok) st_flag(dst + size_t(row) * pitch_words + col / 2, word, tag);
        }
      }
    };
    // The residual of rows (2k + lane parity) for this lane's column pair, requested ahead of the accumulators.
    uint32_t res_w[16];
    auto request_residual = [&](const unsigned long long* src, int pitch_words, int col, uint32_t tag) {
      unsigned long long w[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) { const int row = 2 * k + (lane & 1); w[k] = 0ull; if (row < M && ok) w[k] = ld_flag(src + size_t(row) * pitch_words + col / 2); }
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const int row = 2 * k + (lane & 1);
        if (row < M && ok) ok = poll_flag(src + size_t(row) * pitch_words + col / 2, tag, w[k], failed);
        res_w[k] = uint32_t(w[k]);
      }
    };
    // residual of (row i, this lane's column): own word for rows of this lane's parity, the neighbour's otherwise
    auto residual_of = [&](int k, __half& r_even_row, __half& r_odd_row) {
      const uint32_t theirs = __shfl_xor_sync(0xffffffffu, res_w[k], 1);
      if (lane & 1) { r_even_row = high_half(theirs); r_odd_row = high_half(res_w[k]); }
      else { r_even_row = low_half(res_w[k]); r_odd_row = low_half(theirs); }
    };

    // ---------------------------------------------------------------- decode attention of one (request, head)
    // The arithmetic of attn_decode_staged_kernel: warp w owns the 32-key tiles w, w+8, ...; a tile is a cache page and
    // arrives by two bulk copies.  The query and the newest key/value row come from the tagged QKV buffer.
    auto attention_item = [&](int b, int h, int layer) {
      constexpr int D = 64, W = kStagedWarps, DP = D / 8, KPS = 32 / DP, STEPS = 32 / KPS, kTileBytes = kPageTokens * D * 2;
      const int dp = lane % DP, ksub = lane / DP;
      __half* k_tile = reinterpret_cast<__half*>(scratch + size_t(ww) * 2 * kTileBytes);
      __half* v_tile = k_tile + kPageTokens * D;
      uint64_t* bar = &att_bar[ww];
      const int len = s_len[b];
      const uint32_t tag = tag_base + 1u + uint32_t(layer);
      const int32_t* pages = p.table + size_t(p.slots[b]) * p.table_pitch;
      auto request = [&](int t0) {
        const size_t o = ((size_t(pages[t0 / kPageTokens]) * p.layers + layer) * p.heads + h) * kPageTokens * D;
        mbar_expect_tx(bar, 2 * kTileBytes);
        bulk_load(k_tile, p.k_pool + o, kTileBytes, bar);
        bulk_load(v_tile, p.v_pool + o, kTileBytes, bar);
      };
      const int t_first = ww * 32;
      ok = __all_sync(0xffffffffu, ok);
      fence_async_smem();                                    // earlier generic-proxy traffic of this scratch, before the copies
      __syncwarp();
      if (lane == 0 && t_first < len && ok) request(t_first);
      // the query (every lane its 8 values) and, lanes 0..15, the newest key / value row
      const unsigned long long* qrow = p.qkvf + size_t(b) * (3 * hidden_words);
      unsigned long long qa = 0, qb = 0, qc = 0, qd = 0, na = 0, nb = 0, nc = 0, nd = 0;
      const unsigned long long* qsrc = qrow + (h * D + dp * 8) / 2;
      const unsigned long long* nsrc = qrow + ((lane < DP ? p.hidden : 2 * p.hidden) + h * D + dp * 8) / 2;
      if (ok) { ld_flag2(qsrc, qa, qb); ld_flag2(qsrc + 2, qc, qd); }
      if (ok && lane < 2 * DP) { ld_flag2(nsrc, na, nb); ld_flag2(nsrc + 2, nc, nd); }
      if (ok) ok = poll_flag2(qsrc, tag, qa, qb, failed);
      if (ok) ok = poll_flag2(qsrc + 2, tag, qc, qd, failed);
      if (lane < 2 * DP) {
        if (ok) ok = poll_flag2(nsrc, tag, na, nb, failed);
        if (ok) ok = poll_flag2(nsrc + 2, tag, nc, nd, failed);
      }
      ok = __all_sync(0xffffffffu, ok);
      const uint4 qraw = make_uint4(uint32_t(qa), uint32_t(qb), uint32_t(qc), uint32_t(qd));
      const uint4 fresh = make_uint4(uint32_t(na), uint32_t(nb), uint32_t(nc), uint32_t(nd));
      const __half2* q2 = reinterpret_cast<const __half2*>(&qraw);
      float m = -CUDART_INF_F, l = 0.f, acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int t0 = t_first, it = 0; t0 < len; t0 += W * 32, ++it, ++att_i) {
        if (lane == 0 && ok && it > 0) request(t0);
        if (ok) ok = mbar_wait(bar, uint32_t(att_i) & 1u, kStatusTmaTimeout);
        ok = __all_sync(0xffffffffu, ok);
        if (len - 1 >= t0 && len - 1 < t0 + 32) {
          // this step's key / value row: the copy in the tagged buffer is complete, the cache page may not be yet
          const int j = len - 1 - t0;
          if (lane < 2 * DP) *reinterpret_cast<uint4*>((lane < DP ? k_tile : v_tile) + j * D + dp * 8) = fresh;
          __syncwarp();
        }
        float sc_[STEPS], tile_max = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
          const int j = i * KPS + ksub, key = t0 + j;
          const uint4 kraw = *reinterpret_cast<const uint4*>(k_tile + j * D + dp * 8);
          const __half2* k2 = reinterpret_cast<const __half2*>(&kraw);
          float d = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            d = fma_f16(d, __low2half(q2[e]), __low2half(k2[e]));
            d = fma_f16(d, __high2half(q2[e]), __high2half(k2[e]));
          }
#pragma unroll
          for (int x = 1; x < DP; x <<= 1) d += __shfl_xor_sync(0xffffffffu, d, x);
          sc_[i] = (key < len && ok) ? d * rsqrtf(float(D)) : -CUDART_INF_F;
          tile_max = fmaxf(tile_max, sc_[i]);
        }
#pragma unroll
        for (int x = DP; x < 32; x <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, x));
        if (tile_max > -CUDART_INF_F) {
          const float next = fmaxf(m, tile_max);
          const float alpha = expf(m - next);
          l *= alpha;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] *= alpha;
#pragma unroll
          for (int i = 0; i < STEPS; ++i) {
            const int j = i * KPS + ksub;
            if (t0 + j < len) {
              const float pr = expf(sc_[i] - next);
              l += pr;
              const uint4 vraw = *reinterpret_cast<const uint4*>(v_tile + j * D + dp * 8);
              const __half2* v2 = reinterpret_cast<const __half2*>(&vraw);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                acc[2 * e] = fmaf(pr, __low2float(v2[e]), acc[2 * e]);
                acc[2 * e + 1] = fmaf(pr, __high2float(v2[e]), acc[2 * e + 1]);
              }
            }
          }
          m = next;
        }
        fence_async_smem();
        __syncwarp();
      }
#pragma unroll
      for (int x = DP; x < 32; x <<= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, x);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], x);
      }
      if (lane < DP) {
#pragma unroll
        for (int e = 0; e < 8; ++e) s_acc[ww][dp * 8 + e] = acc[e];
        if (lane == 0) { s_ml[ww][0] = m; s_ml[ww][1] = l; }
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (t < D) {
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < W; ++w) mm = fmaxf(mm, s_ml[w][0]);
        float ll = 0.f, aa = 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w) {
          const float f = s_ml[w][0] > -CUDART_INF_F ? expf(s_ml[w][0] - mm) : 0.f;
          ll += s_ml[w][1] * f; aa += s_acc[w][t] * f;
        }
        const uint32_t mine = __half_as_ushort(f2h(ll > 0.f ? aa / ll : 0.f));
        const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, 1);
        if (!(t & 1) && ok) st_flag(p.attnf + size_t(b) * hidden_words + (h * D + t) / 2, mine | theirs << 16, tag);
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");       // s_acc / s_ml are free again
    };

    // ---------------------------------------------------------------- the step
    // Embedding rows: the last CTAs, one row each (reference embed, llm/src/runtime.cu:25-30) -> x of layer 0.
    if (cta >= grid - M) {
      const int r = grid - 1 - cta;
      const __half* te = p.wte + size_t(max(0, min(p.ids[r], p.vocab - 1))) * p.hidden;
      const __half* pe = p.wpe + size_t(p.row_pos[r]) * p.hidden;
      for (int c = t; c < p.hidden / 8; c += kStepWorkers) {
        uint4 a = *reinterpret_cast<const uint4*>(te + c * 8);
        const uint4 b = *reinterpret_cast<const uint4*>(pe + c * 8);
        __half* ah = reinterpret_cast<__half*>(&a);
        const __half* bh = reinterpret_cast<const __half*>(&b);
#pragma unroll
        for (int e = 0; e < 8; ++e) ah[e] = f2h(h2f(ah[e]) + h2f(bh[e]));
        unsigned long long* dst = p.xf + size_t(r) * hidden_words + c * 4;
        st_flag2(dst, a.x, a.y, tag_base + 1u);
        st_flag2(dst + 2, a.z, a.w, tag_base + 1u);
      }
    }

    int item_index = 0;
    StepItem it{};
    if (n_items > 0) { it = step_item(p, role, cta, grid, 0); prepare(it); }
    const int first_att = ((cta - p.first_helper) % grid + grid) % grid;
    auto next_item = [&]() {
      ++item_index;
      if (item_index < n_items) { it = step_item(p, role, cta, grid, item_index); prepare(it); }
    };

    for (int layer = 0; layer < p.layers; ++layer) {
      const uint32_t tag_in = tag_base + 1u + uint32_t(layer), tag_out = tag_in, tag_next = tag_in + 1u;
      if (role.kind == kItemQkv) {
        // x -> LayerNorm -> c_attn + bias; Q, K, V to the tagged buffer, K and V also to their cache pages
        STEP_MARK(layer, 1);
        gather(p.xf, hidden_words, 0, p.hidden, tag_in);
        asm volatile("bar.sync 2, 256;" ::: "memory");
        STEP_MARK(layer, 2);
        row_statistics();
        asm volatile("bar.sync 2, 256;" ::: "memory");
        STEP_MARK(layer, 3);
        run_stages(it, true);
        STEP_MARK(layer, 4);
        if (warp < 6) {
          const int col = it.n0 + n_local;
          const __half bias = it.bias[col];
          float v[32];
          read_acc(v, it.stages / it.chunk_stages, item_index);
          STEP_MARK(layer, 5);
          __half h[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) h[i] = f2h(v[i] + h2f(bias));
          store_pairs(h, p.qkvf, 3 * hidden_words, col, tag_out);
          if (col >= p.hidden) {
            const int c = col - p.hidden, which = c >= p.hidden, e = which ? c - p.hidden : c;
            __half* pool = (which ? p.v_pool : p.k_pool) + (long long)layer * p.heads * 2048 + (e >> 6) * 2048 + (e & 63);
#pragma unroll
            for (int i = 0; i < 32; ++i) if (i < M && ok) pool[s_row_base[i]] = h[i];
          }
          STEP_MARK(layer, 6);
        }
        next_item();
        STEP_MARK(layer, 7);
      }
      // decode attention: items (request, head) dealt round robin, the helper CTAs first
      for (int a = first_att; a < M * p.heads; a += grid) { STEP_MARK(layer, 8); attention_item(a / p.heads, a % p.heads, layer); STEP_MARK(layer, 9); }
      if (role.kind == kItemProj) {
        // attention output -> attn.c_proj + bias + x -> res
        if (warp < 6) request_residual(p.xf, hidden_words, it.n0 + n_local, tag_in);   // x has been complete since before c_attn
        STEP_MARK(layer, 1);
        gather(p.attnf, hidden_words, 0, p.hidden, tag_in);
        asm volatile("bar.sync 2, 256;" ::: "memory");
        STEP_MARK(layer, 2);
        run_stages(it, false);
        STEP_MARK(layer, 4);
        if (warp < 6) {
          const int col = it.n0 + n_local;
          const __half bias = it.bias[col];
          float v[32];
          read_acc(v, it.stages / it.chunk_stages, item_index);
          STEP_MARK(layer, 5);
          __half h[32];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            __half r0, r1;
            residual_of(k, r0, r1);
            h[2 * k] = f2h(h2f(r0) + h2f(f2h(v[2 * k] + h2f(bias))));
            h[2 * k + 1] = f2h(h2f(r1) + h2f(f2h(v[2 * k + 1] + h2f(bias))));
          }
          store_pairs(h, p.resf, hidden_words, col, tag_out);
          STEP_MARK(layer, 6);
        }
        next_item();
        STEP_MARK(layer, 7);
      }
      if (role.kind == kItemFc) {
        // res -> LayerNorm -> c_fc + bias -> tanh-GELU -> act
        STEP_MARK(layer, 1);
        gather(p.resf, hidden_words, 0, p.hidden, tag_in);
        asm volatile("bar.sync 2, 256;" ::: "memory");
        STEP_MARK(layer, 2);
        row_statistics();
        asm volatile("bar.sync 2, 256;" ::: "memory");
        STEP_MARK(layer, 3);
        run_stages(it, true);
        STEP_MARK(layer, 4);
        if (warp < 6) {
          const int col = it.n0 + n_local;
          const __half bias = it.bias[col];
          float v[32];
          read_acc(v, it.stages / it.chunk_stages, item_index);
          STEP_MARK(layer, 5);
          __half h[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            h[i] = f2h(0.f);
            if (i < M) h[i] = f2h(gelu_tanh(h2f(f2h(v[i] + h2f(bias)))));      // a branch, not a select: tanhf only for rows that exist
          }
          store_pairs(h, p.actf, p.ff / 2, col, tag_out);
          STEP_MARK(layer, 6);
        }
        next_item();
        STEP_MARK(layer, 7);
      }
      if (role.kind == kItemProj2) {
        // act[:, K range] -> partial sums of mlp.c_proj; then this CTA finishes its share of the slab's columns:
        // sum over the K ranges in range order + bias + res -> x of the next layer
        const int ranks = p.ranks_proj2;
        STEP_MARK(layer, 1);
        gather(p.actf, p.ff / 2, it.rank * p.chunk_proj2, p.chunk_proj2, tag_in);
        asm volatile("bar.sync 2, 256;" ::: "memory");
        STEP_MARK(layer, 2);
        run_stages(it, false);
        STEP_MARK(layer, 4);
        if (warp < 6) {
          float v[32];
          read_acc(v, 1, item_index);
          STEP_MARK(layer, 5);
          unsigned long long* dst = p.partf + (size_t(it.slab * ranks + it.rank) * kStepRows) * 128 + n_local;
#pragma unroll
          for (int i = 0; i < 32; ++i) if (i < M && ok) st_flag(dst + size_t(i) * 128, __float_as_uint(v[i]), tag_out);
          STEP_MARK(layer, 6);
        }
        const int pairs = (64 + ranks - 1) / ranks, pair0 = it.rank * pairs, my_pairs = max(0, min(64, pair0 + pairs) - pair0);
#pragma unroll 1
        for (int e = t; e < M * my_pairs; e += kStepWorkers) {
          const int mrow = e / my_pairs, c = 2 * (pair0 + e - mrow * my_pairs), col = it.n0 + c;
          unsigned long long pa[8], pb[8], rw;
          const unsigned long long* src = p.partf + (size_t(it.slab * ranks) * kStepRows + mrow) * 128 + c;
#pragma unroll
          for (int q = 0; q < 8; ++q) { pa[q] = pb[q] = 0ull; if (q < ranks && ok) ld_flag2(src + size_t(q) * kStepRows * 128, pa[q], pb[q]); }
          rw = ok ? ld_flag(p.resf + size_t(mrow) * hidden_words + col / 2) : 0ull;
          const uint32_t bias2 = *reinterpret_cast<const uint32_t*>(it.bias + col);
          float v0 = 0.f, v1 = 0.f;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (q < ranks) {
              if (ok) ok = poll_flag2(src + size_t(q) * kStepRows * 128, tag_out, pa[q], pb[q], failed);
              v0 += __uint_as_float(uint32_t(pa[q])); v1 += __uint_as_float(uint32_t(pb[q]));
            }
          if (ok) ok = poll_flag(p.resf + size_t(mrow) * hidden_words + col / 2, tag_in, rw, failed);
          const __half h0 = f2h(h2f(low_half(uint32_t(rw))) + h2f(f2h(v0 + h2f(low_half(bias2)))));
          const __half h1 = f2h(h2f(high_half(uint32_t(rw))) + h2f(f2h(v1 + h2f(high_half(bias2)))));
          if (ok) st_flag(p.xf + size_t(mrow) * hidden_words + col / 2, pack_halves(h0, h1), tag_next);
        }
        STEP_MARK(layer, 10);
        next_item();
        STEP_MARK(layer, 7);
      }
    }

    // ---------------------------------------------------------------- final LayerNorm, vocabulary projection, argmax
    if (item_index < n_items) {
      STEP_MARK(p.layers, 1);
      gather(p.xf, hidden_words, 0, p.hidden, tag_base + 1u + uint32_t(p.layers));
      asm volatile("bar.sync 2, 256;" ::: "memory");
      STEP_MARK(p.layers, 2);
      row_statistics();
      asm volatile("bar.sync 2, 256;" ::: "memory");
      STEP_MARK(p.layers, 3);
    }
    while (item_index < n_items) {
      run_stages(it, true);
      STEP_MARK(p.layers, 4);
      if (warp < 6) {
        const int col = it.n0 + n_local;
        float v[32];
        read_acc(v, it.stages / it.chunk_stages, item_index);
        if (p.logits && col < p.vocab) {
#pragma unroll
          for (int i = 0; i < 32; ++i) if (i < M && ok) p.logits[size_t(i) * p.logits_pitch + col] = v[i];
        }
        // per row: the largest value of the warp's 32 channels, lowest channel among equals (llm/src/runtime.cu:59-66)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < M) {
            float bv = (col < p.vocab && v[i] == v[i]) ? v[i] : -CUDART_INF_F;
            int bi = (col < p.vocab && v[i] == v[i]) ? col : 0x7fffffff;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
              const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
              const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
              if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) { s_top_v[warp - 2][i] = bv; s_top_i[warp - 2][i] = bi; }
          }
        }
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if (warp == 2 && lane < M) {
          float bv = s_top_v[0][lane]; int bi = s_top_i[0][lane];
#pragma unroll
          for (int w = 1; w < 4; ++w) {
            const float ov = s_top_v[w][lane]; const int oi = s_top_i[w][lane];
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
          }
          if (bi != 0x7fffffff) { const unsigned long long key = argmax_pack(bv, bi); if (key > s_best[lane]) s_best[lane] = key; }
        }
        asm volatile("bar.sync 3, 128;" ::: "memory");
      }
      STEP_MARK(p.layers, 6);
      next_item();
    }
    if (warp == 2 && lane < M && s_best[lane] && ok) atomicMax(p.best + lane, s_best[lane]);
    STEP_MARK(63, 1);
    if (t == 0) s_consumed = raw_i;
  }

  // ------------------------------------------------------------------ the end of the step
  tc_fence_before();
  __syncthreads();
  if (warp == 0 && lane == 0 && *failed) {
    // weight stages that were requested but never taken over: wait for the copies before the CTA leaves
    for (int i = s_consumed; i < s_issued; ++i) mbar_wait(&raw_full[i % kStepRaw], uint32_t(i / kStepRaw) & 1u, kStatusTmaTimeout);
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, tmem_cols); }
  // The CTA that finishes last publishes the tokens and advances the device-resident state (argmax / advance kernels
  // of the launch-per-operation step).
  if (tid == 0) {
    __threadfence();
    const unsigned int ticket = atomicAdd(p.sync + 1, 1u);
    if (ticket == unsigned(grid) - 1u) {
      __threadfence();
      const bool good = *reinterpret_cast<volatile unsigned int*>(&g_device_status) == 0;
      for (int r = 0; r < M; ++r) {
        const unsigned long long key = atomicExch(p.best + r, 0ull);
        const int bi = key ? int(0xffffffffu - uint32_t(key)) : 0x7fffffff;
        if (good) {
          p.log[size_t(step_now) * M + r] = bi;
          p.ids[r] = bi < p.vocab ? bi : 0;                  // a row without any comparable logit must not become an address
          if (bi >= p.vocab) report(kStatusNoToken);
          p.row_pos[r] += 1; p.kv_len[r] += 1;
        }
      }
      if (good) *p.step = step_now + 1;
      p.sync[0] = epoch + 1u;
      p.sync[1] = 0u;
    }
  }
}

}  // namespace tib
