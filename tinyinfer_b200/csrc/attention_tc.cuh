// Ragged causal attention for many query rows per request (prefill) on the sm_100a tensor cores.
//
// Same semantics as attn_tile_kernel / the reference's online_attention (kernels/src/cuda/tc/attention.cu:9-57): key j
// is visible to query i of request b when j < min(kv_len, kv_lengths[b]) and (!causal || j <= offsets[b] + i); scores
// q.k * rsqrt(64); fp32 online softmax; rows that see no key are exact zeros.  What changes is where the two
// contractions run: one CTA owns 128 query rows of one (request, head) and walks the keys 64 at a time,
//   S[128 x 64] = Q . K^T        tcgen05.mma kind::f16, both operands K-major in shared memory, accumulator in TMEM
//   P = exp(S - max) (fp16)      two threads per query row (32 keys of the tile each): their halves of the row of S come
//                                out of TMEM with tcgen05.ld; the tile maximum is exchanged through shared memory under a
//                                barrier the pipeline needs anyway, the denominator is kept in two shares until the end
//   PV[128 x 64] = P . V         tcgen05.mma with P K-major and V as it is stored (head dimension contiguous = MN-major)
//   O = O * alpha + PV           in registers (32 fp32 per thread)
// The two contractions of neighbouring key tiles overlap the softmax: S of tile i+1 is issued before the softmax of tile
// i starts (two S accumulators in TMEM, K/V tiles in a ring of three filled by cp.async one tile ahead), and PV of tile
// i is folded into O only when tile i+1 needs the P buffer -- the additions happen in the same order as if every step
// were waited for at once, so the pipelining does not change a bit of the result.
// The exponentials are the hardware's ex2 (__expf: relative error of a few 2^-23, against the 2^-11 rounding of P that
// follows).  The probabilities enter the second contraction rounded to fp16 (the reference multiplies fp32 p by fp16 v); the
// difference is far inside the operator gate (atol = rtol = 0.02).  A row's result depends on its own keys only -- key
// tiles start at key 0 whatever the query tile -- so it does not change with the batch or with the chunking of a prompt.
// Head dimension 64 only; other shapes stay on the SIMT kernel.
#pragma once
#include <math_constants.h>

#include "attention.cuh"
#include "common.cuh"
#include "gemm_tc.cuh"

namespace tib {

constexpr int kAttnTcRows = 128;      // query rows per CTA = TMEM lanes
constexpr int kAttnTcKeys = 64;       // keys per step
constexpr int kAttnTcMinRows = 64;    // requests with fewer query rows stay on the SIMT kernel (model runtime)

struct AttnTcSmem {
  static constexpr int kTile = kAttnTcKeys * 64 * 2;                // one K or V tile: 8 KB
  static constexpr int kQOff = 0;                                   // Q  [128 x 64]  K-major core matrices, 16 KB
  static constexpr int kRing = 3;                                   // K/V tiles in rotation
  static constexpr int kKOff = kQOff + kAttnTcRows * 64 * 2;        // K  3 x [64 keys x 64]  K-major
  static constexpr int kVOff = kKOff + kRing * kTile;               // V  3 x [64 keys x 64]  MN-major (d contiguous)
  static constexpr int kPOff = kVOff + kRing * kTile;               // P  [128 x 64 keys]  K-major, 16 KB
  static constexpr int kBytes = kPOff + kAttnTcRows * kAttnTcKeys * 2;
};

// 32 lanes x 32 columns twice: one row of a 64-column accumulator
__device__ __forceinline__ void tmem_load64(uint32_t taddr, float (&v)[64]) {
  float lo[32], hi[32];
  tmem_load32(taddr, lo);
  tmem_load32(taddr + 32u, hi);
#pragma unroll
  for (int i = 0; i < 32; ++i) { v[i] = lo[i]; v[32 + i] = hi[i]; }
}

constexpr int kAttnTcThreads = 2 * kAttnTcRows;    // two threads per query row: warps 0-3 hold keys / dims 0..31, warps 4-7 hold 32..63

// grid = (ceil(max query rows / 128), heads, batch), block = 256.  min_q: requests with fewer rows are skipped (another
// kernel serves them); 0 = serve every request.
template <typename KV>
__global__ void __launch_bounds__(kAttnTcThreads, 2)
attn_tc_kernel(const AttnArgs p, const KV kv, const int min_q) {
  using L = AttnTcSmem;
  extern __shared__ __align__(128) uint8_t attn_tc_smem[];
  uint8_t* qs = attn_tc_smem + L::kQOff;
  uint8_t* ks = attn_tc_smem + L::kKOff;
  uint8_t* vs = attn_tc_smem + L::kVOff;
  uint8_t* ps = attn_tc_smem + L::kPOff;
  __shared__ __align__(8) uint64_t s_done, pv_done;
  __shared__ uint32_t tmem_slot;
  __shared__ float s_half_max[2][2][kAttnTcRows];               // [tile parity][half][row]: a half's maximum of the tile, for its partner
  __shared__ float s_half_sum[2][kAttnTcRows];                  // the halves' shares of the softmax denominator (end of the kernel)
  constexpr int D = 64, H = 32;                                 // head size; keys of a tile and output dims per thread
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = tid & (kAttnTcRows - 1), half = tid >> 7;     // TMEM lane = row; a warp reads lanes 32 * (warp % 4) ..
  const int h = blockIdx.y, b = blockIdx.z, q0 = blockIdx.x * kAttnTcRows;
  pdl_wait();
  const int q_len_b = p.q_lengths[b];
  const int q_valid = max(0, min(p.q_len, q_len_b));
  if (q_len_b < min_q || q0 >= (p.row_start ? q_valid : p.q_len)) return;          // uniform per CTA
  const int kv_valid = max(0, min(p.kv_len, p.kv_lengths[b]));
  const long long off = p.offsets[b];
  const long long q_base = p.row_start ? p.row_start[b] * p.q_si : b * p.q_sb;
  const long long o_base = p.row_start ? p.row_start[b] * p.o_si : b * p.o_sb;
  const int qi = q0 + row;                                      // this thread's query row
  const bool active = qi < q_valid;
  const int last_query = min(q_valid, q0 + kAttnTcRows) - 1;
  long long bound = p.causal ? off + last_query + 1 : (long long)kv_valid;
  const int key_end = last_query < q0 || bound < 0 ? 0 : int(bound < (long long)kv_valid ? bound : (long long)kv_valid);
  const long long my_last = p.causal ? off + qi : (long long)kv_valid - 1;

  if (tid == 0) { mbar_init(&s_done, 1); mbar_init(&pv_done, 1); mbar_fence_init(); }
  constexpr uint32_t kTmemCols = 256;                           // S (2 x 64 columns, alternating) at 0 and 64, PV at 128
  if (warp == 0) tmem_alloc(&tmem_slot, kTmemCols);
  // Q rows -> K-major core matrices: (k chunk kc, row group mg) at (kc * 16 + mg) * 128, row m % 8 at 16 bytes each
  {
    const __half* src = p.q + q_base + h * p.q_sh + (long long)qi * p.q_si;
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
      const int kc = half * (D / 16) + c;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (active) v = load8<true>(src + kc * 8);
      *reinterpret_cast<uint4*>(qs + (kc * (kAttnTcRows / 8) + (row >> 3)) * 128 + (row & 7) * 16) = v;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t lane_addr = tmem_base + (uint32_t(32 * (warp & 3)) << 16) + uint32_t(H * half);
  // instruction descriptors: fp32 accumulate, fp16 operands, M = 128, N = 64; S: both K-major; PV: B (= V) MN-major
  constexpr uint32_t idesc_s = (1u << 4) | (uint32_t(kAttnTcKeys >> 3) << 17) | (uint32_t(kAttnTcRows >> 4) << 24);
  constexpr uint32_t idesc_pv = idesc_s | (1u << 16);

  float m = -CUDART_INF_F, l = 0.f, o[H];                       // l: this half's share of the denominator
#pragma unroll
  for (int d = 0; d < H; ++d) o[d] = 0.f;
  uint32_t phase_s = 0, phase_pv = 0;
  bool ok = true;

  // K and V tile `t` (keys 64 t ..) -> ring slot t % 3, asynchronously (16-byte copies straight into the operand layouts,
  // zeros past key_end): 64 keys x 8 chunks of 8 values, 2 chunks per thread each.  One commit group per call, also for a
  // tile past the end (empty), so that the group count does not depend on the data.
  const int tiles = (key_end + kAttnTcKeys - 1) / kAttnTcKeys;
  auto issue_tile = [&](int t) {
    if (t < tiles) {
      const int k0 = t * kAttnTcKeys, slot = t % L::kRing;
      const uint32_t kdst = smem_u32(ks + slot * L::kTile), vdst = smem_u32(vs + slot * L::kTile);
#pragma unroll
      for (int it = 0; it < kAttnTcKeys * 8 / kAttnTcThreads; ++it) {
        const int idx = tid + kAttnTcThreads * it, r = idx >> 3, c = idx & 7, key = k0 + r;
        const bool inside = key < key_end;
        const size_t at = inside ? kv.offset(b, h, key) + c * 8 : 0;
        // K as the B operand of S, K-major: (d chunk c, key group r / 8) at (c * 8 + r / 8) * 128, key r % 8 at 16 bytes each
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                     ::"r"(kdst + uint32_t((c * (kAttnTcKeys / 8) + (r >> 3)) * 128 + (r & 7) * 16)), "l"(kv.k + at), "r"(inside ? 16 : 0) : "memory");
        // V as the B operand of PV, MN-major (d contiguous): (key group r / 8, d chunk c) at ((r / 8) * 8 + c) * 128, key r % 8
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                     ::"r"(vdst + uint32_t(((r >> 3) * (D / 8) + c) * 128 + (r & 7) * 16)), "l"(kv.v + at), "r"(inside ? 16 : 0) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // S of tile t into accumulator t & 1 (one thread; the tile's K has landed and the accumulator has been read)
  auto issue_s = [&](int t) {
    tc_fence_after();
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint64_t da = tc_desc(smem_u32(qs) + kk * 2 * (kAttnTcRows / 8) * 128, (kAttnTcRows / 8) * 128, 128);
      const uint64_t db = tc_desc(smem_u32(ks + (t % L::kRing) * L::kTile) + kk * 2 * (kAttnTcKeys / 8) * 128, (kAttnTcKeys / 8) * 128, 128);
      tc_mma_f16(tmem_base + uint32_t(64 * (t & 1)), da, db, idesc_s, kk > 0 ? 1u : 0u);
    }
    tc_commit(&s_done);
  };
  // O = O * alpha + PV of the tile whose contraction was issued last (alpha is that tile's rescaling factor)
  auto fold_pv = [&](float alpha) {
    if (ok) ok = mbar_wait(&pv_done, phase_pv, kStatusMmaTimeout);
    ok = __all_sync(0xffffffffu, ok);                         // tcgen05.ld is warp-collective
    phase_pv ^= 1u;
    tc_fence_after();
    if (ok) {
      float pv[H];
      tmem_load32(lane_addr + 128u, pv);
#pragma unroll
      for (int d = 0; d < H; ++d) o[d] = o[d] * alpha + pv[d];
    }
  };

  if (tiles > 0) {
    issue_tile(0);
    issue_tile(1);
    asm volatile("cp.async.wait_group 1;" ::: "memory");       // tile 0
    fence_async_smem();
    __syncthreads();
    if (tid == 0) issue_s(0);
  }
  float alpha_pending = 1.f;
  for (int t = 0; t < tiles; ++t) {
    const int k0 = t * kAttnTcKeys + H * half;                 // first key of this thread's half of the tile
    if (ok) ok = mbar_wait(&s_done, phase_s, kStatusMmaTimeout);
    ok = __all_sync(0xffffffffu, ok);
    phase_s ^= 1u;
    tc_fence_after();
    float s[H];
    if (ok) tmem_load32(lane_addr + uint32_t(64 * (t & 1)), s);
    // ---- this half's maximum of the tile goes to the partner through shared memory; the barrier that publishes it is
    // the one the next tile's S needs anyway
    float tile_max = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < H; ++j) {
      const int key = k0 + j;
      const bool visible = ok && active && key < key_end && (long long)key <= my_last;
      s[j] = visible ? s[j] * rsqrtf(float(D)) : -CUDART_INF_F;
      tile_max = fmaxf(tile_max, s[j]);
    }
    s_half_max[t & 1][half][row] = tile_max;
    // ---- the next tile's S runs on the tensor cores while this tile's softmax runs on the CUDA cores
    asm volatile("cp.async.wait_group 0;" ::: "memory");       // tile t + 1, requested one step ago
    fence_async_smem();
    tc_fence_before();
    __syncthreads();                                          // ... by every thread; accumulator (t + 1) & 1 has been read (step t - 1)
    if (tid == 0 && t + 1 < tiles) issue_s(t + 1);
    // ---- online softmax of this row (both halves compute the same maximum and rescaling factor)
    const float next = fmaxf(m, fmaxf(tile_max, s_half_max[t & 1][half ^ 1][row]));
    const float alpha = next > -CUDART_INF_F ? __expf(m - next) : 1.f;      // nothing seen yet: state stays empty
    float tile_sum = 0.f;
    uint32_t packed[H / 2];
#pragma unroll
    for (int j = 0; j < H; j += 2) {
      const float p0 = s[j] > -CUDART_INF_F ? __expf(s[j] - next) : 0.f;
      const float p1 = s[j + 1] > -CUDART_INF_F ? __expf(s[j + 1] - next) : 0.f;
      tile_sum += p0 + p1;
      const __half2 h2 = __floats2half2_rn(p0, p1);
      packed[j / 2] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    l = l * alpha + tile_sum;
    m = next;
    // ---- the previous tile's PV: it frees the P buffer, the PV accumulator and ring slot (t - 1) % 3 = (t + 2) % 3
    if (t > 0) fold_pv(alpha_pending);
    alpha_pending = alpha;
    issue_tile(t + 2);
    // P as the A operand of PV, K-major: (key chunk kc, row group) at (kc * 16 + row / 8) * 128, row % 8; this half's four chunks
#pragma unroll
    for (int c = 0; c < H / 8; ++c)
      *reinterpret_cast<uint4*>(ps + ((half * (H / 8) + c) * (kAttnTcRows / 8) + (row >> 3)) * 128 + (row & 7) * 16) =
          make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();                                          // P is complete; every thread has read the PV accumulator
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < kAttnTcKeys / 16; ++kk) {
        const uint64_t da = tc_desc(smem_u32(ps) + kk * 2 * (kAttnTcRows / 8) * 128, (kAttnTcRows / 8) * 128, 128);
        const uint64_t db = tc_desc(smem_u32(vs + (t % L::kRing) * L::kTile) + kk * 2 * (D / 8) * 128, (D / 8) * 128, 128);
        tc_mma_f16(tmem_base + 128u, da, db, idesc_pv, kk > 0 ? 1u : 0u);
      }
      tc_commit(&pv_done);
    }
  }
  if (tiles > 0) fold_pv(alpha_pending);
  asm volatile("cp.async.wait_group 0;" ::: "memory");         // only empty groups can be left
  pdl_launch_dependents();
  // the denominator is the sum of the two halves' shares (both were rescaled by the same factors)
  s_half_sum[half][row] = l;
  __syncthreads();
  l = s_half_sum[0][row] + s_half_sum[1][row];
  // Padded layout (operator ABI): rows past the request's length are written as zeros.  Packed rows (row_start given): a
  // row past the request's length belongs to another request and is left alone.
  if (ok && (p.row_start ? active : qi < p.q_len)) {
    __half* dst = p.out + o_base + h * p.o_sh + (long long)qi * p.o_si + H * half;
#pragma unroll
    for (int c = 0; c < H / 8; ++c) {
      uint4 packed8;
      __half* hh = reinterpret_cast<__half*>(&packed8);
#pragma unroll
      for (int e = 0; e < 8; ++e) hh[e] = f2h(l > 0.f && active ? o[c * 8 + e] / l : 0.f);
      if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) *reinterpret_cast<uint4*>(dst + c * 8) = packed8;
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[c * 8 + e] = hh[e];
      }
    }
  }
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

}  // namespace tib
