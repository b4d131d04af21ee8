// Ragged causal attention over per-request KV histories, fp16 in / fp32 math / fp16 out.
//
// Semantics are the reference's online_attention (kernels/src/cuda/tc/attention.cu:9-57):
// key j is visible to query i of request b when j < min(kv_len, kv_lengths[b]) and
// (!causal || j <= query_offsets[b] + i); the score is q.k * rsqrt(D); the softmax runs on an
// online (max, sum, acc) state in fp32; query rows at or past q_lengths[b] and rows that see no
// key are written as exact zeros.
//
// Two kernels, both HBM/L2-bound streaming kernels with no tensor-core use:
//   attn_tile_kernel     any number of queries per request (prefill, operator ABI): 8 queries
//                        per CTA share 32-key K/V tiles staged in shared memory.
//   attn_decode_kernel   one query per request (decode): the history of one (request, head) is
//                        cut into chunks, one CTA per chunk, K/V read in place with fully
//                        coalesced 16-byte loads (4 keys x 128 B per warp instruction); chunk
//                        results (max, sum, unnormalised acc) go to a scratch buffer and
//                        attn_combine_kernel merges them.  With a single chunk the result is
//                        written directly.
//
// K/V are reached through an accessor: packed [B,H,K,D] tensors (operator ABI) or the paged
// pool of the model runtime (pages of 32 positions, [page][layer][head][32][D], located through
// a per-slot page table), so the cache is read where it lives -- no gather copy.
#pragma once
#include <math_constants.h>

#include "common.cuh"

namespace tib {

constexpr int kPageTokens = 32;

struct KvPacked {
  const __half* k; const __half* v; int heads, kv_len, d;
  __device__ __forceinline__ size_t offset(int b, int h, int key) const {
    return ((size_t(b) * heads + h) * kv_len + key) * d;
  }
  // A 32-key tile (t0 % 32 == 0) is named by a reference that does not depend on the head; its keys follow
  // each other at stride d from tile_offset(ref, b, h).
  __device__ __forceinline__ int tile_ref(int, int t0) const { return t0; }
  __device__ __forceinline__ size_t tile_offset(int ref, int b, int h) const { return offset(b, h, ref); }
  __device__ __forceinline__ int tile_keys(int t0) const { return max(0, min(kPageTokens, kv_len - t0)); }   // keys that exist in memory
};
struct KvPaged {
  const __half* k; const __half* v;       // page pools
  const int32_t* table;                   // [slots][table_pitch] page ids
  const int32_t* slots;                   // [batch] slot of each request
  int table_pitch, layers, layer, heads, d;
  __device__ __forceinline__ size_t offset(int b, int h, int key) const {
    const int page = table[size_t(slots[b]) * table_pitch + (key / kPageTokens)];
    return (((size_t(page) * layers + layer) * heads + h) * kPageTokens + (key % kPageTokens)) * d;
  }
  __device__ __forceinline__ int tile_ref(int b, int t0) const { return table[size_t(slots[b]) * table_pitch + t0 / kPageTokens]; }   // its page
  __device__ __forceinline__ size_t tile_offset(int ref, int, int h) const {
    return ((size_t(ref) * layers + layer) * heads + h) * kPageTokens * d;
  }
  __device__ __forceinline__ int tile_keys(int) const { return kPageTokens; }
};

struct AttnArgs {
  const __half* q; long long q_sb, q_sh, q_si;      // element strides: request, head, query row
  __half* out; long long o_sb, o_sh, o_si;
  const int32_t* row_start;                        // optional: request b starts at row row_start[b] (replaces b*q_sb, b*o_sb)
  const int32_t* q_lengths; const int32_t* kv_lengths; const int32_t* offsets;
  int batch, heads, q_len, kv_len, causal;
  int skip_single;                                 // requests with exactly one query row are left to the decode kernel
  int skip_min_q;                                  // > 0: requests with at least this many query rows are left to the tensor-core kernel
};

// ------------------------------------------------------------------ tiled kernel (Q >= 1)
constexpr int kAttnTileQ = 8, kAttnTileK = 32;

// Eight consecutive halves: one 16-byte load where the tensors allow it (VEC), else element by element -- the operator
// ABI accepts tensors that are only 2-byte aligned (reference validators, tinyinfer_host_validation.hpp).
template <bool VEC>
__device__ __forceinline__ uint4 load8(const __half* src) {
  if (VEC) return *reinterpret_cast<const uint4*>(src);
  uint4 v;
  __half* h = reinterpret_cast<__half*>(&v);
#pragma unroll
  for (int e = 0; e < 8; ++e) h[e] = src[e];
  return v;
}

template <int D, typename KV, bool VEC = true>
__global__ void __launch_bounds__(256)
attn_tile_kernel(const AttnArgs p, const KV kv) {
  constexpr int PITCH = D + 8;                                  // halves; keeps 16-byte row reads conflict-free
  __shared__ __align__(16) __half ks[kAttnTileK][PITCH];
  __shared__ __align__(16) __half vs[kAttnTileK][D];
  __shared__ __align__(16) __half qs[kAttnTileQ][D];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, b = blockIdx.z, qi = blockIdx.x * kAttnTileQ + warp;
  pdl_wait();
  const int q_valid = max(0, min(p.q_len, p.q_lengths[b]));
  if (p.skip_single && p.q_lengths[b] == 1) return;               // uniform per CTA; nothing is written for this request here
  if (p.skip_min_q && p.q_lengths[b] >= p.skip_min_q) return;
  const int kv_valid = max(0, min(p.kv_len, p.kv_lengths[b]));
  const long long off = p.offsets[b];
  const long long q_base = p.row_start ? p.row_start[b] * p.q_si : b * p.q_sb;
  const long long o_base = p.row_start ? p.row_start[b] * p.o_si : b * p.o_sb;
  const bool active = qi < q_valid;
  const int last_query = min(q_valid - 1, int(blockIdx.x) * kAttnTileQ + kAttnTileQ - 1);
  long long bound = p.causal ? off + last_query + 1 : kv_valid;
  const int end = last_query < 0 || bound < 0 ? 0 : int(bound < (long long)kv_valid ? bound : (long long)kv_valid);
  const long long my_last = p.causal ? off + qi : (long long)kv_valid - 1;   // last visible key of this row

  for (int i = lane; i < D / 8; i += 32) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (active) v = load8<VEC>(p.q + q_base + h * p.q_sh + (long long)qi * p.q_si + i * 8);
    *reinterpret_cast<uint4*>(&qs[warp][i * 8]) = v;
  }
  float m = -CUDART_INF_F, l = 0.f, acc[D / 32];
#pragma unroll
  for (int z = 0; z < D / 32; ++z) acc[z] = 0.f;

  for (int k0 = 0; k0 < end; k0 += kAttnTileK) {
    __syncthreads();
    for (int i = tid; i < kAttnTileK * (D / 8); i += 256) {
      const int r = i / (D / 8), c = i % (D / 8), key = k0 + r;
      uint4 kk = make_uint4(0, 0, 0, 0), vv = kk;
      if (key < end) {
        const size_t o = kv.offset(b, h, key) + c * 8;
        kk = load8<VEC>(kv.k + o);
        vv = load8<VEC>(kv.v + o);
      }
      *reinterpret_cast<uint4*>(&ks[r][c * 8]) = kk;
      *reinterpret_cast<uint4*>(&vs[r][c * 8]) = vv;
    }
    __syncthreads();
    const int key = k0 + lane;
    const bool visible = active && key < end && (long long)key <= my_last;
    float score = 0.f;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      const uint4 qq = *reinterpret_cast<const uint4*>(&qs[warp][c * 8]);
      const uint4 kk = *reinterpret_cast<const uint4*>(&ks[lane][c * 8]);
      const __half2* q2 = reinterpret_cast<const __half2*>(&qq);
      const __half2* k2 = reinterpret_cast<const __half2*>(&kk);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        score = fma_f16(score, __low2half(q2[e]), __low2half(k2[e]));
        score = fma_f16(score, __high2half(q2[e]), __high2half(k2[e]));
      }
    }
    score = visible ? score * rsqrtf(float(D)) : -CUDART_INF_F;
    const float tile_max = warp_max(score);
    if (tile_max > -CUDART_INF_F) {                              // warp-uniform
      const float next = fmaxf(m, tile_max);
      const float alpha = expf(m - next);                        // exp(-inf) = 0 on the first tile
      const float pr = visible ? expf(score - next) : 0.f;
      l = l * alpha + warp_sum(pr);
#pragma unroll
      for (int z = 0; z < D / 32; ++z) acc[z] *= alpha;
      for (int j = 0; j < kAttnTileK; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pr, j);
#pragma unroll
        for (int z = 0; z < D / 32; ++z) acc[z] = fmaf(pj, h2f(vs[j][lane + 32 * z]), acc[z]);
      }
      m = next;
    }
  }
  pdl_launch_dependents();
  // Padded layout: rows past the request's length are written as zeros.  Packed rows (row_start
  // given): a row past the request's length belongs to another request and is left alone.
  if (p.row_start ? active : qi < p.q_len) {
    __half* o = p.out + o_base + h * p.o_sh + (long long)qi * p.o_si;
#pragma unroll
    for (int z = 0; z < D / 32; ++z) o[lane + 32 * z] = f2h(l > 0.f ? acc[z] / l : 0.f);
  }
}

// ------------------------------------------------------------------ decode kernel (Q == 1)
constexpr int kDecodeWarps = 4;          // chunked launches: 128 keys per CTA pass

struct DecodeArgs {
  const __half* q; long long q_sb, q_sh;            // one query row per request
  __half* out; long long o_sb, o_sh;
  const int32_t* kv_lengths;                         // visible keys of each request (its new token included)
  float* part_acc;                                   // scratch fp32 [batch][heads][chunks][D]
  float* part_ml;                                    // scratch fp32 [batch][heads][chunks][2]  (max, sum)
  int* counters;                                     // optional int [batch][heads], all zero between launches: when given, the
                                                     // last chunk CTA of a (request, head) merges the partials itself
  int batch, heads, chunk, chunks;                   // keys per CTA; grid.x
  int kv_len;                                        // keys that exist in memory per request: lengths are clamped to it
  // early: kv_lengths, the page table and every key but each request's newest one were written before the
  // kernel ahead of this one started, so they are read before the dependency wait (their latency then hides
  // behind that kernel); the newest key and the query are read after it.
  // Mixed passes of the model runtime (prompts and single tokens in one call): request b's row is row_start[b] instead
  // of b, and requests whose q_lengths[b] is not 1 are left to the tile kernel.  Both null in a pure decode step.
  const int32_t* row_start; const int32_t* q_lengths;
  int early;
  int early_trigger;                                 // release the next kernel's launch before this one's own wait
};

// grid = (chunks, heads, batch), block = 32 * W.
template <int D, typename KV, int W = kDecodeWarps>
__global__ void __launch_bounds__(W * 32)
attn_decode_kernel(const DecodeArgs p, const KV kv) {
  trace_event(kTrAttnDecode, 0);
  static_assert(D == 64 || D == 128, "head_dim");
  constexpr int DP = D / 8;                           // lanes that share one key (8 dims each)
  constexpr int KPS = 32 / DP;                        // keys per warp instruction
  constexpr int STEPS = 32 / KPS;                     // instructions per 32-key tile
  __shared__ float s_acc[W][D];
  __shared__ float s_ml[W][2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int dp = lane % DP, ksub = lane / DP;
  const int h = blockIdx.y, b = blockIdx.z;
  const int begin = blockIdx.x * p.chunk, t_first = begin + warp * 32;
  uint4 kreg[STEPS], vreg[STEPS];
  // keys [lo, hi) of the tile at t0 into this lane's registers; the rest stay as they are
  auto load_tile = [&](size_t base, int t0, int lo, int hi) {
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
      const int key = t0 + i * KPS + ksub;
      if (key >= lo && key < hi) {
        const size_t o = base + size_t(i * KPS + ksub) * D + dp * 8;
        kreg[i] = *reinterpret_cast<const uint4*>(kv.k + o);
        vreg[i] = *reinterpret_cast<const uint4*>(kv.v + o);
      }
    }
  };
#pragma unroll
  for (int i = 0; i < STEPS; ++i) { kreg[i] = make_uint4(0, 0, 0, 0); vreg[i] = kreg[i]; }
  // Early reads: the length, the references (pages) of this warp's first four tiles, and the first tile's keys.
  constexpr int kRefs = 4;
  int len = 0, refs[kRefs];
#pragma unroll
  for (int r = 0; r < kRefs; ++r) refs[r] = 0;
  if (p.early) {
    len = max(0, min(p.kv_lengths[b], p.kv_len));
    const int end_early = min(len, begin + p.chunk);
#pragma unroll
    for (int r = 0; r < kRefs; ++r) if (t_first + r * W * 32 < end_early) refs[r] = kv.tile_ref(b, t_first + r * W * 32);
    if (t_first < end_early) load_tile(kv.tile_offset(refs[0], b, h), t_first, t_first, min(end_early, len - 1));
  }
  if (p.early_trigger) pdl_launch_dependents();
  pdl_wait();
  trace_event(kTrAttnDecode, 1);
  if (!p.early) len = max(0, min(p.kv_lengths[b], p.kv_len));
  const int end = min(len, begin + p.chunk);
  if (begin >= end && blockIdx.x != 0) return;        // nothing to do for this chunk (uniform per CTA)

  const uint4 qraw = *reinterpret_cast<const uint4*>(p.q + b * p.q_sb + h * p.q_sh + dp * 8);
  const __half2* q2 = reinterpret_cast<const __half2*>(&qraw);
  float m = -CUDART_INF_F, l = 0.f, acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;

  int it = 0;
  for (int t0 = t_first; t0 < end; t0 += W * 32, ++it) {
    if (it == 0 && p.early) {
      load_tile(kv.tile_offset(refs[0], b, h), t0, max(t0, len - 1), end);   // the newest key, if this tile holds it
    } else {
#pragma unroll
      for (int i = 0; i < STEPS; ++i) { kreg[i] = make_uint4(0, 0, 0, 0); vreg[i] = kreg[i]; }
      int ref;
      if (p.early && it < kRefs) ref = it == 1 ? refs[1] : it == 2 ? refs[2] : refs[3];
      else ref = kv.tile_ref(b, t0);
      load_tile(kv.tile_offset(ref, b, h), t0, t0, end);
    }
    float sc[STEPS], tile_max = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
      const __half2* k2 = reinterpret_cast<const __half2*>(&kreg[i]);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        d = fma_f16(d, __low2half(q2[e]), __low2half(k2[e]));
        d = fma_f16(d, __high2half(q2[e]), __high2half(k2[e]));
      }
#pragma unroll
      for (int x = 1; x < DP; x <<= 1) d += __shfl_xor_sync(0xffffffffu, d, x);
      const int key = t0 + i * KPS + ksub;
      sc[i] = key < end ? d * rsqrtf(float(D)) : -CUDART_INF_F;
      tile_max = fmaxf(tile_max, sc[i]);
    }
#pragma unroll
    for (int x = DP; x < 32; x <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, x));
    const float next = fmaxf(m, tile_max);              // the tile holds at least one key
    const float alpha = expf(m - next);
    l *= alpha;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= alpha;
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
      const float pr = expf(sc[i] - next);               // exp(-inf) = 0 for keys past the end
      l += pr;
      const __half2* v2 = reinterpret_cast<const __half2*>(&vreg[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] = fmaf(pr, __low2float(v2[e]), acc[2 * e]);
        acc[2 * e + 1] = fmaf(pr, __high2float(v2[e]), acc[2 * e + 1]);
      }
    }
    m = next;
  }
  // key sub-groups of the warp share `m`; add their sums
#pragma unroll
  for (int x = DP; x < 32; x <<= 1) {
    l += __shfl_xor_sync(0xffffffffu, l, x);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], x);
  }
  if (lane < DP) {
#pragma unroll
    for (int e = 0; e < 8; ++e) s_acc[warp][dp * 8 + e] = acc[e];
    if (lane == 0) { s_ml[warp][0] = m; s_ml[warp][1] = l; }
  }
  __syncthreads();
  pdl_launch_dependents();
  if (tid < D) {
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < W; ++w) mm = fmaxf(mm, s_ml[w][0]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float f = s_ml[w][0] > -CUDART_INF_F ? expf(s_ml[w][0] - mm) : 0.f;
      ll += s_ml[w][1] * f; aa += s_acc[w][tid] * f;
    }
    if (p.chunks == 1) {
      p.out[b * p.o_sb + h * p.o_sh + tid] = f2h(ll > 0.f ? aa / ll : 0.f);
    } else {
      const size_t slot = (size_t(b) * p.heads + h) * p.chunks + blockIdx.x;
      p.part_acc[slot * D + tid] = aa;
      if (tid == 0) { p.part_ml[slot * 2] = mm; p.part_ml[slot * 2 + 1] = ll; }
    }
  }
  if (p.chunks > 1 && p.counters) {
    // Merge in the CTA that finishes last: partials are published (fence), a ticket is taken, and the
    // holder of the last ticket reads everybody's partials.  The counter is left at zero again.
    __shared__ int s_last;
    const int used = max(1, min(p.chunks, (len + p.chunk - 1) / p.chunk));
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* counter = p.counters + b * p.heads + h;
      s_last = atomicAdd(counter, 1) == used - 1;
      if (s_last) *counter = 0;
    }
    __syncthreads();
    if (s_last && tid < D) {
      __threadfence();
      const size_t base = (size_t(b) * p.heads + h) * p.chunks;
      float mm = -CUDART_INF_F;
      for (int c = 0; c < used; ++c) mm = fmaxf(mm, __ldcg(&p.part_ml[(base + c) * 2]));
      float ll = 0.f, aa = 0.f;
      for (int c = 0; c < used; ++c) {
        const float mc = __ldcg(&p.part_ml[(base + c) * 2]);
        const float f = mc > -CUDART_INF_F ? expf(mc - mm) : 0.f;
        ll += __ldcg(&p.part_ml[(base + c) * 2 + 1]) * f;
        aa += __ldcg(&p.part_acc[(base + c) * D + tid]) * f;
      }
      p.out[b * p.o_sb + h * p.o_sh + tid] = f2h(ll > 0.f ? aa / ll : 0.f);
    }
  }
}

// ------------------------------------------------------------------ decode kernel, whole history per CTA
// grid = (heads, batch), block = 256 (8 warps), dynamic shared memory = 8 warps x (K tile + V tile) = 64 KB for D = 64,
// so three CTAs share an SM and a 32-request x 12-head step is resident at once.  Warp w owns tiles w, w+8, ...
// of 32 keys; a tile is contiguous in memory (a cache page, or 32 rows of a packed tensor) and arrives by two
// bulk asynchronous copies that one lane issues and the warp awaits on its own mbarrier -- the data in flight
// lives in shared memory, not in registers.  With `early` the first tile, the length and the page numbers are
// requested ahead of the dependency wait; the newest key, which the kernel before this one writes, is then
// fetched again after the wait and patched into the tile.
constexpr int kStagedWarps = 8;
template <int D> constexpr int staged_smem_bytes() { return kStagedWarps * 2 * kPageTokens * D * 2 + 64; }

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int D, typename KV>
__global__ void __launch_bounds__(kStagedWarps * 32)
attn_decode_staged_kernel(const DecodeArgs p, const KV kv) {
  trace_event(kTrAttnDecode, 0);
  static_assert(D == 64, "head_dim");
  constexpr int W = kStagedWarps, DP = D / 8, KPS = 32 / DP, STEPS = 32 / KPS, kTileBytes = kPageTokens * D * 2;
  extern __shared__ __align__(128) uint8_t staged_smem[];
  __shared__ float s_acc[W][D];
  __shared__ float s_ml[W][2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int dp = lane % DP, ksub = lane / DP;
  const int h = blockIdx.x, b = blockIdx.y;
  __half* k_tile = reinterpret_cast<__half*>(staged_smem + size_t(warp) * 2 * kTileBytes);
  __half* v_tile = k_tile + kPageTokens * D;
  uint64_t* bar = reinterpret_cast<uint64_t*>(staged_smem + size_t(W) * 2 * kTileBytes) + warp;
  if (lane == 0) { mbar_init(bar, 1); mbar_fence_init(); }
  __syncwarp();

  // lane 0: request tile `t0` (reference `ref`) into this warp's buffers
  auto request = [&](int ref, int t0) {
    const uint32_t bytes = uint32_t(kv.tile_keys(t0)) * D * 2;
    const size_t o = kv.tile_offset(ref, b, h);
    mbar_expect_tx(bar, 2 * bytes);
    bulk_load(k_tile, kv.k + o, bytes, bar);
    bulk_load(v_tile, kv.v + o, bytes, bar);
  };
  constexpr int kRefs = 4;
  int len = 0, refs[kRefs] = {0, 0, 0, 0};
  const int t_first = warp * 32;
  bool requested = false;
  if (p.early) {
    len = max(0, min(p.kv_lengths[b], p.kv_len));
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < kRefs; ++r) if (t_first + r * W * 32 < len) refs[r] = kv.tile_ref(b, t_first + r * W * 32);
      if (t_first < len) { request(refs[0], t_first); requested = true; }
    }
  }
  if (p.early_trigger) pdl_launch_dependents();
  pdl_wait();
  trace_event(kTrAttnDecode, 1);
  if (!p.early) len = max(0, min(p.kv_lengths[b], p.kv_len));
  if (p.q_lengths && p.q_lengths[b] != 1) return;      // uniform per CTA (never combined with `early`: nothing is in flight)
  const long long row = p.row_start ? p.row_start[b] : b;

  const uint4 qraw = *reinterpret_cast<const uint4*>(p.q + row * p.q_sb + h * p.q_sh + dp * 8);
  const __half2* q2 = reinterpret_cast<const __half2*>(&qraw);
  float m = -CUDART_INF_F, l = 0.f, acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  bool ok = true;

  int it = 0;
  for (int t0 = t_first; t0 < len; t0 += W * 32, ++it) {
    if (lane == 0 && ok && !(it == 0 && requested)) {
      const int ref = (p.early && it < kRefs) ? (it == 0 ? refs[0] : it == 1 ? refs[1] : it == 2 ? refs[2] : refs[3]) : kv.tile_ref(b, t0);
      request(ref, t0);
    }
    if (ok) ok = mbar_wait(bar, uint32_t(it) & 1u, kStatusTmaTimeout);
    if (p.early && it == 0 && len - 1 >= t0 && len - 1 < t0 + 32) {
      // the newest key was (re)written by the kernel ahead of this one: fetch it again, now that it is complete
      const int j = len - 1 - t0;
      if (lane < 2 * DP) {
        const int ref = __shfl_sync((1u << (2 * DP)) - 1u, refs[0], 0);
        const size_t o = kv.tile_offset(ref, b, h) + size_t(j) * D + (lane % DP) * 8;
        const uint4 fresh = *reinterpret_cast<const uint4*>((lane < DP ? kv.k : kv.v) + o);
        *reinterpret_cast<uint4*>((lane < DP ? k_tile : v_tile) + j * D + (lane % DP) * 8) = fresh;
      }
      __syncwarp();
    }
    float sc[STEPS], tile_max = -CUDART_INF_F;
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
      sc[i] = (key < len && ok) ? d * rsqrtf(float(D)) : -CUDART_INF_F;
      tile_max = fmaxf(tile_max, sc[i]);
    }
#pragma unroll
    for (int x = DP; x < 32; x <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, x));
    if (tile_max > -CUDART_INF_F) {                      // warp-uniform; false only after a failed copy
      const float next = fmaxf(m, tile_max);
      const float alpha = expf(m - next);
      l *= alpha;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= alpha;
#pragma unroll
      for (int i = 0; i < STEPS; ++i) {
        const int j = i * KPS + ksub;
        if (t0 + j < len) {                               // memory past the history is not ours to interpret
          const float pr = expf(sc[i] - next);
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
    fence_async_smem();                                   // this warp's reads and writes of the tile, before the next copy
    __syncwarp();                                         // every lane is done with the tile before it is overwritten
  }
#pragma unroll
  for (int x = DP; x < 32; x <<= 1) {
    l += __shfl_xor_sync(0xffffffffu, l, x);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], x);
  }
  if (lane < DP) {
#pragma unroll
    for (int e = 0; e < 8; ++e) s_acc[warp][dp * 8 + e] = acc[e];
    if (lane == 0) { s_ml[warp][0] = m; s_ml[warp][1] = l; }
  }
  __syncthreads();
  if (!p.early_trigger) pdl_launch_dependents();
  if (tid < D) {
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < W; ++w) mm = fmaxf(mm, s_ml[w][0]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float f = s_ml[w][0] > -CUDART_INF_F ? expf(s_ml[w][0] - mm) : 0.f;
      ll += s_ml[w][1] * f; aa += s_acc[w][tid] * f;
    }
    p.out[row * p.o_sb + h * p.o_sh + tid] = f2h(ll > 0.f ? aa / ll : 0.f);
  }
}

// grid = (heads, batch), block = D.  Merges the chunk partials of one (request, head).
template <int D>
__global__ void __launch_bounds__(D)
attn_combine_kernel(const DecodeArgs p) {
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  pdl_wait();
  const int len = max(0, min(p.kv_lengths[b], p.kv_len));
  const int used = max(1, min(p.chunks, (len + p.chunk - 1) / p.chunk));
  const size_t base = (size_t(b) * p.heads + h) * p.chunks;
  float mm = -CUDART_INF_F;
  for (int c = 0; c < used; ++c) mm = fmaxf(mm, p.part_ml[(base + c) * 2]);
  float ll = 0.f, aa = 0.f;
  for (int c = 0; c < used; ++c) {
    const float mc = p.part_ml[(base + c) * 2];
    const float f = mc > -CUDART_INF_F ? expf(mc - mm) : 0.f;
    ll += p.part_ml[(base + c) * 2 + 1] * f;
    aa += p.part_acc[(base + c) * D + tid] * f;
  }
  pdl_launch_dependents();
  p.out[b * p.o_sb + h * p.o_sh + tid] = f2h(ll > 0.f ? aa / ll : 0.f);
}

}  // namespace tib
