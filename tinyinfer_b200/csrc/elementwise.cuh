// Row-wise LayerNorm / softmax and element-wise tanh-GELU on fp16 rows (fp32 math).
//
// The reference sums a row with 256 threads (thread t takes columns t, t+256, ... in order)
// followed by a halving tree over the 256 partials (block_sum, kernels/src/cuda/tc/
// elementwise.cu:7-14).  Here ONE warp owns a row and replays that exact order: lane L holds
// the partials of the virtual threads L, L+32, ..., L+224; tree levels 128/64/32 fold
// registers inside a lane, levels 16..1 are shuffles.  The fp32 sums -- and therefore mean,
// variance and every output -- carry the same bits as the reference while a 768-wide row costs
// one warp instead of a 256-thread block with eight barriers.
#pragma once
#include <math_constants.h>

#include "common.cuh"

namespace tib {

// Sum of v[j] (virtual thread lane + 32*j) over all 256 virtual threads, reference order.
__device__ __forceinline__ float tree256(float (&v)[8]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] += v[j + 4];
  v[0] += v[2]; v[1] += v[3];
  float x = v[0] + v[1];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) x += __shfl_down_sync(0xffffffffu, x, d);
  return __shfl_sync(0xffffffffu, x, 0);
}

// Mean and 1/sqrt(var+eps) of one row held in shared memory as fp32, by one warp (reference norm,
// elementwise.cu:15-24).  Reading from shared memory keeps the replayed summation order cheap: the
// 2 x cols/32 dependent adds of a lane wait on ~30-cycle loads instead of DRAM round trips.
__device__ __forceinline__ float row_value(const float* x, int c) { return x[c]; }
__device__ __forceinline__ float row_value(const __half* x, int c) { return h2f(x[c]); }
template <typename T>
__device__ __forceinline__ void row_stats(const T* x, int cols, float eps, float& mean, float& inv) {
  // v[j] is the partial of virtual thread lane + 32*j: columns lane + 32*j, + 256, + 512, ... added in that
  // order.  The walk goes 256 columns at a time with the eight partials side by side, so eight independent
  // load/add chains are in flight instead of one.
  const int lane = threadIdx.x & 31;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
#pragma unroll 1
  for (int base = lane; base < cols; base += 256) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { const int c = base + 32 * j; if (c < cols) v[j] += row_value(x, c); }
  }
  mean = tree256(v) / cols;
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
#pragma unroll 1
  for (int base = lane; base < cols; base += 256) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { const int c = base + 32 * j; if (c < cols) { const float z = row_value(x, c) - mean; v[j] += z * z; } }
  }
  inv = rsqrtf(tree256(v) / cols + eps);
}

// One warp copies a row of `cols` halves into shared memory as fp32.  Up to four 16-byte loads per lane are issued
// before the first is used; the fp32 values go out as two 16-byte shared stores (a lane's eight floats lie 32 bytes
// from its neighbour's, so 4-byte stores would hit each bank eight times over).
__device__ __forceinline__ void stage_row(const __half* x, float* dst, int cols) {
  const int lane = threadIdx.x & 31;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (cols & 7) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll 1
    for (int c0 = lane * 8; c0 < cols; c0 += 1024) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 256 * u < cols) raw[u] = *reinterpret_cast<const uint4*>(x + c0 + 256 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 256 * u < cols) {
          const __half* h = reinterpret_cast<const __half*>(&raw[u]);
          float4* out = reinterpret_cast<float4*>(dst + c0 + 256 * u);
          out[0] = make_float4(h2f(h[0]), h2f(h[1]), h2f(h[2]), h2f(h[3]));
          out[1] = make_float4(h2f(h[4]), h2f(h[5]), h2f(h[6]), h2f(h[7]));
        }
    }
  } else {
#pragma unroll 1
    for (int c = lane; c < cols; c += 32) dst[c] = h2f(x[c]);
  }
  __syncwarp();
}

constexpr int kLnMaxCols = 4096;     // rows up to this width are staged in shared memory (16 KB per warp)

// grid = ceil(rows / 4), block = 128: one warp per row; dynamic shared memory (for cols <= kLnMaxCols):
// 4 rows of fp32 + gamma and beta as fp16 = 20 * cols bytes.  gamma / beta are parameters, not produced by
// the previous kernel, so they are staged before the dependency wait and their latency is hidden.
__global__ void __launch_bounds__(128)
layernorm_kernel(const __half* x, const int32_t* row_index, const __half* g, const __half* b, __half* y,
                 int rows, int cols, float eps, int early_trigger) {
  trace_event(kTrLayerNorm, 0);
  if (early_trigger) pdl_launch_dependents();
  extern __shared__ __align__(16) float ln_rows[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, row = blockIdx.x * 4 + warp;
  const bool staged = cols <= kLnMaxCols;
  __half* gs = reinterpret_cast<__half*>(ln_rows + size_t(4) * cols);
  __half* bs = gs + cols;
  if (staged) {
#pragma unroll 1
    for (int c = threadIdx.x; c < cols; c += 128) { gs[c] = g[c]; bs[c] = b[c]; }
    __syncthreads();
  }
  pdl_wait();
  trace_event(kTrLayerNorm, 1);
  if (row >= rows) return;
  const __half* xr = x + size_t(row_index ? row_index[row] : row) * cols;   // optional gather of input rows
  __half* yr = y + size_t(row) * cols;
  float mean, inv;
  if (staged) {
    float* xs = ln_rows + size_t(warp) * cols;
    stage_row(xr, xs, cols);
    row_stats(xs, cols, eps, mean, inv);
    pdl_launch_dependents();
    if ((reinterpret_cast<uintptr_t>(yr) & 15) == 0 && (cols & 7) == 0) {
#pragma unroll 1
      for (int c = lane * 8; c < cols; c += 256) {
        // 16-byte shared loads: the row (two of them per lane), gamma and beta (cols is a multiple of 8, so all three are aligned)
        const float4 lo = *reinterpret_cast<const float4*>(xs + c), hi = *reinterpret_cast<const float4*>(xs + c + 4);
        const uint4 graw = *reinterpret_cast<const uint4*>(gs + c), braw = *reinterpret_cast<const uint4*>(bs + c);
        const __half* gh = reinterpret_cast<const __half*>(&graw);
        const __half* bh = reinterpret_cast<const __half*>(&braw);
        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        uint4 packed;
        __half* h = reinterpret_cast<__half*>(&packed);
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = f2h((v[e] - mean) * inv * h2f(gh[e]) + h2f(bh[e]));
        *reinterpret_cast<uint4*>(yr + c) = packed;
      }
    } else {
#pragma unroll 1
      for (int c = lane; c < cols; c += 32) yr[c] = f2h((xs[c] - mean) * inv * h2f(gs[c]) + h2f(bs[c]));
    }
  } else {
    // very wide rows: same arithmetic straight from global memory
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
#pragma unroll 1
      for (int c = lane + 32 * j; c < cols; c += 256) s += h2f(xr[c]);
      v[j] = s;
    }
    mean = tree256(v) / cols;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
#pragma unroll 1
      for (int c = lane + 32 * j; c < cols; c += 256) { const float z = h2f(xr[c]) - mean; s += z * z; }
      v[j] = s;
    }
    inv = rsqrtf(tree256(v) / cols + eps);
    pdl_launch_dependents();
#pragma unroll 1
    for (int c = lane; c < cols; c += 32) yr[c] = f2h((h2f(xr[c]) - mean) * inv * h2f(g[c]) + h2f(b[c]));
  }
}

// Row softmax (reference normalized_exp, elementwise.cu:34-46), one warp per row.
__global__ void __launch_bounds__(128)
softmax_kernel(const __half* x, __half* y, int rows, int cols) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __half* xr = x + size_t(row) * cols;
  __half* yr = y + size_t(row) * cols;
  float top = -CUDART_INF_F;
  for (int c = lane; c < cols; c += 32) top = fmaxf(top, h2f(xr[c]));
  top = warp_max(top);
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float s = 0.f;
    for (int c = lane + 32 * j; c < cols; c += 256) s += expf(h2f(xr[c]) - top);
    v[j] = s;
  }
  const float denom = tree256(v);
  for (int c = lane; c < cols; c += 32) yr[c] = f2h(expf(h2f(xr[c]) - top) / denom);
}

// tanh-GELU (reference gelu, elementwise.cu:28-33); grid-stride, 8 values per thread when the
// buffers are 16-byte aligned.
__global__ void __launch_bounds__(256)
gelu_kernel(const __half* x, __half* y, long long count, int vector_ok) {
  const long long stride = (long long)gridDim.x * blockDim.x, t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long vec = vector_ok ? count / 8 : 0;
  for (long long i = t; i < vec; i += stride) {
    uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    __half* hv = reinterpret_cast<__half*>(&raw);
#pragma unroll
    for (int e = 0; e < 8; ++e) hv[e] = f2h(gelu_tanh(h2f(hv[e])));
    reinterpret_cast<uint4*>(y)[i] = raw;
  }
  for (long long i = vec * 8 + t; i < count; i += stride) y[i] = f2h(gelu_tanh(h2f(x[i])));
}

}  // namespace tib
