// Small kernels that tie the GPT-2 layers together in the model runtime: token+position
// embedding and the greedy argmax (K/V placement is an epilogue of the QKV projection).  Rows are packed
// (no padding rows): row r belongs to request row_req[r] and sits at absolute position
// row_pos[r] of that request.
#pragma once
#include "attention.cuh"
#include "common.cuh"

namespace tib {

// x[r,:] = fp16(float(wte[id]) + float(wpe[pos]))  (reference embed, llm/src/runtime.cu:25-30).
__global__ void __launch_bounds__(256)
embed_kernel(const int32_t* ids, const int32_t* row_pos, const __half* wte, const __half* wpe,
             __half* x, int rows, int hidden, int vocab) {
  trace_event(kTrEmbed, 0);
  pdl_wait();
  const int chunks = hidden / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)rows * chunks;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / chunks), c = int(i % chunks) * 8;
    uint4 a = *reinterpret_cast<const uint4*>(wte + size_t(max(0, min(ids[r], vocab - 1))) * hidden + c);   // never an address outside the table
    const uint4 b = *reinterpret_cast<const uint4*>(wpe + size_t(row_pos[r]) * hidden + c);
    __half* ah = reinterpret_cast<__half*>(&a);
    const __half* bh = reinterpret_cast<const __half*>(&b);
#pragma unroll
    for (int e = 0; e < 8; ++e) ah[e] = f2h(h2f(ah[e]) + h2f(bh[e]));
    *reinterpret_cast<uint4*>(x + size_t(r) * hidden + c) = a;
  }
  pdl_launch_dependents();
}

// Greedy argmax of fp32 logits, lowest id on ties (reference argmax, llm/src/runtime.cu:59-66).
// grid = (rows, segments), block = 256.  The winner of row r (largest value, lowest index among equals)
// goes to out[(*step) * rows + r] (step = 0 when `step` is null) and, when `feedback` is non-null, to
// feedback[r] as the next step's input id.  With several segments per row each CTA scans one piece and
// publishes (value, index) packed into one 64-bit word through atomicMax on best[r]; the CTA that takes
// the last ticket of the row writes the result and leaves best[r] and tickets[r] at zero again.
// `best` / `tickets`: rows words each, zero before the first launch; unused with one segment.
__global__ void __launch_bounds__(256)
argmax_kernel(const float* logits, long long pitch, int cols, int32_t* out, int32_t* feedback, const int32_t* step,
              unsigned long long* best, unsigned int* tickets) {
  trace_event(kTrArgmax, 0);
  __shared__ float best_v[8];
  __shared__ int best_i[8];
  const int r = blockIdx.x, segments = gridDim.y;
  const int per = ((cols + segments - 1) / segments + 3) & ~3;
  const int begin = blockIdx.y * per, end = min(cols, begin + per);
  const float* row = logits + (long long)r * pitch;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  pdl_wait();
  trace_event(kTrArgmax, 1);
  float bv = -CUDART_INF_F; int bi = 0x7fffffff;
  auto take = [&](float v, int c) { if (v > bv || (v == bv && c < bi)) { bv = v; bi = c; } };
  if (vec) {
    for (int c = begin + threadIdx.x * 4; c < end; c += 1024) {
      if (c + 3 < end) {
        const float4 v = *reinterpret_cast<const float4*>(row + c);
        take(v.x, c); take(v.y, c + 1); take(v.z, c + 2); take(v.w, c + 3);
      } else {
        for (int e = c; e < end; ++e) take(row[e], e);
      }
    }
  } else {
    for (int c = begin + threadIdx.x; c < end; c += 256) take(row[c], c);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
  __syncthreads();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
    bool write = true;
    if (segments > 1) {
      if (bi != 0x7fffffff) atomicMax(best + r, argmax_pack(bv, bi));
      __threadfence();
      write = atomicAdd(tickets + r, 1u) == unsigned(segments - 1);
      if (write) {
        __threadfence();
        const unsigned long long key = atomicExch(best + r, 0ull);
        bi = key ? int(0xffffffffu - uint32_t(key)) : 0x7fffffff;
        tickets[r] = 0;
      }
    }
    if (write) {
      out[(step ? size_t(*step) * gridDim.x : 0) + r] = bi;
      // A row without any comparable logit (all NaN) yields INT_MAX as in the reference, whose host then rejects it as an
      // invalid token.  Here the next step may read the id on the device, so it gets a valid one and the status word
      // makes the host poison the model.
      if (feedback) feedback[r] = bi < cols ? bi : 0;
      if (bi >= cols) report(kStatusNoToken);
    }
  }
}

// Weights [k][ld] -> slab-major tiles [ceil(n/128)][slab_rows][128] with zero fill; one thread per 16 output bytes.
__global__ void retile_i8_kernel(const int8_t* src, long long ld, int k, int n, int8_t* dst, int slab_rows, long long chunks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= chunks) return;
  const int c16 = int(i % 8);
  const long long r = i / 8;
  const int row = int(r % slab_rows), slab = int(r / slab_rows);
  int8_t v[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const int col = slab * 128 + c16 * 16 + e;
    v[e] = row < k && col < n ? src[(long long)row * ld + col] : int8_t(0);
  }
  *reinterpret_cast<uint4*>(dst + i * 16) = *reinterpret_cast<const uint4*>(v);
}

// ---- per-output-channel symmetric INT8 quantiser (reference specification: llm/quantization.py, backend/host_codec.cpp:
// scale[c] = float(double(max_r |w[r][c]|) / 127.0), or 1 for an all-zero column; q = clip(round_half_even(double(w) /
// double(scale)), -127, 127)).  Three launches: column maxima (bit patterns of non-negative floats order like unsigned
// integers, so atomicMax on them is exact), scales, quantisation in fp64 exactly as the host codec computes it.
// flag: set to 1 when an input is NaN or infinite (the host codec rejects such input; here the outputs are then unspecified).
__global__ void quant_absmax_kernel(const __half* w, long long rows, int cols, unsigned int* max_bits, int* flag, int rows_per_block) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const long long r0 = (long long)blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  if (c >= cols) return;
  float best = 0.f; bool bad = false;
  for (long long r = r0; r < r1; ++r) {
    const float a = fabsf(h2f(w[r * cols + c]));
    bad = bad || !(a <= 65504.f);                                // NaN or infinity
    best = fmaxf(best, a);
  }
  atomicMax(max_bits + c, __float_as_uint(best));
  if (bad) *flag = 1;
}
__global__ void quant_scales_kernel(const unsigned int* max_bits, float* scales, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float m = __uint_as_float(max_bits[c]);
  scales[c] = m != 0.f ? float(double(m) / 127.0) : 1.0f;       // max_bits and scales may be the same buffer
}
__global__ void quant_apply_kernel(const __half* w, const float* scales, int8_t* q, long long elements, int cols) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= elements) return;
  const double v = rint(double(h2f(w[i])) / double(scales[i % cols]));      // rint: to nearest, ties to even
  q[i] = int8_t(v < -127.0 ? -127.0 : v > 127.0 ? 127.0 : v);
}

// Last kernel of a decode step whose vocabulary projection merged the argmax itself (GemvArgs::argmax_best): publishes
// the winners (out[step][row], feedback[row] = next step's input id), leaves `best` zero again and moves every request
// one position on -- the work of argmax_kernel's last ticket and of advance_kernel.  One block of 64 threads, rows <= 64.
__global__ void __launch_bounds__(64)
argmax_finish_kernel(unsigned long long* best, int rows, int cols, int32_t* out, int32_t* feedback, int32_t* step,
                     int32_t* row_pos, int32_t* kv_lengths) {
  pdl_wait();
  const int r = threadIdx.x, s = *step;
  __syncthreads();                                              // everybody has read the counter before it moves
  if (r < rows) {
    const unsigned long long key = best[r];
    best[r] = 0ull;
    const int bi = key ? int(0xffffffffu - uint32_t(key)) : 0x7fffffff;
    out[size_t(s) * rows + r] = bi;
    feedback[r] = bi < cols ? bi : 0;                           // see argmax_kernel
    if (bi >= cols) report(kStatusNoToken);
    row_pos[r] += 1; kv_lengths[r] += 1;
  }
  if (r == 0) *step = s + 1;
  pdl_launch_dependents();
}

// Self-test of the bounded waits: one thread waits on an mbarrier nobody ever arrives on, gives up after `polls` polls
// (microseconds), records kStatusPipeTimeout in the device status word exactly as the pipelines do, and returns.  Nothing
// faults and nothing hangs; the host sees the status at its next synchronisation.
__global__ void bounded_wait_selftest_kernel(unsigned int polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    bool arrived = false;
    for (unsigned int spin = 0; spin < polls && !arrived; ++spin) arrived = mbar_try(&bar, 0);
    if (!arrived) report(kStatusPipeTimeout);
  }
}

// End of a device-resident decode step: every request moves one position on.
__global__ void advance_kernel(int32_t* row_pos, int32_t* kv_lengths, int32_t* step, int batch) {
  trace_event(kTrAdvance, 0);
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < batch) { row_pos[b] += 1; kv_lengths[b] += 1; }
  if (b == 0) *step += 1;
  pdl_launch_dependents();
}

// Teacher-forced NLL of `rows` logit rows in FP64 (reference nll_rows, llm/src/runtime.cu:67-76):
// loss[first_position + r] = mask ? max + log(sum exp(logit - max)) - logit[target] : 0.
// grid = rows, block = 256.
__global__ void __launch_bounds__(256)
nll_kernel(const float* logits, long long pitch, int cols, const int32_t* tokens, const uint8_t* mask,
           double* loss, int first_position) {
  __shared__ float s_max[8];
  __shared__ double s_sum[8];
  const int pos = first_position + blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* row = logits + (long long)blockIdx.x * pitch;
  float m = -CUDART_INF_F;
  for (int c = threadIdx.x; c < cols; c += 256) m = fmaxf(m, row[c]);
  m = warp_max(m);
  if (lane == 0) s_max[warp] = m;
  __syncthreads();
  m = s_max[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, s_max[w]);
  double s = 0.0;
  for (int c = threadIdx.x; c < cols; c += 256) s += exp(double(row[c]) - double(m));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  if (lane == 0) s_sum[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int w = 0; w < 8; ++w) total += s_sum[w];
    loss[pos] = mask[pos] ? double(m) + log(total) - double(row[tokens[pos]]) : 0.0;
  }
}

// out[0] = sum of loss[0..length) (reference sum_losses, llm/src/runtime.cu:77-80); one block.
__global__ void __launch_bounds__(256)
sum_f64_kernel(const double* loss, double* out, int length) {
  __shared__ double part[8];
  double v = 0.0;
  for (int i = threadIdx.x; i < length; i += 256) v += loss[i];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) { double t = 0.0; for (int w = 0; w < 8; ++w) t += part[w]; *out = t; }
}

// fp32 C = A.B kept only so the ABI symbol ti_v2_legacy_gemm_f32 resolves (reference legacy_f32,
// kernels/src/cuda/tc/gemm.cu:85-117 serves the FP32 compiler backend, not this path).
__global__ void __launch_bounds__(256)
sgemm_kernel(const float* a, const float* b, float* c, int m, int n, int k) {
  __shared__ float as[16][17], bs[16][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row = blockIdx.y * 16 + ty, col = blockIdx.x * 16 + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < k; k0 += 16) {
    as[ty][tx] = (row < m && k0 + tx < k) ? a[size_t(row) * k + k0 + tx] : 0.f;
    bs[ty][tx] = (k0 + ty < k && col < n) ? b[size_t(k0 + ty) * n + col] : 0.f;
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) acc = fmaf(as[ty][kk], bs[kk][tx], acc);
    __syncthreads();
  }
  if (row < m && col < n) c[size_t(row) * n + col] = acc;
}

}  // namespace tib
