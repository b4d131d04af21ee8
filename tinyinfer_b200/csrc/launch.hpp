// Host-side launch interface of the kernel translation unit (kernels.cu).  Plain C++: no device
// code, usable from the C-ABI front ends (backend_api.cpp, llm_runtime.cpp).  Every function
// only enqueues work on `stream` and returns the launch status.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "step_plan.hpp"

#if defined(__GNUC__)
#define TIB_EXPORT __attribute__((visibility("default")))
#else
#define TIB_EXPORT
#endif

namespace tib {

struct LaunchOpts {
  cudaStream_t stream = nullptr;
  bool pdl = false;              // programmatic dependent launch: prologue may overlap the previous kernel
  // With pdl: release the launch of the kernel after this one at once instead of after this kernel's own dependency
  // wait.  Only sound when that kernel reads nothing but constants (weights, parameters) ahead of its own wait.
  // Honoured by layernorm and gemm (tensor-core path).
  bool early_trigger = false;
};

// Paged KV pool of the model runtime; see attention.cuh for the page layout.
struct PagedKv {
  void* k_pool = nullptr; void* v_pool = nullptr;
  const int32_t* table = nullptr;     // [slots][table_pitch]
  const int32_t* slots = nullptr;     // [batch]
  int table_pitch = 0, layers = 0, layer = 0, heads = 0, head_dim = 0;
};

// out[M,N] = a[M,K] . W[K,N] + bias, fused epilogue; W int8 (+scales) or fp16.
struct GemmCall {
  const void* a = nullptr; int lda = 0;                 // fp16 [M,K]
  const void* w = nullptr; long long ldw = 0;           // [K,N], pitch in elements
  bool w_int8 = true;
  // int8 only: w holds slab-major tiles [ceil(N/128)][w_slab_rows][128] (see retile_i8) instead of [K,N]; w_slab_rows >= k,
  // multiple of 64.  Every 64-row stage of a CTA is then one contiguous 8 KB block of device memory.
  int w_slab_rows = 0;
  const float* scales = nullptr;
  const void* bias = nullptr;                           // fp16 [N] or null
  void* out = nullptr; int ldo = 0; bool out_fp32 = false;
  const void* residual = nullptr;                       // fp16 [M,N] pitch ldo, or null
  bool gelu = false;
  // QKV projection of the model runtime: when kv is set, columns [hidden, 3*hidden) (the K and V thirds)
  // are written to row r's position kv_row_pos[r] of request kv_row_req[r] in the paged pool, not to `out`.
  const PagedKv* kv = nullptr; const int32_t* kv_row_req = nullptr; const int32_t* kv_row_pos = nullptr;
  // LayerNorm prologue: `a` holds rows before normalisation (m <= 32, k <= 768, int8 weights reachable by TMA);
  // gemm() returns cudaErrorNotSupported when the shape cannot take it.
  const void* ln_gamma = nullptr; const void* ln_beta = nullptr; float ln_eps = 1e-5f;
  bool uniform_numerics = false;                         // tensor-core kernel for any row count (batch-invariant results)
  // fp32 output without a K split (vocabulary projection): merge each row's greedy argmax into argmax_best[row]
  // (64-bit words, zero between steps; argmax_finish publishes them); skip_store: do not write the logits.
  void* argmax_best = nullptr; bool skip_store = false;
  const void* w_image = nullptr;                         // optional operand image of the same matrix (wide_image): used from 129 rows on
  int m = 0, n = 0, k = 0;
};
TIB_EXPORT cudaError_t gemm(const GemmCall& call, const LaunchOpts& opts);

// dst[slab][row][c] = row < k && slab*128+c < n ? src[row*ld + slab*128+c] : 0, for ceil(n/128) slabs of slab_rows rows.
TIB_EXPORT cudaError_t retile_i8(const int8_t* src, long long ld, int k, int n, int8_t* dst, int slab_rows, cudaStream_t stream);

// Operand image of a [K,N] weight matrix for many-row passes (gemm_wide.cuh): the fp16 values an INT8 matrix `q` with
// per-column `scales` dequantises to (or the fp16 matrix `w16`; exactly one of the two is given; `ld` = row pitch in
// elements), laid out stage by stage in the shared-memory form of the tensor-core operand.  GemmCall::w_image takes it.
TIB_EXPORT size_t wide_image_bytes(int k, int n);
TIB_EXPORT cudaError_t wide_image(const int8_t* q, const void* w16, long long ld, const float* scales, void* image, int k, int n, cudaStream_t stream);

// Per-output-channel symmetric INT8 quantisation of w[rows][cols] (fp16) on the device, bit-identical to the host codec.
// scales[cols] doubles as the scratch of the column maxima; flag (device int, zeroed here) becomes 1 for non-finite input.
TIB_EXPORT cudaError_t quantize_i8(const void* w, long long rows, int cols, int8_t* q, float* scales, int* flag, cudaStream_t stream);

TIB_EXPORT cudaError_t sgemm(const float* a, const float* b, float* c, int m, int n, int k, cudaStream_t stream);

// Packed-tensor attention of the operator ABI: q[B,H,Q,D], k/v[B,H,K,D].
TIB_EXPORT cudaError_t attention_packed(const void* q, const void* k, const void* v, void* y,
                                        const int32_t* q_lengths, const int32_t* kv_lengths, const int32_t* offsets,
                                        int batch, int heads, int q_len, int kv_len, int head_dim, bool causal,
                                        const LaunchOpts& opts);

// Prefill / mixed lengths: request b owns rows row_start[b] .. row_start[b]+q_lengths[b]-1 of
// qkv[rows, 3*hidden]; attention output goes to out[rows, hidden] (heads merged).
TIB_EXPORT cudaError_t attention_paged(const void* qkv, void* out, const int32_t* row_start,
                                       const int32_t* q_lengths, const int32_t* kv_lengths, const int32_t* offsets,
                                       int batch, int max_q, int max_kv, const PagedKv& kv, const LaunchOpts& opts,
                                       bool skip_single = false, int long_requests = 0, int short_requests = 1);
// long_requests / short_requests: how many requests of the pass have at least / fewer than 64 query rows (the caller
// knows the lengths on the host): the former run on the tensor-core kernel, the latter on the SIMT tile kernel.
// Decode: one row per request.  scratch_acc: fp32 [batch*heads*chunks*D], scratch_ml: fp32
// [batch*heads*chunks*2]; chunks = ceil(max_kv / chunk).
// counters: optional int [batch*heads], zero between launches; when given the merge of the chunk
// partials happens inside the same kernel (no second launch).
// early: kv_lengths, the page table and all keys but each request's newest were complete before the kernel
// ahead of this launch started (true inside a decode step: only the QKV projection precedes it); they are
// then read ahead of the dependency wait.  whole_history: one CTA per (request, head) instead of one per chunk;
// chunk, scratch and counters are not used.  early_trigger: the kernel launched after this one may start at once
// (it must then read nothing but constants ahead of its own dependency wait).  row_start / q_lengths (whole_history
// only): a pass that mixes prompts and single tokens -- request b's row is row_start[b], requests with q_lengths[b] != 1
// are skipped (attention_paged with skip_single handles them).
TIB_EXPORT cudaError_t attention_paged_decode(const void* qkv, void* out, const int32_t* kv_lengths,
                                              int batch, int max_kv, int chunk, float* scratch_acc, float* scratch_ml,
                                              int* counters, const PagedKv& kv, const LaunchOpts& opts,
                                              bool early = false, bool whole_history = false, bool early_trigger = false,
                                              const int32_t* row_start = nullptr, const int32_t* q_lengths = nullptr);
TIB_EXPORT int decode_chunks(int max_kv, int chunk);
// Same decode attention over packed k/v[B,H,K,D] with q[B,H,1,D] (additive operator export).
TIB_EXPORT cudaError_t attention_packed_decode(const void* q, const void* k, const void* v, void* y,
                                               const int32_t* kv_lengths, int batch, int heads, int kv_len, int chunk,
                                               float* scratch_acc, float* scratch_ml, const LaunchOpts& opts);

// y[r,:] = LayerNorm(x[row_index ? row_index[r] : r, :]).
TIB_EXPORT cudaError_t layernorm(const void* x, const int32_t* row_index, const void* gamma, const void* beta, void* y,
                                 int rows, int cols, float eps, const LaunchOpts& opts);
TIB_EXPORT cudaError_t gelu(const void* x, void* y, long long count, cudaStream_t stream);
TIB_EXPORT cudaError_t softmax(const void* x, void* y, int rows, int cols, cudaStream_t stream);

TIB_EXPORT cudaError_t embed(const int32_t* ids, const int32_t* row_pos, const void* wte, const void* wpe,
                             void* x, int rows, int hidden, int vocab, const LaunchOpts& opts);
// out[(*step) * rows + r] = argmax of row r (step may be null = 0); feedback[r] too when non-null.
// scratch: null, or 12 * rows bytes of device memory (8-byte aligned, zero before its first use, left zero
// by every call) that lets several CTAs share a row.
TIB_EXPORT cudaError_t argmax(const float* logits, long long pitch, int rows, int cols, int32_t* out,
                              int32_t* feedback, const int32_t* step, void* scratch, const LaunchOpts& opts);
// After a gemm() with argmax_best: out[(*step) * rows + r] and feedback[r] from best[r] (left zero), then row_pos[r]++,
// kv_lengths[r]++ and (*step)++.  rows <= 64.
TIB_EXPORT cudaError_t argmax_finish(void* best, int rows, int cols, int32_t* out, int32_t* feedback, int32_t* step,
                                     int32_t* row_pos, int32_t* kv_lengths, const LaunchOpts& opts);
// row_pos[b]++, kv_lengths[b]++ for b < batch, and (*step)++.
TIB_EXPORT cudaError_t advance(int32_t* row_pos, int32_t* kv_lengths, int32_t* step, int batch, const LaunchOpts& opts);

TIB_EXPORT cudaError_t nll_rows(const float* logits, long long pitch, int rows, int cols, const int32_t* tokens,
                                const uint8_t* mask, double* loss, int first_position, cudaStream_t stream);
TIB_EXPORT cudaError_t sum_f64(const double* values, double* out, int length, cudaStream_t stream);

// Persistent decode step (decode_step.cuh): one cooperative launch runs embedding .. argmax for plan.batch <= 32
// requests and advances the device-resident state.  step_k_chunk: K rows per range of the K split a [K,N] matrix has
// in gemm() (the plan must use the same ranges: results are then bit-identical to the launch-per-GEMM step).
// step_unsupported: null, or why this shape / device cannot run the persistent step.
struct alignas(64) TileMap { unsigned char bytes[128]; };      // tensor map over the tile arena ([rows][128] int8)
TIB_EXPORT int step_k_chunk(int n, int k);
TIB_EXPORT const char* step_unsupported(const StepPlan& plan);
TIB_EXPORT cudaError_t make_tile_map(const void* arena, long long rows, TileMap* out);
TIB_EXPORT cudaError_t decode_step(const StepPlan& plan, const TileMap& tiles, cudaStream_t stream);

// Enqueues a one-thread kernel whose bounded wait runs out after `polls` polls and records kStatusPipeTimeout (test aid
// for the timeout -> status word -> host error path; nothing faults or hangs).
TIB_EXPORT cudaError_t selftest_bounded_wait(cudaStream_t stream, unsigned int polls);

// Reads and clears the device status word set by a kernel whose bounded wait ran out
// (0 = healthy).  Synchronises `stream` first.
TIB_EXPORT cudaError_t read_device_status(cudaStream_t stream, unsigned int* status);
// Device address of that status word on the current device (for an asynchronous copy).
TIB_EXPORT cudaError_t device_status_address(unsigned int** address);

}  // namespace tib
