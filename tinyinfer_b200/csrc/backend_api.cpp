// Operator C ABI v2 (include/tinyinfer_backend_v2.h): argument validation, the thread-local
// error text and hand-off to the sm_100a launchers of kernels.cu.
//
// Behaviour mirrored from the reference front end (backend/runtime_v2.cu:10-106) and its
// validators (backend/include/tinyinfer_host_validation.hpp:12-70): same status codes, same
// order of checks (device first, then metadata; nothing is enqueued after a failed check), same
// acceptance ranges.  Row counts the reference accepts but one launch's grid cannot carry are run as several launches
// over row blocks (kernels.cu), never surfaced as a failed launch.
//
// Additive exports (ti_b200_*) expose the fused epilogues and the in-place decode attention
// that the model runtime uses, so they can be exercised and timed through the C ABI.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <limits>

#include "launch.hpp"
#include "tinyinfer_b200_ext.h"
#include "tinyinfer_backend_v2.h"

namespace {

thread_local char g_error[256] = "";

int fail(int status, const char* text) {
  std::snprintf(g_error, sizeof g_error, "%s", text);
  return status;
}
int cuda_result(cudaError_t st) { return st == cudaSuccess ? TI_V2_OK : fail(TI_V2_CUDA_ERROR, cudaGetErrorString(st)); }

// The caller must already be on `device` (reference begin(), backend/runtime_v2.cu:19-25).
int enter(int device) {
  g_error[0] = '\0';
  if (device < 0) return fail(TI_V2_INVALID_ARGUMENT, "device must be nonnegative");
  int current = -1;
  const cudaError_t st = cudaGetDevice(&current);
  if (st != cudaSuccess) return cuda_result(st);
  if (current != device) return fail(TI_V2_DEVICE_MISMATCH, "caller must select the supplied CUDA device");
  return TI_V2_OK;
}

bool aligned_to(const void* p, size_t bytes) { return p && reinterpret_cast<uintptr_t>(p) % bytes == 0; }

// All extents positive and the byte size representable in int64.
template <size_t N>
bool extent_ok(const int (&dims)[N], size_t element_bytes) {
  uint64_t total = element_bytes;
  for (int d : dims) {
    if (d <= 0 || total > uint64_t(std::numeric_limits<int64_t>::max()) / uint64_t(d)) return false;
    total *= uint64_t(d);
  }
  return true;
}

int config_tile_rows(int config) { return config % 3 == 0 ? 32 : 64; }

int check_gemm(const void* a, const void* b, const void* bias, const void* y, int m, int n, int k, int dtype, int config,
               bool int8) {
  if (config < 0 || config > 11) return fail(TI_V2_UNSUPPORTED_CONFIG, "GEMM config absent from this compiled allow-list");
  const size_t out_bytes = dtype == 0 ? 2 : 4;
  const int mk[2] = {m, k}, kn[2] = {k, n}, mn[2] = {m, n};
  if ((dtype != 0 && dtype != 1) || !aligned_to(a, 2) || !aligned_to(b, int8 ? 1 : 2) || !aligned_to(y, out_bytes) ||
      (bias && !aligned_to(bias, 2)) || !extent_ok(mk, 2) || !extent_ok(kn, int8 ? 1 : 2) || !extent_ok(mn, out_bytes) ||
      (m - 1) / config_tile_rows(config) + 1 > 65535)
    return fail(TI_V2_INVALID_ARGUMENT, "invalid GEMM shape, pointers, alignment, output dtype or grid");
  return TI_V2_OK;
}
int check_workspace(const void* workspace, int m, int n, int config) {
  const int mn[2] = {m, n};
  if (config >= 6 && (!aligned_to(workspace, 4) || !extent_ok(mn, 4)))
    return fail(TI_V2_INVALID_ARGUMENT, "separate epilogue requires caller-owned FP32[M,N] workspace");
  return TI_V2_OK;
}

int run_gemm(const uint16_t* a, const void* b, const float* scales, const uint16_t* bias, void* y, const uint16_t* residual,
             int gelu, int m, int n, int k, int dtype, bool int8, uintptr_t stream) {
  tib::GemmCall call;
  call.a = a; call.lda = k; call.w = b; call.ldw = n; call.w_int8 = int8; call.scales = scales; call.bias = bias;
  call.out = y; call.ldo = n; call.out_fp32 = dtype == 1; call.residual = residual; call.gelu = gelu != 0;
  call.m = m; call.n = n; call.k = k;
  tib::LaunchOpts opts; opts.stream = reinterpret_cast<cudaStream_t>(stream);
  return cuda_result(tib::gemm(call, opts));
}

}  // namespace

// Helpers shared with attention_static_scratch.cu (same checks, same thread-local error text).
namespace tib_api {
int enter_call(int device) { return enter(device); }
int fail_call(int status, const char* text) { return fail(status, text); }
int cuda_call(cudaError_t st) { return cuda_result(st); }
int check_decode_attention(const void* q, const void* k, const void* v, const void* y, const void* kv_lengths, int batch, int heads,
                           int kv_len, int head_dim, int chunk) {
  const int kd[4] = {batch, heads, kv_len, head_dim};
  if (head_dim != 64 || batch > 65535 || heads > 65535 || !extent_ok(kd, 2) || chunk < 32 || chunk % 32 || !aligned_to(q, 16) ||
      !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(y, 16) || !aligned_to(kv_lengths, 4))
    return fail(TI_V2_INVALID_ARGUMENT, "invalid decode attention arguments (D=64, chunk multiple of 32, 16-byte aligned tensors)");
  return TI_V2_OK;
}
}  // namespace tib_api

extern "C" {

int ti_v2_abi_version(void) { return 2; }
const char* ti_v2_last_error(void) { return g_error; }

const char* ti_v2_gemm_catalog_json(void) {
  // Twelve ids = 3 tile names x {2,1} stages x {fused, separate} epilogue, in the order the
  // Python wrapper's GEMM_CATALOG enumerates them (llm/native_ops.py:14-16).
  static const char* text = [] {
    static char buffer[1400];
    static const char* tiles[3] = {"[32,32,16,4]", "[64,32,32,8]", "[64,64,32,8]"};
    int used = std::snprintf(buffer, sizeof buffer, "{\"schema_version\":1,\"only_config\":-1,\"configs\":[");
    for (int id = 0; id < 12; ++id)
      used += std::snprintf(buffer + used, sizeof buffer - size_t(used), "%s{\"id\":%d,\"tile\":%s,\"stages\":%d,\"epilogue\":\"%s\"}",
                            id ? "," : "", id, tiles[id % 3], ((id >= 3 && id < 6) || id >= 9) ? 1 : 2, id >= 6 ? "separate" : "fused");
    std::snprintf(buffer + used, sizeof buffer - size_t(used), "]}");
    return buffer;
  }();
  return text;
}

int ti_v2_gemm_ex_f16(const uint16_t* a, const uint16_t* b, const uint16_t* bias, void* y, float* workspace,
                      int m, int n, int k, int dtype, int config, uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  st = check_gemm(a, b, bias, y, m, n, k, dtype, config, false); if (st) return st;
  st = check_workspace(workspace, m, n, config); if (st) return st;
  return run_gemm(a, b, nullptr, bias, y, nullptr, 0, m, n, k, dtype, false, stream);
}
int ti_v2_gemm_ex_i8(const uint16_t* a, const int8_t* b, const float* scales, const uint16_t* bias, void* y, float* workspace,
                     int m, int n, int k, int dtype, int config, uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  st = check_gemm(a, b, bias, y, m, n, k, dtype, config, true); if (st) return st;
  if (!aligned_to(scales, 4)) return fail(TI_V2_INVALID_ARGUMENT, "scales pointer must be nonnull aligned FP32[N]");
  st = check_workspace(workspace, m, n, config); if (st) return st;
  return run_gemm(a, b, scales, bias, y, nullptr, 0, m, n, k, dtype, true, stream);
}
int ti_v2_gemm_f16(const uint16_t* a, const uint16_t* b, const uint16_t* bias, void* y, int m, int n, int k, int dtype,
                   int config, uintptr_t stream, int device) {
  return ti_v2_gemm_ex_f16(a, b, bias, y, nullptr, m, n, k, dtype, config, stream, device);
}
int ti_v2_gemm_i8(const uint16_t* a, const int8_t* b, const float* scales, const uint16_t* bias, void* y, int m, int n, int k,
                  int dtype, int config, uintptr_t stream, int device) {
  return ti_v2_gemm_ex_i8(a, b, scales, bias, y, nullptr, m, n, k, dtype, config, stream, device);
}

int ti_v2_legacy_gemm_f32(const float* a, const float* b, float* y, int m, int n, int k, uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  const int mk[2] = {m, k}, kn[2] = {k, n}, mn[2] = {m, n};
  if (!aligned_to(a, 4) || !aligned_to(b, 4) || !aligned_to(y, 4) || !extent_ok(mk, 4) || !extent_ok(kn, 4) ||
      !extent_ok(mn, 4) || (m - 1) / 64 + 1 > 65535)
    return fail(TI_V2_INVALID_ARGUMENT, "invalid FP32 GEMM arguments");
  return cuda_result(tib::sgemm(a, b, y, m, n, k, reinterpret_cast<cudaStream_t>(stream)));
}

int ti_v2_attention_f16(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* y, const int32_t* ql,
                        const int32_t* kl, const int32_t* offsets, int b, int h, int nq, int nk, int d, int causal,
                        int config, uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  if (config < 0 || config > 1) return fail(TI_V2_UNSUPPORTED_CONFIG, "attention config must be 0,1");
  const int qd[4] = {b, h, nq, d}, kd[4] = {b, h, nk, d};
  if ((d != 64 && d != 128) || (causal != 0 && causal != 1) || b > 65535 || h > 65535 || !extent_ok(qd, 2) ||
      !extent_ok(kd, 2) || !aligned_to(q, 2) || !aligned_to(k, 2) || !aligned_to(v, 2) || !aligned_to(y, 2) ||
      !aligned_to(ql, 4) || !aligned_to(kl, 4) || !aligned_to(offsets, 4) || (nq - 1) / 8 + 1 > 2147483647)
    return fail(TI_V2_INVALID_ARGUMENT, "invalid attention arguments");
  tib::LaunchOpts opts; opts.stream = reinterpret_cast<cudaStream_t>(stream);
  return cuda_result(tib::attention_packed(q, k, v, y, ql, kl, offsets, b, h, nq, nk, d, causal != 0, opts));
}

int ti_v2_layernorm_f16(const uint16_t* x, const uint16_t* g, const uint16_t* bt, uint16_t* y, int rows, int cols, float eps,
                        uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  const int rc[2] = {rows, cols};
  if (!extent_ok(rc, 2) || !std::isfinite(eps) || eps <= 0.f || !aligned_to(x, 2) || !aligned_to(g, 2) || !aligned_to(bt, 2) ||
      !aligned_to(y, 2))
    return fail(TI_V2_INVALID_ARGUMENT, "invalid LayerNorm arguments");
  tib::LaunchOpts opts; opts.stream = reinterpret_cast<cudaStream_t>(stream);
  return cuda_result(tib::layernorm(x, nullptr, g, bt, y, rows, cols, eps, opts));
}
int ti_v2_gelu_new_f16(const uint16_t* x, uint16_t* y, int64_t count, uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  if (count <= 0 || count > std::numeric_limits<int64_t>::max() / 2 || !aligned_to(x, 2) || !aligned_to(y, 2))
    return fail(TI_V2_INVALID_ARGUMENT, "invalid GELU arguments");
  return cuda_result(tib::gelu(x, y, count, reinterpret_cast<cudaStream_t>(stream)));
}
int ti_v2_softmax_f16(const uint16_t* x, uint16_t* y, int rows, int cols, uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  const int rc[2] = {rows, cols};
  if (!extent_ok(rc, 2) || !aligned_to(x, 2) || !aligned_to(y, 2)) return fail(TI_V2_INVALID_ARGUMENT, "invalid softmax arguments");
  return cuda_result(tib::softmax(x, y, rows, cols, reinterpret_cast<cudaStream_t>(stream)));
}

// ------------------------------------------------------------------ additive exports
int ti_b200_gemm_i8_fused(const uint16_t* a, const int8_t* b, const float* scales, const uint16_t* bias,
                          const uint16_t* residual, void* y, int m, int n, int k, int dtype, int gelu,
                          uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  st = check_gemm(a, b, bias, y, m, n, k, dtype, 0, true); if (st) return st;
  if (!aligned_to(scales, 4)) return fail(TI_V2_INVALID_ARGUMENT, "scales pointer must be nonnull aligned FP32[N]");
  if ((gelu != 0 && gelu != 1) || (dtype == 1 && (gelu || residual)) || (residual && !aligned_to(residual, 2)))
    return fail(TI_V2_INVALID_ARGUMENT, "GELU / residual epilogues need FP16 output");
  return run_gemm(a, b, scales, bias, y, residual, gelu, m, n, k, dtype, true, stream);
}

int ti_b200_quantize_f16(const uint16_t* w, int64_t rows, int64_t columns, int8_t* q, float* scales, int32_t* nonfinite,
                         uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  if (rows < 1 || columns < 1 || columns > 0x7fffffff || rows > (int64_t(1) << 40) / columns || !aligned_to(w, 2) || !q ||
      !aligned_to(scales, 4) || !aligned_to(nonfinite, 4))
    return fail(TI_V2_INVALID_ARGUMENT, "invalid quantiser arguments (w FP16[rows,columns], q INT8, scales FP32[columns], flag INT32)");
  return cuda_result(tib::quantize_i8(w, rows, int(columns), q, scales, nonfinite, reinterpret_cast<cudaStream_t>(stream)));
}

int64_t ti_b200_attention_decode_scratch_floats(int batch, int heads, int kv_len, int chunk) {
  if (batch <= 0 || heads <= 0 || kv_len <= 0 || chunk <= 0) return -1;
  return int64_t(batch) * heads * tib::decode_chunks(kv_len, chunk) * (64 + 2);
}

int ti_b200_attention_decode_f16(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* y,
                                 const int32_t* kv_lengths, int batch, int heads, int kv_len, int head_dim, int chunk,
                                 float* scratch, int64_t scratch_floats, uintptr_t stream, int device) {
  int st = enter(device); if (st) return st;
  st = tib_api::check_decode_attention(q, k, v, y, kv_lengths, batch, heads, kv_len, head_dim, chunk); if (st) return st;
  const int64_t need = ti_b200_attention_decode_scratch_floats(batch, heads, kv_len, chunk);
  if (!aligned_to(scratch, 16) || scratch_floats < need)
    return fail(TI_V2_INVALID_ARGUMENT, "decode attention scratch too small or misaligned");
  const int64_t acc_floats = int64_t(batch) * heads * tib::decode_chunks(kv_len, chunk) * 64;
  tib::LaunchOpts opts; opts.stream = reinterpret_cast<cudaStream_t>(stream);
  return cuda_result(tib::attention_packed_decode(q, k, v, y, kv_lengths, batch, heads, kv_len, chunk, scratch,
                                                 scratch + acc_floats, opts));
}

}  // extern "C"
