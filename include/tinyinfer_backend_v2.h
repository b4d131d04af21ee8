/* Operator C ABI, version 2 -- the device-pointer entry points llm/native_ops.py binds with
 * ctypes and the model runtime links.  Signature-for-signature replacement of the reference's
 * backend/include/tinyinfer_backend_v2.h:7-38; implemented for sm_100a in
 * tinyinfer_b200/csrc/backend_api.cu.
 *
 * Contract shared by every launch entry point:
 *   - every pointer is device memory on `device`, contiguous row-major, owned by the caller,
 *     outputs alias nothing;
 *   - `stream` is a cudaStream_t passed as an integer; the call only enqueues ("OK" = queued);
 *   - the calling thread must already have `device` current, else TI_V2_DEVICE_MISMATCH
 *     (reference backend/runtime_v2.cu:19-25);
 *   - arguments are validated on the host before anything is enqueued
 *     (reference backend/include/tinyinfer_host_validation.hpp:23-70);
 *   - the message of the last failing call on this thread is kept until the thread's next call.
 */
#ifndef TINYINFER_BACKEND_V2_H
#define TINYINFER_BACKEND_V2_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum ti_v2_status {
  TI_V2_OK = 0, TI_V2_INVALID_ARGUMENT = 1, TI_V2_DEVICE_MISMATCH = 2,
  TI_V2_UNSUPPORTED_CONFIG = 3, TI_V2_CUDA_ERROR = 4
};
enum ti_v2_output_dtype { TI_V2_FP16 = 0, TI_V2_FP32 = 1 };

/* reference backend/runtime_v2.cu:31 -- always 2. */
int ti_v2_abi_version(void);
/* reference backend/runtime_v2.cu:32 -- thread-local text of the last failure. */
const char* ti_v2_last_error(void);
/* reference backend/runtime_v2.cu:33-53 -- JSON describing the 12 GEMM config ids.  The ids
 * are kept as ABI values only: this build runs one kernel family per problem shape and ignores
 * the tile/stage meaning of `config` (it is still range-checked). */
const char* ti_v2_gemm_catalog_json(void);

/* y[M,N] = a[M,K] (fp16) . b[K,N] (fp16) + bias[N] (fp16, nullable); y is fp16 or fp32.
 * reference backend/runtime_v2.cu:54-57 and :62-68. */
int ti_v2_gemm_f16(const uint16_t* a, const uint16_t* b, const uint16_t* bias, void* y,
                   int m, int n, int k, int output_dtype, int config, uintptr_t stream, int device);
int ti_v2_gemm_ex_f16(const uint16_t* a, const uint16_t* b, const uint16_t* bias, void* y, float* workspace,
                      int m, int n, int k, int output_dtype, int config, uintptr_t stream, int device);

/* Weight-only INT8: b is int8[K,N], scales fp32[N]; the weight used in the product is
 * fp16_rn(float(b) * scales[col]).  reference backend/runtime_v2.cu:58-61 and :69-76.
 * `workspace` (fp32[M,N]) must be non-null and 4-byte aligned for config >= 6, as in the
 * reference; it is never written by this build (the epilogue is always fused). */
int ti_v2_gemm_i8(const uint16_t* a, const int8_t* b, const float* scales, const uint16_t* bias, void* y,
                  int m, int n, int k, int output_dtype, int config, uintptr_t stream, int device);
int ti_v2_gemm_ex_i8(const uint16_t* a, const int8_t* b, const float* scales, const uint16_t* bias, void* y,
                     float* workspace, int m, int n, int k, int output_dtype, int config,
                     uintptr_t stream, int device);

/* fp32 GEMM kept as an ABI symbol; reference backend/runtime_v2.cu:77-81. */
int ti_v2_legacy_gemm_f32(const float* a, const float* b, float* y, int m, int n, int k,
                          uintptr_t stream, int device);

/* q[B,H,Q,D], k/v[B,H,K,D] fp16, metadata int32[B]; D is 64 or 128.  Key j is visible to
 * query i of request b when j < min(K, kv_lengths[b]) and (!causal or j <= query_offsets[b]+i);
 * rows i >= q_lengths[b] and rows that see no key are written as exact zeros.
 * reference backend/runtime_v2.cu:82-90, kernels/src/cuda/tc/attention.cu:9-57. */
int ti_v2_attention_f16(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* y,
                        const int32_t* q_lengths, const int32_t* kv_lengths, const int32_t* query_offsets,
                        int batch, int heads, int q_len, int kv_len, int head_dim, int causal, int config,
                        uintptr_t stream, int device);

/* reference backend/runtime_v2.cu:91-106, kernels/src/cuda/tc/elementwise.cu:15-57. */
int ti_v2_layernorm_f16(const uint16_t* x, const uint16_t* gamma, const uint16_t* beta, uint16_t* y,
                        int rows, int cols, float eps, uintptr_t stream, int device);
int ti_v2_gelu_new_f16(const uint16_t* x, uint16_t* y, int64_t count, uintptr_t stream, int device);
int ti_v2_softmax_f16(const uint16_t* x, uint16_t* y, int rows, int cols, uintptr_t stream, int device);

#ifdef __cplusplus
}
#endif
#endif
