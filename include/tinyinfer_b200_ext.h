/* Additive operator exports of the B200 build.  Same calling contract as
 * tinyinfer_backend_v2.h (device pointers, caller-owned stream, device already current,
 * host-side validation before anything is enqueued, ti_v2_last_error for the text).
 * The reference has no such entry points: it runs these steps as separate kernels
 * (ti_v2_gemm_ex_i8 -> ti_v2_gelu_new_f16 / add, gather_cache -> ti_v2_attention_f16,
 * llm/src/runtime.cu:142-154); they exist so the fused forms the model runtime uses can be
 * called, checked against that sequence and timed on their own.
 */
#ifndef TINYINFER_B200_EXT_H
#define TINYINFER_B200_EXT_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* INT8-weight GEMM with the epilogue fused:
 *   t = fp16(acc + bias);  if (gelu) t = fp16(gelu_tanh(t));  if (residual) t = fp16(residual + t)
 * i.e. the rounding points of reference ti_v2_gemm_ex_i8 (backend/runtime_v2.cu:69-76) followed
 * by ti_v2_gelu_new_f16 (:97-101) and the runtime's residual add (llm/src/runtime.cu:31-33).
 * output_dtype 1 (fp32) allows neither gelu nor residual.  residual is fp16 [M,N], nullable. */
int ti_b200_gemm_i8_fused(const uint16_t* a, const int8_t* b, const float* scales, const uint16_t* bias,
                          const uint16_t* residual, void* y, int m, int n, int k, int output_dtype, int gelu,
                          uintptr_t stream, int device);

/* Per-output-channel symmetric INT8 quantiser on the GPU: w[rows, columns] fp16 -> q[rows, columns] int8 and
 * scales[columns] fp32, bit-identical to ti_host_quantize_f16 (backend/host_codec.cpp, specification
 * llm/quantization.py): scale = float(double(max|w|) / 127.0) (1 for an all-zero column),
 * q = clip(round_half_even(double(w) / double(scale)), -127, 127).  All pointers are device memory and must not
 * overlap; nonfinite (device int32, required) is set to 1 when an input is NaN or infinite -- the host
 * codec rejects such input, here q and scales are then unspecified.  Asynchronous on `stream`.  The reference has
 * no device-side quantiser; its exporter quantises on the host. */
int ti_b200_quantize_f16(const uint16_t* w, int64_t rows, int64_t columns, int8_t* q, float* scales,
                         int32_t* nonfinite, uintptr_t stream, int device);

/* Decode attention (one query per request) reading k/v[B,H,K,64] in place:
 * q[B,H,1,64] -> y[B,H,1,64], keys 0..kv_lengths[b]-1 visible.  Equals reference
 * ti_v2_attention_f16 (backend/runtime_v2.cu:82-90) with q_len 1 and
 * query_offsets = kv_lengths-1.  Each (request, head) history is cut into chunks of `chunk`
 * keys (multiple of 32) processed by separate CTAs (a chunk that covers kv_len: one CTA of eight
 * warps walks the whole history and no partial results leave the chip); partial results live in `scratch`,
 * device memory of at least ti_b200_attention_decode_scratch_floats(...) floats, 16-byte
 * aligned, owned by the caller and private to this call until it completes. */
int64_t ti_b200_attention_decode_scratch_floats(int batch, int heads, int kv_len, int chunk);
int ti_b200_attention_decode_f16(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* y,
                                 const int32_t* kv_lengths, int batch, int heads, int kv_len, int head_dim,
                                 int chunk, float* scratch, int64_t scratch_floats, uintptr_t stream, int device);

/* No counterpart in the reference.  ti_b200_attention_decode_f16 for callers that cannot allocate
 * device memory (a serving loop with a fixed memory budget, an operator hosted by a program that
 * owns all device memory, a process at its memory limit): same inputs, outputs and results, but the
 * scratch is a fixed 4 MiB array inside the library (ti_b200_attention_decode_static_capacity_floats()
 * floats; every GPU that loads the library holds it until exit).  Calls no cudaMalloc / cudaFree.
 * Problems needing more than that (see ti_b200_attention_decode_scratch_floats) are rejected with
 * TI_V2_INVALID_ARGUMENT.  The first call on a device looks up the array's address; make it during
 * start-up, before any stream capture on that device.  All calls on a device share the array, so
 * calls that can overlap on the GPU race: serialise them.  Nothing in the array needs clearing. */
long long ti_b200_attention_decode_static_capacity_floats(void);
int ti_b200_attention_decode_static_f16(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* y,
                                        const int32_t* kv_lengths, int batch, int heads, int kv_len, int head_dim,
                                        int chunk, uintptr_t stream, int device);

/* Exported by libtinyinfer_llm.so.  Verifies manifest.json + weights.bin exactly as
 * ti_llm_create does before touching the GPU (reference llm/src/artifact.hpp:153-199; the
 * reference only reaches these checks through ti_llm_create) and reports the model shape.
 * Pure host code.  Returns a ti_llm_status; ti_llm_last_error() has the text.  Out-pointers
 * are optional. */
int ti_b200_artifact_check(const char* manifest_path, int32_t* layers, int32_t* heads, int32_t* hidden,
                           int32_t* int8_weights);

/* Exported by libtinyinfer_llm.so.  Runs `steps` greedy decode steps for `batch` requests whose
 * slots already hold a prefix (ti_llm_forward_batch), starting from the input ids first_tokens[B]
 * (normally the argmax the prefill returned).  Tokens, positions and the KV cache stay on the GPU
 * between steps -- the host is involved once, at the end.  out_tokens (host, nullable) receives
 * [steps][batch] ids; device_ms (nullable) the time between the first and the last kernel of the
 * steps measured with CUDA events on the model's stream.  Each slot advances by `steps`.
 * The reference has no counterpart: its ti_llm_greedy_batch returns to the host after every
 * token (llm/src/runtime.cu:196-200).  ti_llm_greedy_batch of this build runs on the same
 * mechanism; this entry point exposes it for measurement.  Returns a ti_llm_status. */
struct ti_llm_model;
int ti_b200_llm_decode_steps(struct ti_llm_model* model, const int32_t* slots, const int32_t* first_tokens,
                             int32_t batch, int32_t steps, int32_t* out_tokens, double* device_ms);

/* Exported by libtinyinfer_llm.so.  Selects how a greedy decode step of up to 32 requests runs: 0 = one launch per
 * operation replayed as a CUDA graph (the default), 1 = one persistent kernel per step (one CTA per SM, activations
 * handed between CTAs as tagged words; available where the model shape and the device allow it), -1 = leave as is.
 * Both plans produce the same bits.  active (nullable) receives the plan in force afterwards.  The reference has one plan only
 * (a launch per operation, llm/src/runtime.cu:135-168).  Returns a ti_llm_status; TI_LLM_INVALID when plan 1 is
 * asked for a shape it does not cover. */
int ti_b200_llm_decode_plan(struct ti_llm_model* model, int32_t select, int32_t* active);

/* Exported by libtinyinfer_llm.so.  Test hook for the failure paths; the reference has none (its tests never reach
 * llm/src/runtime.cu:127,172-174).  kind 0: the forward call after `after_calls` more valid ones fails on the host
 * the way a failed launch does (TI_LLM_CUDA, the model is poisoned).  kind 1: enqueues a one-thread kernel whose
 * bounded mbarrier wait runs out after about a thousand polls and records a timeout in the device status word -- the
 * path every pipeline wait takes on expiry -- so the next call that synchronises returns TI_LLM_CUDA and poisons the
 * model.  Neither faults, traps or hangs the GPU. */
int ti_b200_llm_inject_failure(struct ti_llm_model* model, int32_t kind, int32_t after_calls);
#ifdef __cplusplus
}
#endif
#endif
