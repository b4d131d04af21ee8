/* Model C ABI, version 1 -- the synchronous host API llm/runtime.py binds with ctypes and the
 * batching server links.  Replaces the reference's llm/include/tinyinfer_llm.h:12-60
 * (implementation llm/src/runtime.cu:172-211); implemented in tinyinfer_b200/csrc/llm_runtime.cu.
 *
 * All token / logit / output pointers are HOST pointers.  A model context owns its device
 * selection, one CUDA stream, the weights, the paged KV pool and its scratch.  Calls on one
 * context must be serialised by the caller; contexts are independent, so one thread per GPU
 * may each drive its own context.  Validation failures (TI_LLM_INVALID) enqueue nothing and
 * leave every slot length unchanged; TI_LLM_CUDA / TI_LLM_INTERNAL poison the context, after
 * which every call fails until it is destroyed.
 */
#ifndef TINYINFER_LLM_H
#define TINYINFER_LLM_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct ti_llm_model ti_llm_model;
enum ti_llm_status { TI_LLM_OK = 0, TI_LLM_INVALID = 1, TI_LLM_IO = 2, TI_LLM_CUDA = 3, TI_LLM_INTERNAL = 4 };

/* 28 bytes; struct_size must equal sizeof(ti_llm_options).  reference tinyinfer_llm.h:15-19.
 * Ranges: device >= 0, max_batch 1..64 (the reference stops at 32), cache_slots
 * max_batch..1024, capacity 2..1024, gemm_config 0..11, attention_config 0..1 (the last two
 * are range-checked ABI values; this build has one kernel family per shape). */
typedef struct ti_llm_options {
  uint32_t struct_size;
  int32_t device, max_batch, cache_slots, capacity;
  int32_t gemm_config, attention_config;
} ti_llm_options;

/* 96 bytes of logical-operation counters, bumped on the host once per logical operation a
 * forward pass performs, fused or not.  reference tinyinfer_llm.h:20-23. */
typedef struct ti_llm_trace {
  uint64_t forward_calls, embedding, gemm_fp16, gemm_int8, layernorm;
  uint64_t gelu, attention, residual, kv_scatter_gather, lm_head, argmax, nll;
} ti_llm_trace;

int ti_llm_abi_version(void);                 /* reference runtime.cu:176 -- always 1 */
const char* ti_llm_last_error(void);          /* reference runtime.cu:177 -- thread-local */
/* reference runtime.cu:178-184.  manifest_path names manifest.json; weights.bin sits beside it. */
int ti_llm_create(const char* manifest_path, const ti_llm_options* options, ti_llm_model** out);
int ti_llm_destroy(ti_llm_model* model);                                   /* runtime.cu:185 */
int ti_llm_reset(ti_llm_model* model, int32_t slot);                       /* runtime.cu:186 */
int ti_llm_lengths(ti_llm_model* model, int32_t* out, int32_t count);      /* runtime.cu:187; count == cache_slots */
int ti_llm_get_trace(ti_llm_model* model, ti_llm_trace* out);              /* runtime.cu:188 */

/* Append tokens[B, token_stride] (lengths[B] >= 1 valid per row, padding ignored) to distinct
 * slots at each slot's current length.  last_logits (nullable) receives fp32 [B, 50257] of each
 * request's last position; next_tokens (nullable) the greedy argmax, lowest id on ties.
 * reference runtime.cu:157-168,189. */
int ti_llm_forward_batch(ti_llm_model* model, const int32_t* slots, const int32_t* tokens,
                         const int32_t* lengths, int32_t batch, int32_t token_stride,
                         float* last_logits, int32_t* next_tokens);

/* Greedy generation from empty distinct slots.  Every request produces exactly
 * max_new_tokens[i] ids (no EOS stop); output[B, output_stride] is padded with -1; the last id
 * of a request is returned but not appended to its cache.  ttft_ms / total_ms (nullable) are
 * host wall-clock milliseconds from entry to the first / last token of each request.
 * reference runtime.cu:190-203. */
int ti_llm_greedy_batch(ti_llm_model* model, const int32_t* slots, const int32_t* prompts,
                        const int32_t* prompt_lengths, const int32_t* max_new_tokens,
                        int32_t batch, int32_t prompt_stride, int32_t* output, int32_t output_stride,
                        int32_t* output_lengths, double* ttft_ms, double* total_ms);

/* Teacher-forced NLL of one window on an internal slot; public slots are untouched.
 * mask[0] == 0; position t (mask[t] == 1) is scored from the hidden state of t-1.
 * reference runtime.cu:204-210. */
int ti_llm_score_window(ti_llm_model* model, const int32_t* tokens, const uint8_t* mask,
                        int32_t length, double* sum_nll, uint64_t* target_count,
                        double* loss_by_position);
#ifdef __cplusplus
}
#endif
#endif
