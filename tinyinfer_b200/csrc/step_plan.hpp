// Description of a persistent decode step (decode_step.cuh), shared by the kernel and the host code that fills it.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>

#if defined(__CUDACC__)
#define TIB_HD __host__ __device__ __forceinline__
#else
#define TIB_HD inline
#endif

namespace tib {

constexpr int kStepRows = 32;          // requests per step (rows of the MMA tile)
constexpr int kStepMaxHidden = 1024;   // widest activation row the kernel stages in shared memory
constexpr int kStepMaxRanges = 8;      // K ranges (TMEM accumulators) of one item

// One INT8 matrix inside the tile arena: slab-major tiles [ceil(N/128)][slab_rows][128], first row tile_row0 of the arena.
struct StepLinear {
  int tile_row0 = 0, slab_rows = 0;
  const float* scales = nullptr;       // fp32 [N]
  const __half* bias = nullptr;        // fp16 [N] or null
};
struct StepLayer {
  StepLinear qkv, proj, fc, proj2;
  const __half *ln1_g = nullptr, *ln1_b = nullptr, *ln2_g = nullptr, *ln2_b = nullptr;
};

struct StepPlan {
  int hidden = 0, heads = 0, layers = 0, ff = 0, vocab = 0;
  // K rows per range of the K split each GEMM has in the launch-per-GEMM path (a function of N and K only)
  int chunk_qkv = 0, chunk_proj = 0, chunk_fc = 0, chunk_proj2 = 0, chunk_head = 0;
  int ranks_proj2 = 0;                 // ff / chunk_proj2: CTAs that share one slab of mlp.c_proj
  int head_slabs = 0;                  // ceil(vocab / 128)
  int first_helper = 0;                // CTAs below this index own a GEMM item in every layer
  int batch = 0;                       // requests of this step, 1..kStepRows
  float ln_eps = 1e-5f;
  const StepLayer* layer = nullptr;    // device array [layers]
  StepLinear head;
  const __half *lnf_g = nullptr, *lnf_b = nullptr, *wte = nullptr, *wpe = nullptr;
  // device-resident state of the decode segment
  int32_t *ids = nullptr, *row_pos = nullptr, *kv_len = nullptr;
  const int32_t* slots = nullptr;
  int32_t *step = nullptr, *log = nullptr;
  const int32_t* table = nullptr; int table_pitch = 0;
  __half *k_pool = nullptr, *v_pool = nullptr;
  // tagged exchange buffers (64-bit words), kStepRows rows each
  unsigned long long *xf = nullptr, *qkvf = nullptr, *attnf = nullptr, *resf = nullptr, *actf = nullptr, *partf = nullptr;
  unsigned int* sync = nullptr;        // [0] tag epoch, [1] finish tickets
  unsigned long long* best = nullptr;  // [kStepRows] argmax merge words, zero between steps
  float* logits = nullptr; int logits_pitch = 0;   // optional fp32 [batch][logits_pitch]
  // development builds (-DTIB_STEP_TIMELINE): [CTA][1024] words (event code << 48 | %globaltimer) of worker thread 0
  unsigned long long* timeline = nullptr;
};

// What CTA `cta` owns in every layer.  kind: 0 c_attn slab, 1 attn.c_proj slab, 2 c_fc slab, 3 (slab, K range) of
// mlp.c_proj, -1 nothing (helper).
struct StepRole { int kind, slab, rank; };
TIB_HD StepRole step_role(const StepPlan& p, int cta) {
  const int qkv = 3 * p.hidden / 128, proj = p.hidden / 128, fc = p.ff / 128;
  if (cta < qkv) return StepRole{0, cta, 0};
  cta -= qkv;
  if (cta < proj) return StepRole{1, cta, 0};
  cta -= proj;
  if (cta < fc) return StepRole{2, cta, 0};
  cta -= fc;
  if (cta < proj * p.ranks_proj2) return StepRole{3, cta / p.ranks_proj2, cta % p.ranks_proj2};
  return StepRole{-1, 0, 0};
}
TIB_HD int step_role_ctas(const StepPlan& p) { return 3 * p.hidden / 128 + p.hidden / 128 + p.ff / 128 + p.hidden / 128 * p.ranks_proj2; }

}  // namespace tib
