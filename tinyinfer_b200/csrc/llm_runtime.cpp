// Model C ABI v1 (include/tinyinfer_llm.h): GPT-2 forward / greedy / scoring on one GPU.
//
// Same observable behaviour as the reference runtime (llm/src/runtime.cu:97-211) -- argument
// validation before anything is enqueued, transactional slot lengths, poison on execution
// failure, exactly-N greedy tokens with the last one not appended, logical-operation trace
// counters -- on a different execution plan:
//   * rows are packed (a ragged prefill carries no padding rows);
//   * the KV history lives in a paged pool (32 positions per page) addressed through a per-slot
//     page table and is read in place by the attention kernels (the reference copies every
//     request's whole history into a packed buffer for every layer of every step);
//   * bias, GELU and the residual adds are epilogues of the weight-streaming GEMM, K/V are
//     written to their pages by one small kernel, heads are merged by the attention store;
//   * all per-call metadata reaches the GPU in one pinned-memory copy.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "artifact.hpp"
#include "launch.hpp"
#include "tinyinfer_b200_ext.h"
#include "tinyinfer_backend_v2.h"
#include "tinyinfer_llm.h"

namespace {

using tib::InvalidInput;
struct GpuFailure : std::runtime_error { using std::runtime_error::runtime_error; };

thread_local std::string g_error;

void ck(cudaError_t st) { if (st != cudaSuccess) throw GpuFailure(cudaGetErrorString(st)); }

struct DeviceGuard {
  int before = -1; bool switched = false;
  explicit DeviceGuard(int device) {
    ck(cudaGetDevice(&before));
    if (before != device) { ck(cudaSetDevice(device)); switched = true; }
  }
  ~DeviceGuard() { if (switched) cudaSetDevice(before); }
};

using Clock = std::chrono::steady_clock;
double elapsed_ms(Clock::time_point from) { return std::chrono::duration<double, std::milli>(Clock::now() - from).count(); }

constexpr int kScoreRows = 16;       // vocabulary rows scored per lm_head pass (reference SCORE_ROWS)
constexpr int kDecodeChunk = 128;    // keys per decode-attention CTA

struct Linear {
  const void* w = nullptr; const float* scales = nullptr; const void* bias = nullptr;
  int k = 0, n = 0; long long ldw = 0;
  int slab_rows = 0;                 // > 0: w holds slab-major tiles [ceil(n/128)][slab_rows][128] (int8 only)
  long long tile_row0 = 0;           // first row of those tiles inside the model's tile arena ([rows][128] int8)
  const void* image = nullptr;       // operand image of the matrix for many-row passes (tib::wide_image)
};
struct Block { const void *ln1_g, *ln1_b, *ln2_g, *ln2_b; Linear qkv, proj, fc, proj2; };

}  // namespace

struct ti_llm_model {
  ti_llm_options opt{};
  tib::ModelShape shape;
  bool int8 = false, poisoned = false;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;                 // results of steps launched ahead travel here, beside the next step
  ti_llm_trace trace{};
  std::vector<void*> owned;                      // cudaMalloc'ed
  std::vector<void*> pinned;                     // cudaMallocHost'ed
  // weights
  const void *wte = nullptr, *wpe = nullptr, *lnf_g = nullptr, *lnf_b = nullptr;
  std::vector<Block> blocks;
  Linear head; int vpitch = 0;
  // activations
  void *x = nullptr, *res = nullptr, *norm = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *last = nullptr;
  float* logits = nullptr;
  float *att_acc = nullptr, *att_ml = nullptr;
  int* att_counters = nullptr;                   // per (request, head) tickets of the decode attention, zero between launches
  int8_t* tile_arena = nullptr; long long tile_rows = 0;   // slab-major tiles of every INT8 matrix
  // KV pool
  void *k_pool = nullptr, *v_pool = nullptr;
  int pages_per_slot = 0;
  std::vector<int32_t> table, page_count, free_pages, lengths;
  int32_t* d_table = nullptr; bool table_dirty = true;
  // metadata staging: [ids | row_req | row_pos] (rows each) then 6 per-request arrays
  int32_t *h_meta = nullptr, *d_meta = nullptr; size_t max_rows = 0;
  int32_t *d_next = nullptr, *h_next = nullptr;
  unsigned int *h_status = nullptr, *d_status_addr = nullptr;
  // scoring
  int32_t* d_score_tokens = nullptr; uint8_t* d_score_mask = nullptr; double *d_loss = nullptr, *d_loss_sum = nullptr;

  template <class T> T* dev(size_t count) { void* p = nullptr; ck(cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T))); owned.push_back(p); return static_cast<T*>(p); }
  template <class T> T* host(size_t count) { void* p = nullptr; ck(cudaMallocHost(&p, std::max<size_t>(count, 1) * sizeof(T))); pinned.push_back(p); return static_cast<T*>(p); }

  ~ti_llm_model() {
    int before = -1;
    cudaGetDevice(&before);
    cudaSetDevice(opt.device);
    if (stream) cudaStreamSynchronize(stream);
    if (copy_stream) cudaStreamSynchronize(copy_stream);
    for (const StepGraph& g : graphs) cudaGraphExecDestroy(g.exec);
    for (cudaEvent_t e : spec_done) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : step_end) if (e) cudaEventDestroy(e);
    if (copy_stream) cudaStreamDestroy(copy_stream);
    for (void* p : owned) cudaFree(p);
    for (void* p : pinned) cudaFreeHost(p);
    if (stream) cudaStreamDestroy(stream);
    if (before >= 0) cudaSetDevice(before);
  }

  void ensure_usable() const { if (poisoned) throw GpuFailure("model poisoned by earlier execution failure; destroy/recreate required"); }

  // ------------------------------------------------------------ load
  void load(const tib::Artifact& art) {
    shape = art.shape; int8 = art.precision == "int8";
    const int H = shape.hidden, V = shape.vocab;
    const char* linear_dtype = int8 ? "int8" : "float16";
    uint8_t* blob = dev<uint8_t>(art.blob.size());
    ck(cudaMemcpyAsync(blob, art.blob.data(), art.blob.size(), cudaMemcpyHostToDevice, stream));
    size_t seen = 0;
    auto at = [&](const std::string& name, std::vector<int> dims, const char* dtype) -> const void* {
      ++seen; return blob + art.need(name, dims, dtype).offset;
    };
    auto linear = [&](const std::string& name, int k, int n, bool bias) {
      Linear l; l.k = k; l.n = n; l.ldw = n;
      l.w = at(name + ".weight", {k, n}, linear_dtype);
      if (bias) l.bias = at(name + ".bias", {n}, "float16");
      if (int8) l.scales = static_cast<const float*>(at(name + ".weight.scales", {n}, "float32"));
      return l;
    };
    wte = at("transformer.wte.weight", {V, H}, "float16");
    wpe = at("transformer.wpe.weight", {shape.positions, H}, "float16");
    lnf_g = at("transformer.ln_f.weight", {H}, "float16");
    lnf_b = at("transformer.ln_f.bias", {H}, "float16");
    blocks.resize(size_t(shape.layers));
    for (int l = 0; l < shape.layers; ++l) {
      const std::string p = "transformer.h." + std::to_string(l) + ".";
      Block& b = blocks[size_t(l)];
      b.ln1_g = at(p + "ln_1.weight", {H}, "float16"); b.ln1_b = at(p + "ln_1.bias", {H}, "float16");
      b.ln2_g = at(p + "ln_2.weight", {H}, "float16"); b.ln2_b = at(p + "ln_2.bias", {H}, "float16");
      b.qkv = linear(p + "attn.c_attn", H, 3 * H, true);
      b.proj = linear(p + "attn.c_proj", H, H, true);
      b.fc = linear(p + "mlp.c_fc", H, 4 * H, true);
      b.proj2 = linear(p + "mlp.c_proj", 4 * H, H, true);
    }
    head = linear("lm_head", H, V, false);
    if (seen != art.tensors.size()) throw InvalidInput("unexpected tensor(s) in artifact");
    // The vocabulary projection is re-pitched so its rows start on 128-byte boundaries and can be
    // streamed by TMA; the pad columns are zero weights that are never stored.
    vpitch = (V + 127) / 128 * 128;
    const size_t esize = int8 ? 1 : 2;
    uint8_t* padded = dev<uint8_t>(size_t(H) * vpitch * esize);
    ck(cudaMemsetAsync(padded, 0, size_t(H) * vpitch * esize, stream));
    ck(cudaMemcpy2DAsync(padded, size_t(vpitch) * esize, head.w, size_t(V) * esize, size_t(V) * esize, size_t(H),
                         cudaMemcpyDeviceToDevice, stream));
    head.w = padded; head.ldw = vpitch;
    // INT8 matrices are re-tiled once into slab-major order: the 128 output channels of a CTA become
    // one contiguous run of K x 128 bytes, so each TMA stage is a single 8 KB block of device memory
    // instead of 64 separate 128-byte pieces one matrix row apart.
    bool tiled = int8 && H % 8 == 0;
#ifdef TIB_DEV_KNOBS
    if (const char* v = std::getenv("TINYINFER_B200_TILED")) tiled = tiled && std::atoi(v) != 0;
#endif
    {
      // Many-row passes (prefill) read every matrix from its operand image -- the fp16 values the INT8 weights dequantise
      // to, already in the layout the tensor cores read -- instead of converting each weight once per row tile; decode
      // keeps the int8 tiles (half the bytes).  Built here, before the int8 pointers move to the tile arena.  About twice
      // the bytes of the INT8 weights (247 MB for GPT-2 small).
      auto widen = [&](Linear& l) {
        void* image = dev<uint8_t>(tib::wide_image_bytes(l.k, l.n));
        ck(tib::wide_image(int8 ? static_cast<const int8_t*>(l.w) : nullptr, int8 ? nullptr : l.w, l.ldw, l.scales, image, l.k, l.n, stream));
        l.image = image;
      };
      for (Block& b : blocks) { widen(b.qkv); widen(b.proj); widen(b.fc); widen(b.proj2); }
    }
    if (tiled) {
      // One arena holds the tiles of every matrix, so that a single tensor map (and a row offset per matrix) reaches
      // all of them: the persistent decode step streams the weights of a whole step through it.
      std::vector<Linear*> all;
      for (Block& b : blocks) { all.push_back(&b.qkv); all.push_back(&b.proj); all.push_back(&b.fc); all.push_back(&b.proj2); }
      all.push_back(&head);
      long long rows_total = 0;
      for (Linear* l : all) { l->slab_rows = (l->k + 63) / 64 * 64; l->tile_row0 = rows_total; rows_total += (long long)((l->n + 127) / 128) * l->slab_rows; }
      tile_arena = dev<int8_t>(size_t(rows_total) * 128); tile_rows = rows_total;
      for (Linear* l : all) {
        int8_t* tiles = tile_arena + size_t(l->tile_row0) * 128;
        ck(tib::retile_i8(static_cast<const int8_t*>(l->w), l->ldw, l->k, l->n, tiles, l->slab_rows, stream));
        l->w = tiles;
      }
    }

    max_rows = size_t(opt.max_batch) * opt.capacity;
    const size_t r = max_rows;
    x = dev<uint16_t>(r * H); res = dev<uint16_t>(r * H); norm = dev<uint16_t>(r * H); attn = dev<uint16_t>(r * H);
    qkv = dev<uint16_t>(r * 3 * H); act = dev<uint16_t>(r * 4 * H);
    last = dev<uint16_t>(size_t(std::max(opt.max_batch, kScoreRows)) * H);
    logits = dev<float>(size_t(std::max(opt.max_batch, kScoreRows)) * vpitch);
    int chunks = 1;                                              // decode segments round the chunk count up to a power of two
    while (chunks * kDecodeChunk < opt.capacity) chunks *= 2;
    att_acc = dev<float>(size_t(opt.max_batch) * shape.heads * chunks * 64);
    att_ml = dev<float>(size_t(opt.max_batch) * shape.heads * chunks * 2);
    att_counters = dev<int>(size_t(opt.max_batch) * shape.heads);
    ck(cudaMemsetAsync(att_counters, 0, size_t(opt.max_batch) * shape.heads * sizeof(int), stream));

    pages_per_slot = (opt.capacity + tib_page_tokens() - 1) / tib_page_tokens();
    const int slots = opt.cache_slots + 1;                       // +1: private slot of score_window
    const size_t pages = size_t(slots) * pages_per_slot;
    const size_t page_halfs = size_t(shape.layers) * shape.heads * tib_page_tokens() * 64;
    k_pool = dev<uint16_t>(pages * page_halfs); v_pool = dev<uint16_t>(pages * page_halfs);
    table.assign(size_t(slots) * pages_per_slot, 0); page_count.assign(size_t(slots), 0); lengths.assign(size_t(slots), 0);
    free_pages.resize(pages);
    for (size_t i = 0; i < pages; ++i) free_pages[i] = int32_t(pages - 1 - i);
    d_table = dev<int32_t>(table.size());

    const size_t meta = 3 * r + 6 * size_t(opt.max_batch);
    h_meta = host<int32_t>(meta); d_meta = dev<int32_t>(meta);
    d_next = dev<int32_t>(size_t(opt.max_batch)); h_next = host<int32_t>(size_t(opt.max_batch));
    d_seg = dev<int32_t>(size_t(5) * opt.max_batch); h_seg = host<int32_t>(size_t(5) * opt.max_batch);
    d_step = dev<int32_t>(1);
    for (int i = 0; i < 2; ++i) {
      h_spec[i] = host<int32_t>(size_t(opt.max_batch) + 1);
      ck(cudaEventCreateWithFlags(&spec_done[i], cudaEventDisableTiming));
      ck(cudaEventCreateWithFlags(&step_end[i], cudaEventDisableTiming));
    }
    ck(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
    if (const char* v = std::getenv("TINYINFER_B200_SPECULATE")) { spec_after = std::atoi(v); speculate = spec_after > 0; }
    d_argmax = dev<uint8_t>(size_t(12) * opt.max_batch + 8);
    ck(cudaMemsetAsync(d_argmax, 0, size_t(12) * opt.max_batch + 8, stream));
    d_best = dev<unsigned long long>(64);
    ck(cudaMemsetAsync(d_best, 0, 64 * sizeof(unsigned long long), stream));
    d_log = dev<int32_t>(size_t(opt.capacity) * opt.max_batch); h_log = host<int32_t>(size_t(opt.capacity) * opt.max_batch);
    if (const char* v = std::getenv("TINYINFER_B200_GRAPH")) use_graph = std::atoi(v) != 0;   // debugging aids: 0 = plain launches
    if (const char* v = std::getenv("TINYINFER_B200_PDL")) use_pdl = std::atoi(v) != 0;
#ifdef TIB_DEV_KNOBS                 // measurement aids of development builds
    if (const char* v = std::getenv("TINYINFER_B200_ATTN_EARLY")) attn_early = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_LN_TRIGGER")) ln_trigger = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_GEMM_TRIGGER")) gemm_trigger = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_MIXED_ATTN")) mixed_attention = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_TC_ATTN")) tc_attention = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_WIDE_GEMM")) wide_gemm = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_ATTN_TRIGGER")) attn_trigger = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_ATTN_WHOLE")) attn_whole = std::atoi(v) != 0;
    if (const char* v = std::getenv("TINYINFER_B200_FUSE_LN")) fuse_ln_rows = std::min(1024, std::atoi(v));
#endif
    fuse_ln = int8 && shape.hidden <= 1024 && fuse_ln_rows > 0;
    h_status = host<unsigned int>(1); *h_status = 0;
    d_score_tokens = dev<int32_t>(size_t(opt.capacity)); d_score_mask = dev<uint8_t>(size_t(opt.capacity));
    d_loss = dev<double>(size_t(opt.capacity)); d_loss_sum = dev<double>(1);
    build_step_plan();
    ck(cudaStreamSynchronize(stream));
  }

  // ------------------------------------------------------------ persistent decode step
  // One launch per greedy step for up to 32 requests (decode_step.cuh) instead of the 65-kernel graph; same bits.
  // Off unless selected (ti_b200_llm_decode_plan, TINYINFER_B200_PERSISTENT=1): measured on a B200 it trails the graph of
  // separate kernels at every batch size (its GEMM items span the whole K, six to twelve dequantisation stages on one SM
  // where the separate kernels split K over a cluster), so it is kept as the second, bit-identical plan.
  tib::StepPlan plan; tib::TileMap plan_tiles; bool plan_ready = false, use_persistent = false;
  uint8_t* plan_words = nullptr; size_t plan_words_bytes = 0;     // the tagged exchange buffers, one allocation
  uint64_t plan_epochs = 0;                                        // launches since the buffers were last cleared

  void build_step_plan() {
    if (!tile_arena || shape.hidden % 128 || shape.hidden > tib::kStepMaxHidden) return;
    const int H = shape.hidden, F = 4 * H;
    tib::StepPlan p;
    p.hidden = H; p.heads = shape.heads; p.layers = shape.layers; p.ff = F; p.vocab = shape.vocab;
    p.chunk_qkv = tib::step_k_chunk(3 * H, H); p.chunk_proj = tib::step_k_chunk(H, H); p.chunk_fc = tib::step_k_chunk(F, H);
    p.chunk_proj2 = tib::step_k_chunk(H, F); p.chunk_head = tib::step_k_chunk(shape.vocab, H);
    p.ranks_proj2 = p.chunk_proj2 > 0 ? F / p.chunk_proj2 : 0;
    p.head_slabs = (shape.vocab + 127) / 128; p.first_helper = tib::step_role_ctas(p);
    if (tib::step_unsupported(p)) return;
    auto lin = [](const Linear& l) { tib::StepLinear s; s.tile_row0 = int(l.tile_row0); s.slab_rows = l.slab_rows; s.scales = l.scales; s.bias = static_cast<const __half*>(l.bias); return s; };
    if (tile_rows > 0x7fffffffLL) return;
    std::vector<tib::StepLayer> layers(blocks.size());
    for (size_t l = 0; l < blocks.size(); ++l) {
      const Block& b = blocks[l];
      layers[l].qkv = lin(b.qkv); layers[l].proj = lin(b.proj); layers[l].fc = lin(b.fc); layers[l].proj2 = lin(b.proj2);
      layers[l].ln1_g = static_cast<const __half*>(b.ln1_g); layers[l].ln1_b = static_cast<const __half*>(b.ln1_b);
      layers[l].ln2_g = static_cast<const __half*>(b.ln2_g); layers[l].ln2_b = static_cast<const __half*>(b.ln2_b);
    }
    tib::StepLayer* d_layers = dev<tib::StepLayer>(layers.size());
    ck(cudaMemcpyAsync(d_layers, layers.data(), layers.size() * sizeof(tib::StepLayer), cudaMemcpyHostToDevice, stream));
    ck(cudaStreamSynchronize(stream));                             // `layers` is a local
    p.layer = d_layers; p.head = lin(head);
    p.lnf_g = static_cast<const __half*>(lnf_g); p.lnf_b = static_cast<const __half*>(lnf_b);
    p.wte = static_cast<const __half*>(wte); p.wpe = static_cast<const __half*>(wpe);
    p.ids = seg(0); p.row_pos = seg(2); p.kv_len = seg(3); p.slots = seg(4); p.step = d_step; p.log = d_log;
    p.table = d_table; p.table_pitch = pages_per_slot;
    p.k_pool = static_cast<__half*>(k_pool); p.v_pool = static_cast<__half*>(v_pool);
    // tagged buffers: 8 bytes per pair of fp16 values (or per fp32 partial sum), 32 rows each
    const size_t R = tib::kStepRows;
    const size_t words_x = R * H / 2, words_qkv = R * 3 * H / 2, words_act = R * F / 2, words_part = size_t(H / 128) * p.ranks_proj2 * R * 128;
    const size_t total = 3 * words_x + words_qkv + words_act + words_part;
    plan_words_bytes = total * 8 + 16 + R * 8;
    plan_words = dev<uint8_t>(plan_words_bytes);
    ck(cudaMemsetAsync(plan_words, 0, plan_words_bytes, stream));
    auto* w = reinterpret_cast<unsigned long long*>(plan_words);
    p.xf = w; w += words_x; p.attnf = w; w += words_x; p.resf = w; w += words_x; p.qkvf = w; w += words_qkv; p.actf = w; w += words_act;
    p.partf = w; w += words_part;
    p.best = w; w += R;
    p.sync = reinterpret_cast<unsigned int*>(w);
    const unsigned int first_epoch[2] = {1u, 0u};
    ck(cudaMemcpyAsync(p.sync, first_epoch, sizeof first_epoch, cudaMemcpyHostToDevice, stream));
    ck(cudaStreamSynchronize(stream));
    p.logits_pitch = vpitch;
    ck(tib::make_tile_map(tile_arena, tile_rows, &plan_tiles));
#ifdef TIB_STEP_TIMELINE
    p.timeline = dev<unsigned long long>(size_t(256) * 1024);
    ck(cudaMemsetAsync(p.timeline, 0, size_t(256) * 1024 * 8, stream));
#endif
    plan = p; plan_ready = true; plan_epochs = 0;
    if (const char* v = std::getenv("TINYINFER_B200_PERSISTENT")) use_persistent = std::atoi(v) != 0;
  }
  bool persistent_step(int batch) const { return plan_ready && use_persistent && int8 && batch <= tib::kStepRows; }
  void launch_persistent(int batch, bool want_logits) {
    if (++plan_epochs > (1ull << 25)) {                            // long before the 32-bit tags could repeat
      ck(cudaMemsetAsync(plan_words, 0, plan_words_bytes, stream));
      const unsigned int first_epoch[2] = {1u, 0u};
      ck(cudaMemcpyAsync(plan.sync, first_epoch, sizeof first_epoch, cudaMemcpyHostToDevice, stream));   // pageable source: copied before the call returns
      plan_epochs = 1;
    }
    tib::StepPlan p = plan;
    p.batch = batch; p.logits = want_logits ? logits : nullptr;
    ck(tib::decode_step(p, plan_tiles, stream));
  }
  static int tib_page_tokens() { return 32; }

  // ------------------------------------------------------------ paging
  void reserve(int slot, int new_length) {
    const int need = (new_length + tib_page_tokens() - 1) / tib_page_tokens();
    while (page_count[size_t(slot)] < need) {
      if (free_pages.empty()) throw std::runtime_error("KV page pool exhausted");
      table[size_t(slot) * pages_per_slot + page_count[size_t(slot)]++] = free_pages.back();
      free_pages.pop_back();
      table_dirty = true;
    }
  }
  void release(int slot) {
    spec.armed = false; spec.inflight = 0;
    for (int i = page_count[size_t(slot)] - 1; i >= 0; --i) free_pages.push_back(table[size_t(slot) * pages_per_slot + i]);
    page_count[size_t(slot)] = 0; lengths[size_t(slot)] = 0;
  }

  // ------------------------------------------------------------ one pass over the layers
  // ln_g / ln_b: LayerNorm applied to `a` inside the GEMM (decode-sized calls only, see fuse_ln).
  void gemm(const void* a, const Linear& l, void* out, int rows, bool fp32, const void* residual, bool gelu,
            const tib::PagedKv* kv = nullptr, const int32_t* row_req = nullptr, const int32_t* row_pos = nullptr,
            const void* ln_g = nullptr, const void* ln_b = nullptr, void* argmax_best = nullptr, bool skip_store = false) {
    tib::GemmCall c;
    c.argmax_best = argmax_best; c.skip_store = skip_store;
    c.kv = kv; c.kv_row_req = row_req; c.kv_row_pos = row_pos; c.ln_gamma = ln_g; c.ln_beta = ln_b;
    c.a = a; c.lda = l.k; c.w = l.w; c.ldw = l.ldw; c.w_slab_rows = l.slab_rows; c.w_int8 = int8; c.scales = l.scales; c.bias = l.bias;
    if (wide_gemm) c.w_image = l.image;
    c.out = out; c.ldo = fp32 ? vpitch : l.n; c.out_fp32 = fp32; c.residual = residual; c.gelu = gelu;
    c.m = rows; c.n = l.n; c.k = l.k;
    // One kernel family for every batch size: logits of a request are bit-identical whatever it is
    // batched with, the property the reference's gates rely on (llm/gpu_correctness.py:62-66).
    c.uniform_numerics = true;
    tib::LaunchOpts o; o.stream = stream; o.pdl = use_pdl; o.early_trigger = gemm_trigger;
    ck(tib::gemm(c, o));
  }

  // Device-resident description of the rows of one pass.
  struct Meta {
    const int32_t *ids, *row_req, *row_pos;                       // per row
    const int32_t *row_start, *qlens, *offsets, *kvlens, *slots;   // per request
    int rows, batch, max_q, max_kv;
    int singles;                                                  // requests with exactly one row in this pass
    int longs;                                                    // requests with at least 64 rows (tensor-core attention)
  };

  // Embedding and every transformer block; leaves the final hidden state in `x`.
  void run_layers(const Meta& m) {
    const int H = shape.hidden;
    tib::LaunchOpts o; o.stream = stream; o.pdl = use_pdl;
    ck(tib::embed(m.ids, m.row_pos, wte, wpe, x, m.rows, H, shape.vocab, o));
    tib::PagedKv kv; kv.k_pool = k_pool; kv.v_pool = v_pool; kv.table = d_table; kv.slots = m.slots;
    kv.table_pitch = pages_per_slot; kv.layers = shape.layers; kv.heads = shape.heads; kv.head_dim = 64;
    for (int l = 0; l < shape.layers; ++l) {
      const Block& b = blocks[size_t(l)];
      kv.layer = l;
      // LayerNorm as a prologue of the consuming GEMM for decode-sized passes (one 32-row tile): up to 8 rows every CTA
      // computes the row statistics itself, beyond that the CTAs of a K-split cluster share the rows out.
      const bool fused = fuse_ln && m.rows <= fuse_ln_rows;
      if (fused) gemm(x, b.qkv, qkv, m.rows, false, nullptr, false, &kv, m.row_req, m.row_pos, b.ln1_g, b.ln1_b);
      else {
        ck(tib::layernorm(x, nullptr, b.ln1_g, b.ln1_b, norm, m.rows, H, 1e-5f, ln_opts()));
        gemm(norm, b.qkv, qkv, m.rows, false, nullptr, false, &kv, m.row_req, m.row_pos);   // Q -> qkv buffer, K/V -> their pages
      }
      if (m.max_q == 1) {
        ck(tib::attention_paged_decode(qkv, attn, m.kvlens, m.batch, m.max_kv, kDecodeChunk, att_acc, att_ml, att_counters, kv, o, attn_early, attn_whole, attn_trigger));
      } else {
        // Prompts and single tokens in one pass (the server folds admissions into a decode step): the single-token
        // requests take the decode kernel -- the same arithmetic as in a pure decode step, so their tokens do not
        // depend on what else is admitted -- and the tile kernel skips them.
        const bool split = attn_whole && mixed_attention && m.singles > 0;
        if (split) ck(tib::attention_paged_decode(qkv, attn, m.kvlens, m.batch, m.max_kv, kDecodeChunk, att_acc, att_ml, att_counters, kv, o,
                                                  false, true, false, m.row_start, m.qlens));
        const int shorts = m.batch - m.longs - (split ? m.singles : 0);
        ck(tib::attention_paged(qkv, attn, m.row_start, m.qlens, m.kvlens, m.offsets, m.batch, m.max_q, m.max_kv, kv, o, split,
                                tc_attention ? m.longs : 0, tc_attention ? shorts : 1));
      }
      gemm(attn, b.proj, res, m.rows, false, x, false);             // res = x + proj(attn)
      if (fused) gemm(res, b.fc, act, m.rows, false, nullptr, true, nullptr, nullptr, nullptr, b.ln2_g, b.ln2_b);
      else {
        ck(tib::layernorm(res, nullptr, b.ln2_g, b.ln2_b, norm, m.rows, H, 1e-5f, ln_opts()));
        gemm(norm, b.fc, act, m.rows, false, nullptr, true);        // act = gelu(fc(norm))
      }
      gemm(act, b.proj2, x, m.rows, false, res, false);             // x = res + proj2(act)
    }
  }
  // Logical operations of one pass, counted as the reference counts its separate kernels
  // (llm/src/runtime.cu:131-165) although several of them are fused here.
  void count_pass() {
    const uint64_t L = uint64_t(shape.layers);
    ++trace.forward_calls; ++trace.embedding;
    trace.layernorm += 2 * L + 1; (int8 ? trace.gemm_int8 : trace.gemm_fp16) += 4 * L;
    trace.kv_scatter_gather += L; trace.attention += L; trace.residual += 2 * L; trace.gelu += L;
  }
  void count_head(bool with_argmax) { ++trace.lm_head; ++(int8 ? trace.gemm_int8 : trace.gemm_fp16); if (with_argmax) ++trace.argmax; }

  void upload_table() {
    if (!table_dirty) return;
    ck(cudaMemcpyAsync(d_table, table.data(), table.size() * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    table_dirty = false;
  }

  // General pass (prefill, mixed lengths, scoring).  slots/lens describe the requests; tokens are
  // packed request after request.  LayerNorm_f of each request's last row lands in `last`, or of
  // every row in `norm` when all_rows is set.
  void transform(const std::vector<int32_t>& ss, const std::vector<int32_t>& packed, const std::vector<int32_t>& lens, bool all_rows) {
    spec.armed = false; spec.inflight = 0; spec.streak = 0;
    const int batch = int(ss.size()), H = shape.hidden;
    Meta m{}; m.batch = batch;
    for (int b = 0; b < batch; ++b) {
      m.rows += lens[size_t(b)]; m.max_q = std::max(m.max_q, lens[size_t(b)]); m.singles += lens[size_t(b)] == 1; m.longs += lens[size_t(b)] >= 64;
    }
    const int rows = m.rows;
    int32_t* ids = h_meta; int32_t* row_req = ids + rows; int32_t* row_pos = row_req + rows; int32_t* per = row_pos + rows;
    int32_t *row_start = per, *qlens = per + batch, *offsets = per + 2 * batch, *kvlens = per + 3 * batch,
            *slot_of = per + 4 * batch, *last_row = per + 5 * batch;
    int r = 0;
    for (int b = 0; b < batch; ++b) {
      const int s = ss[size_t(b)], n = lens[size_t(b)], start = lengths[size_t(s)];
      reserve(s, start + n);
      row_start[b] = r; qlens[b] = n; offsets[b] = start; kvlens[b] = start + n; slot_of[b] = s; last_row[b] = r + n - 1;
      m.max_kv = std::max(m.max_kv, start + n);
      for (int t = 0; t < n; ++t, ++r) { ids[r] = packed[size_t(r)]; row_req[r] = b; row_pos[r] = start + t; }
    }
    upload_table();
    ck(cudaMemcpyAsync(d_meta, h_meta, size_t(3 * rows + 6 * batch) * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    const int32_t* per_d = d_meta + 3 * rows;
    m.ids = d_meta; m.row_req = d_meta + rows; m.row_pos = d_meta + 2 * rows;
    m.row_start = per_d; m.qlens = per_d + batch; m.offsets = per_d + 2 * batch; m.kvlens = per_d + 3 * batch; m.slots = per_d + 4 * batch;
    // A one-token-per-request pass through this path (e.g. with logits requested) still uses the tile
    // attention when any request is longer; decode attention needs max_q == 1.
    count_pass();
    run_layers(m);
    tib::LaunchOpts o; o.stream = stream; o.pdl = use_pdl;
    if (all_rows) ck(tib::layernorm(x, nullptr, lnf_g, lnf_b, norm, rows, H, 1e-5f, o));
    else ck(tib::layernorm(x, per_d + 5 * batch, lnf_g, lnf_b, last, batch, H, 1e-5f, o));
  }

  void finish() {
    ck(cudaMemcpyAsync(h_status, d_status_addr, sizeof(unsigned int), cudaMemcpyDeviceToHost, stream));
    ck(cudaStreamSynchronize(stream));
    if (*h_status) {
      const unsigned int code = *h_status; *h_status = 0;
      unsigned int ignored = 0; tib::read_device_status(stream, &ignored);
      throw GpuFailure("device wait timed out (status " + std::to_string(code) + ")");
    }
  }

  // ------------------------------------------------------------ device-resident greedy decode
  // A decode segment keeps its state on the GPU: d_seg = [ids | row_req | row_pos | kvlens | slots]
  // (max_batch each) and a step counter.  One step = embedding .. lm_head .. argmax, whose winner is
  // written straight into ids[] (next step's input) and into d_log[step][request]; a last small
  // kernel advances positions, lengths and the counter.  Nothing returns to the host between steps,
  // so a step can be replayed as a CUDA graph; graphs are cached per (batch, attention chunk count).
  struct StepGraph { int batch, chunks; bool logits; cudaGraphExec_t exec; };
  std::vector<StepGraph> graphs;
  uint8_t* d_argmax = nullptr;      // per-row merge words of the argmax kernel (zero between launches)
  unsigned long long* d_best = nullptr;   // per-row merge words of the argmax fused into the vocabulary projection (zero between steps)
  // Speculative continuation of step-by-step decoding through ti_llm_forward_batch: once a caller has fed back the
  // model's own outputs for the same slots `spec_after` times in a row, the next step is launched from the state that
  // is already on the GPU before the call returns; the following call only checks that it asks for exactly that step
  // (same slots, the ids just returned, untouched lengths) and collects the result.  A call that asks for anything else
  // simply finds an extra step ahead of its work in the stream; that step's writes (a K/V row at a position the next
  // real step rewrites, device-side counters that every call re-uploads) are never read.
  // Up to two such steps are in flight: when a call finds its step under way it first launches the one after it and
  // only then waits (on an event, not on the stream) for its own ids, so the GPU never idles between steps.
  struct Speculation {
    bool armed = false;                               // inflight > 0 and nothing but matching forward calls since
    int inflight = 0, oldest = 0;                     // steps launched ahead, and which buffer the oldest one fills
    int streak = 0;                                   // consecutive calls that continued the previous one
    std::vector<int32_t> slots, last_out, lens_expected;
  } spec;
  bool speculate = true;
  int spec_after = 8, host_step = 0;                  // host_step mirrors the device step counter
  int32_t* h_spec[2] = {nullptr, nullptr};            // pinned: ids of a step launched ahead, then the device status word
  cudaEvent_t spec_done[2] = {nullptr, nullptr}, step_end[2] = {nullptr, nullptr};
  int32_t *d_seg = nullptr, *h_seg = nullptr, *d_step = nullptr, *d_log = nullptr, *h_log = nullptr;
  bool use_graph = true, use_pdl = true;
  // Early release of the next launch (see LaunchOpts::early_trigger).  After a GEMM comes a kernel whose reads ahead
  // of its own wait are constants or state of earlier steps (LayerNorm parameters, weights, the cache history), so it
  // may start at once; measured: a few microseconds per step at small batches.  After a LayerNorm it did not pay.
  bool ln_trigger = false, gemm_trigger = true;
  tib::LaunchOpts ln_opts() const { tib::LaunchOpts o; o.stream = stream; o.pdl = use_pdl; o.early_trigger = ln_trigger; return o; }
  bool wide_gemm = true;                         // passes of 129 rows and more run their GEMMs from the operand images
  bool tc_attention = true;                      // requests with 64 or more rows in a pass: attention on the tensor cores
  bool mixed_attention = true;                   // mixed passes: single-token requests through the decode kernel
  bool attn_trigger = true;                      // the projection GEMM after attention prefetches its weights meanwhile
  bool attn_early = true, attn_whole = true;     // decode attention: reads ahead of the dependency wait; one CTA per (request, head)
  int fuse_ln_rows = 128;            // largest row count whose LayerNorms run inside the consuming GEMM
  bool fuse_ln = false;             // int8 weights and rows of at most 1024 values: LayerNorm runs inside the consuming GEMM

  int32_t* seg(int field) const { return d_seg + size_t(field) * opt.max_batch; }

  // want_logits: the fp32 logits are stored too (a caller asked for them); the greedy argmax is merged by the vocabulary
  // projection itself either way (int8 weights: the tensor-core kernel), so a greedy step never reads logits back.
  void enqueue_step(int batch, int max_kv, bool want_logits) {
    Meta m{};
    m.ids = seg(0); m.row_req = seg(1); m.row_pos = seg(2); m.kvlens = seg(3); m.slots = seg(4);
    m.rows = batch; m.batch = batch; m.max_q = 1; m.max_kv = max_kv;
    run_layers(m);
    tib::LaunchOpts o; o.stream = stream; o.pdl = use_pdl;
    void* best = int8 ? d_best : nullptr;
    const bool skip = best && !want_logits;
    if (fuse_ln && shape.hidden <= 768 && batch <= std::min(fuse_ln_rows, 8))
      gemm(x, head, logits, batch, true, nullptr, false, nullptr, nullptr, nullptr, lnf_g, lnf_b, best, skip);
    else {
      ck(tib::layernorm(x, nullptr, lnf_g, lnf_b, last, batch, shape.hidden, 1e-5f, ln_opts()));
      gemm(last, head, logits, batch, true, nullptr, false, nullptr, nullptr, nullptr, nullptr, nullptr, best, skip);
    }
    if (best) ck(tib::argmax_finish(best, batch, shape.vocab, d_log, seg(0), d_step, seg(2), seg(3), o));
    else {
      ck(tib::argmax(logits, vpitch, batch, shape.vocab, d_log, seg(0), d_step, d_argmax, o));
      ck(tib::advance(seg(2), seg(3), d_step, batch, o));
    }
  }

  cudaGraphExec_t step_graph(int batch, int chunks, bool want_logits = false) {
    for (const StepGraph& g : graphs) if (g.batch == batch && g.chunks == chunks && g.logits == want_logits) return g.exec;
    cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr;
    ck(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    try { enqueue_step(batch, chunks * kDecodeChunk, want_logits); }
    catch (...) { cudaStreamEndCapture(stream, &graph); if (graph) cudaGraphDestroy(graph); throw; }
    ck(cudaStreamEndCapture(stream, &graph));
    const cudaError_t st = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    ck(st);
    graphs.push_back({batch, chunks, want_logits, exec});
    return exec;
  }

  // Runs `steps` greedy steps for the requests in ss, starting from input ids `first`; the ids
  // produced land in h_log[step * batch + request] once finish() has returned.  Does not touch
  // `lengths` (the caller advances them) but reserves the pages the steps will write.
  // before / after, when given, are recorded around the steps on the model's stream.
  void enqueue_segment(const std::vector<int32_t>& ss, const int32_t* first, int steps, cudaEvent_t before = nullptr,
                       cudaEvent_t after = nullptr, bool want_logits = false) {
    const int batch = int(ss.size()), mb = opt.max_batch;
    spec.armed = false; spec.inflight = 0; host_step = steps;
    int max_kv = 0;
    for (int b = 0; b < batch; ++b) {
      const int s = ss[size_t(b)], start = lengths[size_t(s)];
      reserve(s, start + steps);
      h_seg[b] = first[b]; h_seg[mb + b] = b; h_seg[2 * mb + b] = start; h_seg[3 * mb + b] = start + 1; h_seg[4 * mb + b] = s;
      max_kv = std::max(max_kv, start + steps);
    }
    upload_table();
    ck(cudaMemcpyAsync(d_seg, h_seg, size_t(5) * mb * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    ck(cudaMemsetAsync(d_step, 0, sizeof(int32_t), stream));
    int chunks = 1;
    while (chunks * kDecodeChunk < max_kv) chunks *= 2;            // few distinct graphs: 1, 2, 4, 8 chunks
    if (before) ck(cudaEventRecord(before, stream));
    if (persistent_step(batch)) {
      for (int i = 0; i < steps; ++i) launch_persistent(batch, want_logits);
    } else if (use_graph) {
      cudaGraphExec_t exec = step_graph(batch, chunks, want_logits);
      for (int i = 0; i < steps; ++i) ck(cudaGraphLaunch(exec, stream));
    } else {
      for (int i = 0; i < steps; ++i) enqueue_step(batch, chunks * kDecodeChunk, want_logits);
    }
    if (after) ck(cudaEventRecord(after, stream));
    ck(cudaMemcpyAsync(h_log, d_log, size_t(steps) * batch * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    for (int i = 0; i < steps; ++i) { count_pass(); count_head(true); }
  }

  // ------------------------------------------------------------ ABI bodies
  int fail_after = -1;                               // test hook (ti_b200_llm_inject_failure): forward calls left before one fails
  void forward(const int32_t* s, const int32_t* tokens, const int32_t* lens, int batch, int stride, float* out, int32_t* greedy,
               bool internal = false) {
    ensure_usable();
    if (!s || !tokens || !lens || batch < 1 || batch > opt.max_batch || stride < 1 || stride > opt.capacity)
      throw InvalidInput("invalid batch/host pointers/stride");
    std::vector<int32_t> ss(s, s + batch), ll(lens, lens + batch), packed;
    std::vector<char> used(size_t(opt.cache_slots) + 1, 0);
    bool single = true;
    for (int b = 0; b < batch; ++b) {
      const int slot = s[b], n = lens[b];
      if (slot < 0 || slot >= opt.cache_slots + (internal ? 1 : 0) || used[size_t(slot)] || n < 1 || n > stride ||
          lengths[size_t(slot)] + n > opt.capacity)
        throw InvalidInput("duplicate/invalid slot, length or capacity");
      used[size_t(slot)] = 1; single = single && n == 1;
      for (int t = 0; t < n; ++t) {
        const int32_t id = tokens[size_t(b) * stride + t];
        if (id < 0 || id >= shape.vocab) throw InvalidInput("token ID outside GPT-2 vocabulary");
        packed.push_back(id);
      }
    }
    if (fail_after >= 0 && fail_after-- == 0) throw GpuFailure("injected execution failure (test hook)");   // after validation, like a failed launch
    if (single && greedy) {
      // One token per request and the argmax wanted: one device-resident step -- already under way if this call
      // continues the previous one exactly (see Speculation).
      bool hit = spec.armed && spec.inflight > 0 && !out && ss == spec.slots && packed == spec.last_out;
      for (int b = 0; hit && b < batch; ++b) hit = lengths[size_t(s[b])] == spec.lens_expected[size_t(b)];
      const bool continues = !out && ss == spec.slots && packed == spec.last_out;
      // One more step ahead of the `spec.inflight` already launched, if there is room for the position it writes.
      auto launch_ahead = [&]() -> bool {
        if (!speculate || !(use_graph || persistent_step(batch)) || spec.inflight >= 2 || host_step + 1 >= opt.capacity) return false;
        int max_kv = 0;
        for (int b = 0; b < batch; ++b) {
          const int rows = lengths[size_t(s[b])] + spec.inflight + 1;
          if (rows > opt.capacity) return false;
          max_kv = std::max(max_kv, rows);
        }
        for (int b = 0; b < batch; ++b) reserve(s[b], lengths[size_t(s[b])] + spec.inflight + 1);
        upload_table();
        int chunks = 1;
        while (chunks * kDecodeChunk < max_kv) chunks *= 2;
        const int buffer = (spec.oldest + spec.inflight) & 1;
        if (persistent_step(batch)) launch_persistent(batch, false);
        else ck(cudaGraphLaunch(step_graph(batch, chunks), stream));
        // the step's ids and the status word go home on the side stream: the next step does not queue behind the copies
        ck(cudaEventRecord(step_end[buffer], stream));
        ck(cudaStreamWaitEvent(copy_stream, step_end[buffer], 0));
        ck(cudaMemcpyAsync(h_spec[buffer], d_log + size_t(host_step) * batch, size_t(batch) * sizeof(int32_t), cudaMemcpyDeviceToHost, copy_stream));
        ck(cudaMemcpyAsync(h_spec[buffer] + opt.max_batch, d_status_addr, sizeof(unsigned int), cudaMemcpyDeviceToHost, copy_stream));
        ck(cudaEventRecord(spec_done[buffer], copy_stream));
        ++host_step; ++spec.inflight;
        return true;
      };
      if (hit) {
        launch_ahead();                                                    // the step after the one this call collects
        const int buffer = spec.oldest;
        ck(cudaEventSynchronize(spec_done[buffer]));
        if (h_spec[buffer][opt.max_batch]) {
          const unsigned int code = unsigned(h_spec[buffer][opt.max_batch]);
          unsigned int ignored = 0; tib::read_device_status(stream, &ignored);
          throw GpuFailure("device wait timed out (status " + std::to_string(code) + ")");
        }
        std::memcpy(greedy, h_spec[buffer], size_t(batch) * sizeof(int32_t));
        spec.oldest ^= 1; --spec.inflight;
        count_pass(); count_head(true);
      } else {
        enqueue_segment(ss, packed.data(), 1, nullptr, nullptr, out != nullptr);
        if (out) ck(cudaMemcpy2DAsync(out, size_t(shape.vocab) * 4, logits, size_t(vpitch) * 4, size_t(shape.vocab) * 4, size_t(batch),
                                      cudaMemcpyDeviceToHost, stream));
        finish();
        std::memcpy(greedy, h_log, size_t(batch) * sizeof(int32_t));
      }
      spec.streak = continues ? spec.streak + 1 : 0;
      spec.slots = ss; spec.last_out.assign(greedy, greedy + batch);
      for (int b = 0; b < batch; ++b) lengths[size_t(s[b])] += 1;
      // Keep (or start) a step ahead if the caller has been continuing long enough.
      if (!out && spec.streak >= spec_after && spec.inflight == 0) launch_ahead();
      spec.armed = spec.inflight > 0;
      if (spec.armed) {
        spec.lens_expected.resize(size_t(batch));
        for (int b = 0; b < batch; ++b) spec.lens_expected[size_t(b)] = lengths[size_t(s[b])];
      }
      return;
    } else {
      transform(ss, packed, ll, false);
      tib::LaunchOpts o; o.stream = stream; o.pdl = use_pdl;
      if (out || greedy) {
        count_head(greedy != nullptr);
        gemm(last, head, logits, batch, true, nullptr, false);
        if (out) ck(cudaMemcpy2DAsync(out, size_t(shape.vocab) * 4, logits, size_t(vpitch) * 4, size_t(shape.vocab) * 4, size_t(batch),
                                      cudaMemcpyDeviceToHost, stream));
        if (greedy) {
          ck(tib::argmax(logits, vpitch, batch, shape.vocab, d_next, nullptr, nullptr, d_argmax, o));
          ck(cudaMemcpyAsync(h_next, d_next, size_t(batch) * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
        }
      }
      finish();
      if (greedy) std::memcpy(greedy, h_next, size_t(batch) * sizeof(int32_t));
    }
    for (int b = 0; b < batch; ++b) lengths[size_t(s[b])] += lens[b];
  }
};

namespace {

template <class F>
int guarded(ti_llm_model* model, F&& body) {
  g_error.clear();
  try {
    if (!model) throw InvalidInput("null model");
    DeviceGuard device(model->opt.device);
    model->ensure_usable();
    body();
    return TI_LLM_OK;
  } catch (const InvalidInput& e) { g_error = e.what(); return TI_LLM_INVALID;
  } catch (const tib::IoFailure& e) { g_error = e.what(); return TI_LLM_IO;
  } catch (const GpuFailure& e) { if (model) model->poisoned = true; g_error = e.what(); return TI_LLM_CUDA;
  } catch (const std::exception& e) { if (model) model->poisoned = true; g_error = e.what(); return TI_LLM_INTERNAL;
  } catch (...) { if (model) model->poisoned = true; g_error = "unknown native failure"; return TI_LLM_INTERNAL; }
}

}  // namespace

extern "C" {

int ti_llm_abi_version(void) { return 1; }
const char* ti_llm_last_error(void) { return g_error.c_str(); }

int ti_llm_create(const char* path, const ti_llm_options* o, ti_llm_model** out) {
  g_error.clear();
  if (out) *out = nullptr;
  try {
    if (!path || !o || !out || o->struct_size != sizeof(ti_llm_options) || o->device < 0 || o->max_batch < 1 || o->max_batch > 64 ||
        o->cache_slots < o->max_batch || o->cache_slots > 1024 || o->capacity < 2 || o->capacity > 1024 || o->gemm_config < 0 ||
        o->gemm_config > 11 || o->attention_config < 0 || o->attention_config > 1)
      throw InvalidInput("invalid options/ABI size");
    if (ti_v2_abi_version() != 2) throw InvalidInput("v2 kernel ABI required");
    tib::Artifact art(path);
    if (o->capacity > art.shape.positions) throw InvalidInput("capacity exceeds the model's learned positions");
    DeviceGuard device(o->device);
    std::unique_ptr<ti_llm_model> model(new ti_llm_model);
    model->opt = *o;
    ck(cudaStreamCreateWithFlags(&model->stream, cudaStreamNonBlocking));
    unsigned int cleared = 0;
    ck(tib::read_device_status(model->stream, &cleared));
    ck(tib::device_status_address(&model->d_status_addr));
    model->load(art);
    *out = model.release();
    return TI_LLM_OK;
  } catch (const InvalidInput& e) { g_error = e.what(); return TI_LLM_INVALID;
  } catch (const tib::IoFailure& e) { g_error = e.what(); return TI_LLM_IO;
  } catch (const GpuFailure& e) { g_error = e.what(); return TI_LLM_CUDA;
  } catch (const std::exception& e) { g_error = e.what(); return TI_LLM_INTERNAL;
  } catch (...) { g_error = "unknown create failure"; return TI_LLM_INTERNAL; }
}

// Host-only verification of an artifact (no CUDA call): same checks ti_llm_create performs
// before it touches the GPU.  Declared in include/tinyinfer_b200_ext.h.
int ti_b200_artifact_check(const char* path, int32_t* layers, int32_t* heads, int32_t* hidden, int32_t* int8_weights) {
  g_error.clear();
  try {
    if (!path) throw InvalidInput("null manifest path");
    tib::Artifact art(path);
    if (layers) *layers = art.shape.layers;
    if (heads) *heads = art.shape.heads;
    if (hidden) *hidden = art.shape.hidden;
    if (int8_weights) *int8_weights = art.precision == "int8";
    return TI_LLM_OK;
  } catch (const InvalidInput& e) { g_error = e.what(); return TI_LLM_INVALID;
  } catch (const tib::IoFailure& e) { g_error = e.what(); return TI_LLM_IO;
  } catch (const std::exception& e) { g_error = e.what(); return TI_LLM_INTERNAL; }
}

int ti_llm_destroy(ti_llm_model* model) {
  g_error.clear();
  if (!model) { g_error = "null model"; return TI_LLM_INVALID; }
  delete model;
  return TI_LLM_OK;
}

int ti_llm_reset(ti_llm_model* m, int32_t slot) {
  return guarded(m, [&] {
    if (slot < 0 || slot >= m->opt.cache_slots) throw InvalidInput("invalid public slot");
    m->release(slot);
  });
}
int ti_llm_lengths(ti_llm_model* m, int32_t* out, int32_t count) {
  return guarded(m, [&] {
    if (!out || count != m->opt.cache_slots) throw InvalidInput("wrong lengths output extent");
    std::copy(m->lengths.begin(), m->lengths.begin() + count, out);
  });
}
int ti_llm_get_trace(ti_llm_model* m, ti_llm_trace* out) {
  return guarded(m, [&] { if (!out) throw InvalidInput("null trace output"); *out = m->trace; });
}

int ti_llm_forward_batch(ti_llm_model* m, const int32_t* slots, const int32_t* tokens, const int32_t* lengths, int32_t batch,
                         int32_t stride, float* logits, int32_t* next) {
  return guarded(m, [&] { m->forward(slots, tokens, lengths, batch, stride, logits, next); });
}

int ti_llm_greedy_batch(ti_llm_model* m, const int32_t* slots, const int32_t* prompts, const int32_t* prompt_lengths,
                        const int32_t* requested, int32_t batch, int32_t stride, int32_t* output, int32_t out_stride,
                        int32_t* output_lengths, double* ttft, double* total) {
  return guarded(m, [&] {
    if (!slots || !prompts || !prompt_lengths || !requested || !output || batch < 1 || batch > m->opt.max_batch || stride < 1 ||
        stride > m->opt.capacity || out_stride < 1 || out_stride > m->opt.capacity)
      throw InvalidInput("invalid greedy arguments");
    std::vector<char> used(size_t(m->opt.cache_slots), 0);
    for (int i = 0; i < batch; ++i) {
      const int s = slots[i];
      if (s < 0 || s >= m->opt.cache_slots || used[size_t(s)] || m->lengths[size_t(s)] || prompt_lengths[i] < 1 ||
          prompt_lengths[i] > stride || requested[i] < 1 || requested[i] > out_stride ||
          requested[i] + prompt_lengths[i] > m->opt.capacity)
        throw InvalidInput("greedy needs empty distinct slots and bounded positive lengths");
      used[size_t(s)] = 1;
      for (int t = 0; t < prompt_lengths[i]; ++t) {
        const int32_t id = prompts[size_t(i) * stride + t];
        if (id < 0 || id >= m->shape.vocab) throw InvalidInput("invalid prompt token");
      }
    }
    std::fill(output, output + size_t(batch) * out_stride, -1);
    if (output_lengths) std::fill(output_lengths, output_lengths + batch, 0);
    const auto start = Clock::now();
    std::vector<int32_t> next(static_cast<size_t>(batch), 0), produced(static_cast<size_t>(batch), 1);
    m->forward(slots, prompts, prompt_lengths, batch, stride, nullptr, next.data());
    const double first = elapsed_ms(start);
    for (int i = 0; i < batch; ++i) {
      output[size_t(i) * out_stride] = next[size_t(i)];
      if (ttft) ttft[i] = first;
      if (total && requested[i] == 1) total[i] = first;
    }
    // Decode in device-resident segments: each runs until the next request has all its tokens,
    // with one host round trip per segment instead of one per token.
    std::vector<int32_t> live_slots, live_ids, owner;
    for (;;) {
      live_slots.clear(); live_ids.clear(); owner.clear();
      int steps = m->opt.capacity;
      for (int i = 0; i < batch; ++i)
        if (produced[size_t(i)] < requested[i]) {
          live_slots.push_back(slots[i]); live_ids.push_back(next[size_t(i)]); owner.push_back(i);
          steps = std::min(steps, requested[i] - produced[size_t(i)]);
        }
      if (owner.empty()) break;
      m->enqueue_segment(live_slots, live_ids.data(), steps);
      m->finish();
      const double now = elapsed_ms(start);
      const size_t n = owner.size();
      for (size_t j = 0; j < n; ++j) {
        const int i = owner[j];
        for (int t = 0; t < steps; ++t) output[size_t(i) * out_stride + produced[size_t(i)] + t] = m->h_log[size_t(t) * n + j];
        next[size_t(i)] = m->h_log[size_t(steps - 1) * n + j];
        produced[size_t(i)] += steps;
        m->lengths[size_t(slots[i])] += steps;
        if (total && produced[size_t(i)] == requested[i]) total[i] = now;
      }
    }
    if (output_lengths) for (int i = 0; i < batch; ++i) output_lengths[i] = produced[size_t(i)];
  });
}

// Declared in include/tinyinfer_b200_ext.h: `steps` greedy steps with every intermediate on the GPU.
int ti_b200_llm_decode_steps(ti_llm_model* m, const int32_t* slots, const int32_t* first_tokens, int32_t batch, int32_t steps,
                             int32_t* out_tokens, double* device_ms) {
  return guarded(m, [&] {
    if (!slots || !first_tokens || batch < 1 || batch > m->opt.max_batch || steps < 1) throw InvalidInput("invalid decode-steps arguments");
    std::vector<char> used(size_t(m->opt.cache_slots), 0);
    for (int i = 0; i < batch; ++i) {
      const int s = slots[i];
      if (s < 0 || s >= m->opt.cache_slots || used[size_t(s)] || m->lengths[size_t(s)] < 1 || m->lengths[size_t(s)] + steps > m->opt.capacity ||
          first_tokens[i] < 0 || first_tokens[i] >= m->shape.vocab)
        throw InvalidInput("decode steps need distinct prefilled slots, room for the steps and valid ids");
      used[size_t(s)] = 1;
    }
    cudaEvent_t before = nullptr, after = nullptr;
    ck(cudaEventCreate(&before)); ck(cudaEventCreate(&after));
    try {
      m->enqueue_segment(std::vector<int32_t>(slots, slots + batch), first_tokens, steps, before, after);
      m->finish();
      float ms = 0.f;
      ck(cudaEventElapsedTime(&ms, before, after));
      if (device_ms) *device_ms = double(ms);
    } catch (...) { cudaEventDestroy(before); cudaEventDestroy(after); throw; }
    cudaEventDestroy(before); cudaEventDestroy(after);
    if (out_tokens) std::memcpy(out_tokens, m->h_log, size_t(steps) * batch * sizeof(int32_t));
    for (int i = 0; i < batch; ++i) m->lengths[size_t(slots[i])] += steps;
  });
}

// Declared in include/tinyinfer_b200_ext.h: test hook for the failure paths.
int ti_b200_llm_inject_failure(ti_llm_model* m, int32_t kind, int32_t after_calls) {
  return guarded(m, [&] {
    if (kind == 0 && after_calls >= 0) m->fail_after = after_calls;
    else if (kind == 1) ck(tib::selftest_bounded_wait(m->stream, 1000));
    else throw InvalidInput("inject failure: kind 0 (host, after N valid forward calls) or 1 (device wait that runs out)");
  });
}

// Declared in include/tinyinfer_b200_ext.h: which plan runs a greedy decode step of up to 32 requests.
int ti_b200_llm_decode_plan(ti_llm_model* m, int32_t select, int32_t* active) {
  return guarded(m, [&] {
    if (select < -1 || select > 1) throw InvalidInput("decode plan: -1 (query), 0 (one launch per operation) or 1 (persistent step)");
    if (select == 1 && !m->plan_ready) throw InvalidInput("the persistent decode step does not support this model shape or device");
    if (select >= 0) {
      ck(cudaStreamSynchronize(m->stream));
      m->spec.armed = false; m->spec.inflight = 0; m->spec.streak = 0;
      m->use_persistent = select == 1;
    }
    if (active) *active = m->plan_ready && m->use_persistent ? 1 : 0;
  });
}

#ifdef TIB_STEP_TIMELINE
// Development builds: copies the per-CTA event log of the last persistent step ([256][1024] words) and clears it.
int ti_b200_step_timeline(ti_llm_model* m, unsigned long long* out) {
  return guarded(m, [&] {
    ck(cudaStreamSynchronize(m->stream));
    ck(cudaMemcpy(out, m->plan.timeline, size_t(256) * 1024 * 8, cudaMemcpyDeviceToHost));
    ck(cudaMemset(m->plan.timeline, 0, size_t(256) * 1024 * 8));
  });
}
#endif

int ti_llm_score_window(ti_llm_model* m, const int32_t* tokens, const uint8_t* mask, int32_t length, double* nll, uint64_t* count,
                        double* positions) {
  return guarded(m, [&] {
    if (!tokens || !mask || !nll || !count || length < 2 || length > m->opt.capacity || mask[0]) throw InvalidInput("invalid score window");
    uint64_t targets = 0;
    for (int i = 0; i < length; ++i) {
      if (tokens[i] < 0 || tokens[i] >= m->shape.vocab || mask[i] > 1) throw InvalidInput("invalid score token/mask");
      targets += mask[i];
    }
    if (!targets) throw InvalidInput("no shifted targets selected");
    const int slot = m->opt.cache_slots, rows = length - 1, H = m->shape.hidden;
    m->release(slot);
    m->transform({slot}, std::vector<int32_t>(tokens, tokens + rows), {rows}, true);
    ck(cudaMemcpyAsync(m->d_score_tokens, tokens, size_t(length) * sizeof(int32_t), cudaMemcpyHostToDevice, m->stream));
    ck(cudaMemcpyAsync(m->d_score_mask, mask, size_t(length), cudaMemcpyHostToDevice, m->stream));
    ck(cudaMemsetAsync(m->d_loss, 0, size_t(length) * sizeof(double), m->stream));
    for (int row = 0; row < rows; row += kScoreRows) {
      const int n = std::min(kScoreRows, rows - row);
      m->count_head(false);
      m->gemm(static_cast<const uint16_t*>(m->norm) + size_t(row) * H, m->head, m->logits, n, true, nullptr, false);
      ++m->trace.nll;
      ck(tib::nll_rows(m->logits, m->vpitch, n, m->shape.vocab, m->d_score_tokens, m->d_score_mask, m->d_loss, row + 1, m->stream));
    }
    ck(tib::sum_f64(m->d_loss, m->d_loss_sum, length, m->stream));
    ck(cudaMemcpyAsync(nll, m->d_loss_sum, sizeof(double), cudaMemcpyDeviceToHost, m->stream));
    if (positions) ck(cudaMemcpyAsync(positions, m->d_loss, size_t(length) * sizeof(double), cudaMemcpyDeviceToHost, m->stream));
    m->finish();
    m->release(slot);
    if (!std::isfinite(*nll) || *nll < 0) throw GpuFailure("nonfinite/negative NLL");
    *count = targets;
  });
}

}  // extern "C"
