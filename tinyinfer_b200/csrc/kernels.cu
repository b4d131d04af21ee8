// The single device translation unit of libtinyinfer_backend.so: every sm_100a kernel of the
// INT8-weight decode path plus the host functions that configure and enqueue them
// (declared in launch.hpp).
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "launch.hpp"

namespace tib { __device__ unsigned int g_device_status = 0; }
#define TIB_STATUS_DEFINED
#include "attention.cuh"
#include "attention_tc.cuh"
#include "common.cuh"
#include "decode_step.cuh"
#include "elementwise.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "gemm_wide.cuh"
#include "model_glue.cuh"

namespace tib {
namespace {

// ---------------------------------------------------------------- generic launch helper
template <typename... KArgs, typename... Args>
cudaError_t launch_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, const LaunchOpts& o,
                             dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = o.stream;
  cudaLaunchAttribute attrs[2]; unsigned n = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster.x; attrs[n].val.clusterDim.y = cluster.y; attrs[n].val.clusterDim.z = cluster.z; ++n;
  }
  if (o.pdl) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1; ++n;
  }
  cfg.attrs = attrs; cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, const LaunchOpts& o,
                   int cluster_y, Args&&... args) {
  return launch_clustered(kernel, grid, block, smem, o, dim3(1, unsigned(std::max(cluster_y, 1)), 1), std::forward<Args>(args)...);
}

// ---------------------------------------------------------------- tensor maps
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr; cudaDriverEntryPointQueryResult q{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D map over a row-major [rows, cols] matrix with `pitch` elements per row; box = (box_cols, box_rows).
bool make_map_2d(CUtensorMap* map, const void* base, bool int8, uint64_t rows, uint64_t cols, uint64_t pitch,
                 uint32_t box_cols, uint32_t box_rows, bool swizzle128 = false) {
  const uint64_t esize = int8 ? 1 : 2;
  if (!encode_tiled() || reinterpret_cast<uintptr_t>(base) % 16 || (pitch * esize) % 16 || pitch * esize >= (1ull << 40) ||
      rows == 0 || cols == 0 || rows > 0xffffffffull || cols > 0xffffffffull)
    return false;
  const cuuint64_t dims[2] = {cols, rows}, strides[1] = {pitch * esize};
  const cuuint32_t box[2] = {box_cols, box_rows}, estr[2] = {1, 1};
  return encode_tiled()(map, int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Opt-in to more than 48 KB of dynamic shared memory.  The attribute belongs to (kernel, device), and one
// process may drive several GPUs (one model context per device), so it is set once per device, not once
// per process.
template <typename K>
cudaError_t allow_smem(K kernel, int bytes) {
  static std::mutex lock;
  static std::map<const void*, uint64_t> done;                 // kernel -> bit per device already configured
  int device = -1;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return st;
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> hold(lock);
  uint64_t& mask = done[reinterpret_cast<const void*>(kernel)];
  if (mask >> device & 1) return cudaSuccess;
  st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (st == cudaSuccess) mask |= uint64_t(1) << device;
  return st;
}

int sm_count() {
  static int n = [] { int dev = 0, v = 148; if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev); return v; }();
  return n;
}

template <typename WT, int MT, bool TMA>
cudaError_t launch_gemv(const CUtensorMap& map, const GemvArgs& args, dim3 grid, const LaunchOpts& o) {
  const cudaError_t ready = allow_smem(gemv_kernel<WT, MT, TMA>, GemvSmem::kBytes);
  if (ready != cudaSuccess) return ready;
  return launch(gemv_kernel<WT, MT, TMA>, grid, dim3(kGemvThreads), GemvSmem::kBytes, o, int(grid.y), map, args);
}
template <typename WT, bool TMA>
cudaError_t launch_gemv_mt(int mt, const CUtensorMap& map, const GemvArgs& args, dim3 grid, const LaunchOpts& o) {
  switch (mt) {
    case 1: return launch_gemv<WT, 1, TMA>(map, args, grid, o);
    case 2: return launch_gemv<WT, 2, TMA>(map, args, grid, o);
    default: return launch_gemv<WT, 4, TMA>(map, args, grid, o);
  }
}

template <int NMMA, int LN = 0, bool LEAN = false, bool DIRECT = false, typename WT = int8_t>
cudaError_t launch_tc(const CUtensorMap& map, const GemvArgs& args, dim3 grid, const LaunchOpts& o) {
  constexpr int kBytes = TcSmem<NMMA, LEAN, int(sizeof(WT))>::kBytes;
  const cudaError_t ready = allow_smem(gemm_tc_kernel<NMMA, LN, LEAN, DIRECT, WT>, kBytes);
  if (ready != cudaSuccess) return ready;
  return launch(gemm_tc_kernel<NMMA, LN, LEAN, DIRECT, WT>, grid, dim3(kTcThreads), kBytes, o, int(grid.y), map, args);
}

// Measurement aids of development builds (-DTIB_DEV_KNOBS): an environment variable may override a dispatch
// threshold.  Release builds ignore the environment here.
int env_int(const char* name, int fallback) {
#ifdef TIB_DEV_KNOBS
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
#else
  (void)name;
  return fallback;
#endif
}

// K split of the tensor-core GEMM, chosen from the matrix alone (never from M): the summation grouping of an
// output element is then the same for every batch size and batch composition.  Few stages per CTA matter more
// than full tiles: a stage costs about a microsecond of serial latency.
int tc_splits(int n, int k) {
  const int slabs = (n + 127) / 128;
  int splits = 1;
  while (splits < 8 && slabs * splits < sm_count() && (k + splits * 2 - 1) / (splits * 2) >= kTcStageK) splits *= 2;
  static const int forced_splits = env_int("TINYINFER_B200_TC_SPLITS", 0);
  if (forced_splits > 0) splits = forced_splits;
  return splits;
}
constexpr int kWideMinRows = 129;       // fewer rows: 32 / 64-row tiles of the decode-shaped kernel with its LayerNorm prologue (measured from 129 rows up: 63 decode rows + a prompt of n rows, and single prompts, are faster on the many-row kernel)
int tc_chunk(int k, int splits) {
  const int chunk = (k + splits - 1) / splits;
  return (chunk + kTcStageK - 1) / kTcStageK * kTcStageK;
}

}  // namespace

// ---------------------------------------------------------------- GEMM
cudaError_t gemm(const GemmCall& c, const LaunchOpts& o) {
  GemvArgs a{};
  a.a = static_cast<const __half*>(c.a); a.w = c.w; a.scales = c.scales; a.bias = static_cast<const __half*>(c.bias);
  a.out = c.out; a.residual = static_cast<const __half*>(c.residual);
  a.lda = c.lda; a.ldo = c.ldo; a.ldw = c.ldw; a.m = c.m; a.n = c.n; a.k = c.k;
  a.out_fp32 = c.out_fp32; a.gelu = c.gelu; a.early_trigger = o.early_trigger && o.pdl ? 1 : 0;
  a.argmax_best = static_cast<unsigned long long*>(c.argmax_best); a.skip_store = c.skip_store ? 1 : 0;
  if (c.kv) {
    a.k_pool = static_cast<__half*>(c.kv->k_pool); a.v_pool = static_cast<__half*>(c.kv->v_pool);
    a.kv_table = c.kv->table; a.kv_slots = c.kv->slots; a.kv_row_req = c.kv_row_req; a.kv_row_pos = c.kv_row_pos;
    a.kv_table_pitch = c.kv->table_pitch; a.kv_layers = c.kv->layers; a.kv_layer = c.kv->layer; a.kv_heads = c.kv->heads;
    a.kv_hidden = c.kv->heads * c.kv->head_dim;
  }
  // Many rows (prefill) of a matrix that has an operand image: the tile kernel built for that regime (gemm_wide.cuh), with
  // the K ranges of the split below, so a row's result is the one the decode-shaped kernel gives.
  static const int wide_min_rows = env_int("TINYINFER_B200_WIDE_MIN_ROWS", kWideMinRows);    // measurement aid
  if (c.w_image && c.m >= wide_min_rows && !c.out_fp32 && !c.ln_gamma && c.k % 8 == 0 && c.lda % 8 == 0 && reinterpret_cast<uintptr_t>(c.a) % 16 == 0) {
    CUtensorMap rows; std::memset(&rows, 0, sizeof rows);
    if (make_map_2d(&rows, c.a, false, uint64_t(c.m), uint64_t(c.k), uint64_t(c.lda), 64, uint32_t(kWideRows), true)) {
      GemvArgs w = a;
      w.w = c.w_image;
      w.k_chunk = tc_chunk(c.k, tc_splits(c.n, c.k));
      const int tiles = ((c.n + 127) / 128) * ((c.m + kWideRows - 1) / kWideRows);
      const cudaError_t ready = allow_smem(gemm_wide_kernel, WideSmem::kBytes);
      if (ready != cudaSuccess) return ready;
      return launch(gemm_wide_kernel, dim3(unsigned(std::min(tiles, sm_count()))), dim3(kWideThreads), WideSmem::kBytes, o, 1, rows, w);
    }
  }
  // Tensor-core path: int8 weights, 5 or more rows of A, operands addressable by TMA / 16-byte loads.
  static const int tc_min_rows = env_int("TINYINFER_B200_TC_MIN_ROWS", 5);      // measurement aid: where the SIMT kernel hands over
  // With `uniform_numerics` every row count takes this path, so a row's result does not depend on
  // how many other rows share the call (the K split below depends on N and K only).
  if (c.w_int8 && (c.uniform_numerics || c.m >= tc_min_rows) && c.k % 8 == 0 && c.lda % 8 == 0 && reinterpret_cast<uintptr_t>(c.a) % 16 == 0) {
    CUtensorMap map; std::memset(&map, 0, sizeof map);
    const uint64_t slab_count = uint64_t(c.n + 127) / 128;
    if (c.w_slab_rows && (c.w_slab_rows < c.k || c.w_slab_rows % kTcStageK)) return cudaErrorInvalidValue;
    a.w_slab_rows = c.w_slab_rows;
    const bool mapped = c.w_slab_rows ? make_map_2d(&map, c.w, true, slab_count * uint64_t(c.w_slab_rows), 128, 128, 128, uint32_t(kTcStageK), true)
                                      : make_map_2d(&map, c.w, true, uint64_t(c.k), uint64_t(c.n), uint64_t(c.ldw), 128, uint32_t(kTcStageK), true);
    // No tensor map (row pitch or base not 16-byte aligned, e.g. N = 50257): the same kernel with a producer warp that
    // copies the weight tiles itself.
    // (measured on 768x50257: faster than the SIMT kernel from about 16 rows on)
    const bool direct = !mapped && !c.w_slab_rows && !c.ln_gamma && c.m >= 16;
    if (mapped || direct) {
      const int slabs = (c.n + 127) / 128;
      const int splits = tc_splits(c.n, c.k);
      // 33..1024 rows of a K-split matrix: tiles of 64 rows in the decode kernel's form (push reduction, LayerNorm
      // prologue, two CTAs per SM): a 64-request step still runs every GEMM as one wave of clusters, and a single prompt's
      // prefill (measured at 150..900 rows) is faster than with 256-row tiles reduced by remote reads.
      static const int tile64_rows = env_int("TINYINFER_B200_TC_TILE64_ROWS", 1024);   // measurement aid
      const int nmma = c.m <= 32 ? 32 : (c.m <= 64 || (splits > 1 && c.m <= tile64_rows)) ? 64 : c.m <= 128 ? 128 : 256;
      if (c.ln_gamma) {
        if (nmma > 64 || (nmma == 64 && splits == 1) || c.k > 1024 || c.lda != c.k) return cudaErrorNotSupported;
        // rows wider than 768: shared mode only, and the strips of the rows one CTA prepares must fit the B-operand ring
        if (c.k > 768 && (splits == 1 || size_t(nmma / splits) * c.k * 2 > size_t(nmma == 64 ? 2 : kTcOpStages) * nmma * kTcStageK * 2))
          return cudaErrorNotSupported;
        a.ln_gamma = static_cast<const __half*>(c.ln_gamma); a.ln_beta = static_cast<const __half*>(c.ln_beta); a.ln_eps = c.ln_eps;
      }
      const int m_tiles = (c.m + nmma - 1) / nmma;
      a.k_chunk = tc_chunk(c.k, splits);
      // Many rows (prefill): a cluster reduction of 64..256-row partial tiles would cost more than the MMAs.  One CTA
      // then walks the whole K with one TMEM accumulator per K range and adds them in range order -- the very sums
      // of the split launch, so a row's result still does not depend on how many rows share the call.
      const int wide = std::min(256, 512 / splits);
      static const int serial_ok = env_int("TINYINFER_B200_TC_SERIAL", 1);       // measurement aid
      if (serial_ok && splits > 1 && c.m > 32 && !c.ln_gamma && slabs * ((c.m + wide - 1) / wide) >= sm_count()) {
        a.serial_chunks = splits;
        const dim3 grid(slabs, 1, (c.m + wide - 1) / wide);
        switch (wide) {
          case 64: return direct ? launch_tc<64, 0, false, true>(map, a, grid, o) : launch_tc<64>(map, a, grid, o);
          case 128: return direct ? launch_tc<128, 0, false, true>(map, a, grid, o) : launch_tc<128>(map, a, grid, o);
          default: return direct ? launch_tc<256, 0, false, true>(map, a, grid, o) : launch_tc<256>(map, a, grid, o);
        }
      }
      const dim3 grid(slabs, splits, m_tiles);
      static const int lean_ok = env_int("TINYINFER_B200_TC_LEAN", 1);           // measurement aid
      if (direct) {
        switch (nmma) {
          case 32: return launch_tc<32, 0, false, true>(map, a, grid, o);
          case 64: return launch_tc<64, 0, false, true>(map, a, grid, o);
          case 128: return launch_tc<128, 0, false, true>(map, a, grid, o);
          default: return launch_tc<256, 0, false, true>(map, a, grid, o);
        }
      }
      switch (nmma) {
        case 32:
          // no K split, many slabs (vocabulary projection): the lean layout runs three CTAs per SM
          if (!c.ln_gamma && splits == 1 && lean_ok && slabs > 2 * sm_count()) return launch_tc<32, 0, true>(map, a, grid, o);
          if (!c.ln_gamma) return launch_tc<32>(map, a, grid, o);
          // up to 8 rows every CTA prepares them itself; more are shared out over the K-split cluster
          if (c.k > 768) return launch_tc<32, 3>(map, a, grid, o);
          return splits > 1 && c.m > 8 ? launch_tc<32, 2>(map, a, grid, o) : launch_tc<32, 1>(map, a, grid, o);
        case 64: return !c.ln_gamma ? launch_tc<64>(map, a, grid, o) : c.k > 768 ? launch_tc<64, 3>(map, a, grid, o) : launch_tc<64, 2>(map, a, grid, o);
        case 128: return launch_tc<128>(map, a, grid, o);
        default: return launch_tc<256>(map, a, grid, o);
      }
    }
  }
  // fp16 weights on the same tensor-core kernel: the tiles are rearranged instead of dequantised.  Same K split and the
  // same tile forms as the int8 path, so a matrix gives the same bits whether it arrives as int8 + scales or as the fp16
  // values those dequantise to.
  if (!c.w_int8 && !c.ln_gamma && !c.w_slab_rows && (c.uniform_numerics || c.m >= tc_min_rows) && c.k % 8 == 0 && c.lda % 8 == 0 &&
      reinterpret_cast<uintptr_t>(c.a) % 16 == 0) {
    CUtensorMap map; std::memset(&map, 0, sizeof map);
    if (make_map_2d(&map, c.w, false, uint64_t(c.k), uint64_t(c.n), uint64_t(c.ldw), 64, uint32_t(kTcStageK), true)) {
      const int slabs = (c.n + 127) / 128, splits = tc_splits(c.n, c.k);
      a.k_chunk = tc_chunk(c.k, splits);
      const int wide = std::min(256, 512 / splits);
      if (splits > 1 && c.m > 32 && slabs * ((c.m + wide - 1) / wide) >= sm_count()) {
        a.serial_chunks = splits;
        const dim3 grid(slabs, 1, (c.m + wide - 1) / wide);
        switch (wide) {
          case 64: return launch_tc<64, 0, false, false, __half>(map, a, grid, o);
          case 128: return launch_tc<128, 0, false, false, __half>(map, a, grid, o);
          default: return launch_tc<256, 0, false, false, __half>(map, a, grid, o);
        }
      }
      const int nmma = c.m <= 32 ? 32 : (c.m <= 64 || (splits > 1 && c.m <= 1024)) ? 64 : c.m <= 128 ? 128 : 256;
      const dim3 grid(slabs, splits, (c.m + nmma - 1) / nmma);
      switch (nmma) {
        case 32: return splits == 1 && slabs > 2 * sm_count() ? launch_tc<32, 0, true, false, __half>(map, a, grid, o)
                                                              : launch_tc<32, 0, false, false, __half>(map, a, grid, o);
        case 64: return launch_tc<64, 0, false, false, __half>(map, a, grid, o);
        case 128: return launch_tc<128, 0, false, false, __half>(map, a, grid, o);
        default: return launch_tc<256, 0, false, false, __half>(map, a, grid, o);
      }
    }
  }
  if (c.ln_gamma || c.w_slab_rows) return cudaErrorNotSupported;   // only the tensor-core kernel has the LayerNorm prologue / reads tiles
  // Row tiles run along grid.z (at most 65535): more rows than that go out as several launches over row blocks.
  constexpr int kSimtRowsPerLaunch = 4 * 65535;
  if (c.m > kSimtRowsPerLaunch) {
    for (int row0 = 0; row0 < c.m; row0 += kSimtRowsPerLaunch) {
      GemmCall part = c;
      part.m = std::min(kSimtRowsPerLaunch, c.m - row0);
      part.a = static_cast<const __half*>(c.a) + size_t(row0) * c.lda;
      part.out = c.out_fp32 ? static_cast<void*>(static_cast<float*>(c.out) + size_t(row0) * c.ldo) : static_cast<void*>(static_cast<__half*>(c.out) + size_t(row0) * c.ldo);
      if (c.residual) part.residual = static_cast<const __half*>(c.residual) + size_t(row0) * c.ldo;
      const cudaError_t st = gemm(part, o);
      if (st != cudaSuccess) return st;
    }
    return cudaSuccess;
  }
  const int bn = c.w_int8 ? 128 : 64;
  const int mt = c.m >= 3 ? 4 : c.m;
  const int slabs = (c.n + bn - 1) / bn, m_tiles = (c.m + mt - 1) / mt;
  // Split K over a cluster until the grid covers the SMs (or a CTA would own less than one stage).
  int splits = 1;
  while (splits < 8 && slabs * m_tiles * splits < sm_count() && (c.k + splits * 2 - 1) / (splits * 2) >= kGemvStageRows) splits *= 2;
  int chunk = (c.k + splits - 1) / splits;
  chunk = (chunk + kGemvStageRows - 1) / kGemvStageRows * kGemvStageRows;
  a.k_chunk = chunk;
  CUtensorMap map; std::memset(&map, 0, sizeof map);
  const bool tma = make_map_2d(&map, c.w, c.w_int8, uint64_t(c.k), uint64_t(c.n), uint64_t(c.ldw),
                               uint32_t(bn), uint32_t(kGemvStageRows));
  const dim3 grid(slabs, splits, m_tiles);
  if (c.w_int8) return tma ? launch_gemv_mt<int8_t, true>(mt, map, a, grid, o) : launch_gemv_mt<int8_t, false>(mt, map, a, grid, o);
  return tma ? launch_gemv_mt<__half, true>(mt, map, a, grid, o) : launch_gemv_mt<__half, false>(mt, map, a, grid, o);
}

cudaError_t retile_i8(const int8_t* src, long long ld, int k, int n, int8_t* dst, int slab_rows, cudaStream_t stream) {
  if (!src || !dst || k < 1 || n < 1 || slab_rows < k) return cudaErrorInvalidValue;
  const long long chunks = (long long)((n + 127) / 128) * slab_rows * 8;
  retile_i8_kernel<<<unsigned((chunks + 255) / 256), 256, 0, stream>>>(src, ld, k, n, dst, slab_rows, chunks);
  return cudaGetLastError();
}

size_t wide_image_bytes(int k, int n) { return size_t((n + 127) / 128) * size_t((k + kTcStageK - 1) / kTcStageK) * kWideImageStage; }

cudaError_t wide_image(const int8_t* q, const void* w16, long long ld, const float* scales, void* image, int k, int n, cudaStream_t stream) {
  if ((!q && !w16) || (q && !scales) || !image || k < 1 || n < 1) return cudaErrorInvalidValue;
  const int stages = (k + kTcStageK - 1) / kTcStageK;
  const long long chunks = (long long)(wide_image_bytes(k, n) / 16);
  wide_image_kernel<<<unsigned((chunks + 255) / 256), 256, 0, stream>>>(q, static_cast<const __half*>(w16), ld, scales, static_cast<uint8_t*>(image), k, n, stages, chunks);
  return cudaGetLastError();
}

cudaError_t quantize_i8(const void* w, long long rows, int cols, int8_t* q, float* scales, int* flag, cudaStream_t stream) {
  if (!w || !q || !scales || !flag || rows < 1 || cols < 1) return cudaErrorInvalidValue;
  cudaError_t st = cudaMemsetAsync(scales, 0, size_t(cols) * sizeof(float), stream);
  if (st == cudaSuccess) st = cudaMemsetAsync(flag, 0, sizeof(int), stream);
  if (st != cudaSuccess) return st;
  const int col_blocks = (cols + 127) / 128;
  // enough row groups to fill the device without more atomics than needed
  const int groups = int(std::max<long long>(1, std::min<long long>(rows, (4LL * sm_count() + col_blocks - 1) / col_blocks)));
  const int rows_per_block = int((rows + groups - 1) / groups);
  const auto* half = static_cast<const __half*>(w);
  auto* bits = reinterpret_cast<unsigned int*>(scales);
  quant_absmax_kernel<<<dim3(col_blocks, unsigned((rows + rows_per_block - 1) / rows_per_block)), 128, 0, stream>>>(half, rows, cols, bits, flag, rows_per_block);
  quant_scales_kernel<<<col_blocks, 128, 0, stream>>>(bits, scales, cols);
  const long long elements = rows * cols;
  quant_apply_kernel<<<unsigned((elements + 255) / 256), 256, 0, stream>>>(half, scales, q, elements, cols);
  return cudaGetLastError();
}

cudaError_t sgemm(const float* a, const float* b, float* c, int m, int n, int k, cudaStream_t stream) {
  // 16-row tiles along grid.y (at most 65535 of them per launch): row blocks beyond that take further launches
  constexpr int kRowsPerLaunch = 16 * 65535;
  for (int row0 = 0; row0 < m; row0 += kRowsPerLaunch) {
    const int rows = std::min(kRowsPerLaunch, m - row0);
    sgemm_kernel<<<dim3((n + 15) / 16, (rows + 15) / 16), 256, 0, stream>>>(a + size_t(row0) * k, b, c + size_t(row0) * n, rows, n, k);
    const cudaError_t st = cudaGetLastError();
    if (st != cudaSuccess) return st;
  }
  return cudaSuccess;
}

// ---------------------------------------------------------------- attention
cudaError_t attention_packed(const void* q, const void* k, const void* v, void* y, const int32_t* ql, const int32_t* kl,
                             const int32_t* off, int batch, int heads, int q_len, int kv_len, int d, bool causal,
                             const LaunchOpts& o) {
  AttnArgs p{};
  p.q = static_cast<const __half*>(q); p.out = static_cast<__half*>(y);
  p.q_sb = (long long)heads * q_len * d; p.q_sh = (long long)q_len * d; p.q_si = d;
  p.o_sb = p.q_sb; p.o_sh = p.q_sh; p.o_si = d;
  p.row_start = nullptr;
  p.q_lengths = ql; p.kv_lengths = kl; p.offsets = off;
  p.batch = batch; p.heads = heads; p.q_len = q_len; p.kv_len = kv_len; p.causal = causal;
  KvPacked kv{static_cast<const __half*>(k), static_cast<const __half*>(v), heads, kv_len, d};
  const bool vec = (reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) % 16 == 0;
  // Many query rows of 64-wide heads: both contractions on the tensor cores.
  if (d == 64 && q_len >= kAttnTcMinRows && vec) {
    const cudaError_t ready = allow_smem(attn_tc_kernel<KvPacked>, AttnTcSmem::kBytes);
    if (ready != cudaSuccess) return ready;
    const dim3 tc_grid((q_len + kAttnTcRows - 1) / kAttnTcRows, heads, batch);
    return launch(attn_tc_kernel<KvPacked>, tc_grid, dim3(kAttnTcThreads), AttnTcSmem::kBytes, o, 1, p, kv, 0);
  }
  const dim3 grid((q_len + kAttnTileQ - 1) / kAttnTileQ, heads, batch);
  if (d == 64) return vec ? launch(attn_tile_kernel<64, KvPacked, true>, grid, dim3(256), 0, o, 1, p, kv)
                          : launch(attn_tile_kernel<64, KvPacked, false>, grid, dim3(256), 0, o, 1, p, kv);
  if (d == 128) return vec ? launch(attn_tile_kernel<128, KvPacked, true>, grid, dim3(256), 0, o, 1, p, kv)
                           : launch(attn_tile_kernel<128, KvPacked, false>, grid, dim3(256), 0, o, 1, p, kv);
  return cudaErrorInvalidValue;
}

static KvPaged paged(const PagedKv& kv) {
  return KvPaged{static_cast<const __half*>(kv.k_pool), static_cast<const __half*>(kv.v_pool), kv.table, kv.slots,
                 kv.table_pitch, kv.layers, kv.layer, kv.heads, kv.head_dim};
}

cudaError_t attention_paged(const void* qkv, void* out, const int32_t* row_start, const int32_t* ql, const int32_t* kl,
                            const int32_t* off, int batch, int max_q, int max_kv, const PagedKv& kv, const LaunchOpts& o, bool skip_single,
                            int long_requests, int short_requests) {
  if (kv.head_dim != 64) return cudaErrorInvalidValue;
  const int hidden = kv.heads * kv.head_dim;
  AttnArgs p{};
  p.q = static_cast<const __half*>(qkv); p.out = static_cast<__half*>(out);
  p.q_sb = 0; p.q_sh = kv.head_dim; p.q_si = 3LL * hidden;
  p.o_sb = 0; p.o_sh = kv.head_dim; p.o_si = hidden;
  p.row_start = row_start;
  p.q_lengths = ql; p.kv_lengths = kl; p.offsets = off;
  p.batch = batch; p.heads = kv.heads; p.q_len = max_q; p.kv_len = max_kv; p.causal = 1; p.skip_single = skip_single ? 1 : 0;
  // Requests with at least kAttnTcMinRows rows in this pass take the tensor-core kernel, the others the SIMT tile kernel;
  // the choice depends on the request's own row count only, never on what shares its pass.
  if (long_requests > 0) {
    const cudaError_t ready = allow_smem(attn_tc_kernel<KvPaged>, AttnTcSmem::kBytes);
    if (ready != cudaSuccess) return ready;
    const dim3 tc_grid((max_q + kAttnTcRows - 1) / kAttnTcRows, kv.heads, batch);
    const cudaError_t st = launch(attn_tc_kernel<KvPaged>, tc_grid, dim3(kAttnTcThreads), AttnTcSmem::kBytes, o, 1, p, paged(kv), kAttnTcMinRows);
    if (st != cudaSuccess || short_requests == 0) return st;
    p.skip_min_q = kAttnTcMinRows;
  }
  int short_q = max_q;
  if (long_requests > 0) short_q = std::min(max_q, kAttnTcMinRows - 1);      // the SIMT grid only has to cover the short requests
  p.q_len = max_q;
  const dim3 grid((short_q + kAttnTileQ - 1) / kAttnTileQ, kv.heads, batch);
  return launch(attn_tile_kernel<64, KvPaged, true>, grid, dim3(256), 0, o, 1, p, paged(kv));
}

int decode_chunks(int max_kv, int chunk) { return std::max(1, (max_kv + chunk - 1) / chunk); }

cudaError_t attention_paged_decode(const void* qkv, void* out, const int32_t* kl, int batch, int max_kv, int chunk,
                                   float* scratch_acc, float* scratch_ml, int* counters, const PagedKv& kv, const LaunchOpts& o,
                                   bool early, bool whole_history, bool early_trigger, const int32_t* row_start, const int32_t* q_lengths) {
  if (kv.head_dim != 64) return cudaErrorInvalidValue;
  const int hidden = kv.heads * kv.head_dim;
  DecodeArgs p{};
  p.q = static_cast<const __half*>(qkv); p.q_sb = 3LL * hidden; p.q_sh = kv.head_dim;
  p.out = static_cast<__half*>(out); p.o_sb = hidden; p.o_sh = kv.head_dim;
  p.kv_lengths = kl; p.part_acc = scratch_acc; p.part_ml = scratch_ml; p.counters = counters;
  p.batch = batch; p.heads = kv.heads; p.early = early && !q_lengths ? 1 : 0; p.early_trigger = early_trigger ? 1 : 0;
  p.kv_len = kv.table_pitch * kPageTokens;              // positions a slot's page table can name
  p.row_start = row_start; p.q_lengths = q_lengths;
  if ((row_start || q_lengths) && !whole_history) return cudaErrorNotSupported;
  if (whole_history) {
    // One CTA of 8 warps walks the whole history of a (request, head) and merges in shared memory: no partials in
    // global memory, no second stage, and a grid small enough to be resident at once.
    p.chunk = 1 << 30; p.chunks = 1;
    const cudaError_t ready = allow_smem(attn_decode_staged_kernel<64, KvPaged>, staged_smem_bytes<64>());
    if (ready != cudaSuccess) return ready;
    return launch(attn_decode_staged_kernel<64, KvPaged>, dim3(kv.heads, batch), dim3(kStagedWarps * 32), staged_smem_bytes<64>(), o, 1, p, paged(kv));
  }
  p.chunk = chunk; p.chunks = decode_chunks(max_kv, chunk);
  cudaError_t st = launch(attn_decode_kernel<64, KvPaged>, dim3(p.chunks, kv.heads, batch), dim3(kDecodeWarps * 32), 0, o, 1, p, paged(kv));
  if (st != cudaSuccess || p.chunks == 1 || counters) return st;
  return launch(attn_combine_kernel<64>, dim3(kv.heads, batch), dim3(64), 0, o, 1, p);
}

cudaError_t attention_packed_decode(const void* q, const void* k, const void* v, void* y, const int32_t* kl, int batch,
                                    int heads, int kv_len, int chunk, float* scratch_acc, float* scratch_ml,
                                    const LaunchOpts& o) {
  DecodeArgs p{};
  p.q = static_cast<const __half*>(q); p.q_sb = 64LL * heads; p.q_sh = 64;
  p.out = static_cast<__half*>(y); p.o_sb = 64LL * heads; p.o_sh = 64;
  p.kv_lengths = kl; p.part_acc = scratch_acc; p.part_ml = scratch_ml;
  p.batch = batch; p.heads = heads; p.chunk = chunk; p.chunks = decode_chunks(kv_len, chunk); p.kv_len = kv_len;
  KvPacked kv{static_cast<const __half*>(k), static_cast<const __half*>(v), heads, kv_len, 64};
  // A chunk that spans the whole history: one CTA of 8 warps per (request, head), merged in shared memory.
  if (p.chunks == 1 && kv_len > kDecodeWarps * 32) {
    const cudaError_t ready = allow_smem(attn_decode_staged_kernel<64, KvPacked>, staged_smem_bytes<64>());
    if (ready != cudaSuccess) return ready;
    return launch(attn_decode_staged_kernel<64, KvPacked>, dim3(heads, batch), dim3(kStagedWarps * 32), staged_smem_bytes<64>(), o, 1, p, kv);
  }
  cudaError_t st = launch(attn_decode_kernel<64, KvPacked>, dim3(p.chunks, heads, batch), dim3(kDecodeWarps * 32), 0, o, 1, p, kv);
  if (st != cudaSuccess || p.chunks == 1) return st;
  return launch(attn_combine_kernel<64>, dim3(heads, batch), dim3(64), 0, o, 1, p);
}

// ---------------------------------------------------------------- elementwise / glue
cudaError_t layernorm(const void* x, const int32_t* row_index, const void* g, const void* b, void* y, int rows, int cols,
                      float eps, const LaunchOpts& o) {
  const size_t smem = cols <= kLnMaxCols ? size_t(20) * cols : 0;
  if (smem > 48 * 1024) {
    const cudaError_t ready = allow_smem(layernorm_kernel, 20 * kLnMaxCols);
    if (ready != cudaSuccess) return ready;
  }
  return launch(layernorm_kernel, dim3((rows + 3) / 4), dim3(128), smem, o, 1, static_cast<const __half*>(x), row_index,
                static_cast<const __half*>(g), static_cast<const __half*>(b), static_cast<__half*>(y), rows, cols, eps, o.pdl && o.early_trigger ? 1 : 0);
}
cudaError_t gelu(const void* x, void* y, long long count, cudaStream_t stream) {
  const int vec = (reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) ? 1 : 0;
  const long long work = vec ? (count + 7) / 8 : count;
  const int blocks = int(std::min<long long>((work + 255) / 256, 148LL * 16));
  gelu_kernel<<<std::max(blocks, 1), 256, 0, stream>>>(static_cast<const __half*>(x), static_cast<__half*>(y), count, vec);
  return cudaGetLastError();
}
cudaError_t softmax(const void* x, void* y, int rows, int cols, cudaStream_t stream) {
  softmax_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(static_cast<const __half*>(x), static_cast<__half*>(y), rows, cols);
  return cudaGetLastError();
}
cudaError_t embed(const int32_t* ids, const int32_t* row_pos, const void* wte, const void* wpe, void* x, int rows,
                  int hidden, int vocab, const LaunchOpts& o) {
  const long long work = (long long)rows * (hidden / 8);
  const int blocks = int(std::min<long long>((work + 255) / 256, 148LL * 8));
  return launch(embed_kernel, dim3(std::max(blocks, 1)), dim3(256), 0, o, 1, ids, row_pos, static_cast<const __half*>(wte),
                static_cast<const __half*>(wpe), static_cast<__half*>(x), rows, hidden, vocab);
}
cudaError_t argmax(const float* logits, long long pitch, int rows, int cols, int32_t* out, int32_t* feedback,
                   const int32_t* step, void* scratch, const LaunchOpts& o) {
  // Enough CTAs to pull a row set of any size at memory speed: about two per SM in total.
  int segments = 1;
  if (scratch) segments = std::max(1, std::min({32, (2 * sm_count() + rows - 1) / rows, cols / 1024}));
  auto* best = static_cast<unsigned long long*>(scratch);
  auto* tickets = reinterpret_cast<unsigned int*>(best + rows);
  return launch(argmax_kernel, dim3(rows, segments), dim3(256), 0, o, 1, logits, pitch, cols, out, feedback, step, best, tickets);
}
cudaError_t argmax_finish(void* best, int rows, int cols, int32_t* out, int32_t* feedback, int32_t* step, int32_t* row_pos,
                          int32_t* kv_lengths, const LaunchOpts& o) {
  if (rows < 1 || rows > 64) return cudaErrorInvalidValue;
  return launch(argmax_finish_kernel, dim3(1), dim3(64), 0, o, 1, static_cast<unsigned long long*>(best), rows, cols, out, feedback, step, row_pos, kv_lengths);
}
cudaError_t advance(int32_t* row_pos, int32_t* kv_lengths, int32_t* step, int batch, const LaunchOpts& o) {
  return launch(advance_kernel, dim3((batch + 63) / 64), dim3(64), 0, o, 1, row_pos, kv_lengths, step, batch);
}

cudaError_t nll_rows(const float* logits, long long pitch, int rows, int cols, const int32_t* tokens, const uint8_t* mask,
                     double* loss, int first_position, cudaStream_t stream) {
  nll_kernel<<<rows, 256, 0, stream>>>(logits, pitch, cols, tokens, mask, loss, first_position);
  return cudaGetLastError();
}
cudaError_t sum_f64(const double* values, double* out, int length, cudaStream_t stream) {
  sum_f64_kernel<<<1, 256, 0, stream>>>(values, out, length);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- persistent decode step
int step_k_chunk(int n, int k) { return tc_chunk(k, tc_splits(n, k)); }

const char* step_unsupported(const StepPlan& p) {
  if (p.hidden < 128 || p.hidden % 128 || p.hidden > kStepMaxHidden) return "hidden size must be a multiple of 128 up to 1024";
  if (p.heads * 64 != p.hidden) return "heads of 64 values";
  if (p.ff % 128 || p.layers < 1 || p.layers > 60) return "layer shape";
  const int chunks[4] = {p.chunk_qkv, p.chunk_proj, p.chunk_fc, p.chunk_head};
  for (int c : chunks)
    if (c < kTcStageK || c % kTcStageK || p.hidden % c || p.hidden / c > kStepMaxRanges) return "K split of a hidden-wide GEMM";
  if (p.chunk_proj2 < kTcStageK || p.chunk_proj2 % kTcStageK || p.chunk_proj2 > kStepMaxHidden || p.ff % p.chunk_proj2 ||
      p.ranks_proj2 != p.ff / p.chunk_proj2 || p.ranks_proj2 > kStepMaxRanges)
    return "K split of the MLP projection";
  if (step_role_ctas(p) > sm_count() || sm_count() < kStepRows) return "more GEMM items per layer than SMs";
  if (p.first_helper != step_role_ctas(p) || p.head_slabs != (p.vocab + 127) / 128) return "inconsistent plan";
  return nullptr;
}

cudaError_t make_tile_map(const void* arena, long long rows, TileMap* out) {
  CUtensorMap map; std::memset(&map, 0, sizeof map);
  static_assert(sizeof(CUtensorMap) == sizeof(TileMap), "tensor map size");
  if (!make_map_2d(&map, arena, true, uint64_t(rows), 128, 128, 128, uint32_t(kTcStageK), true)) return cudaErrorInvalidValue;
  std::memcpy(out, &map, sizeof map);
  return cudaSuccess;
}

cudaError_t decode_step(const StepPlan& plan, const TileMap& tiles, cudaStream_t stream) {
  if (plan.batch < 1 || plan.batch > kStepRows || step_unsupported(plan)) return cudaErrorInvalidValue;
  const cudaError_t ready = allow_smem(decode_step_kernel, StepSmem::kBytes);
  if (ready != cudaSuccess) return ready;
  CUtensorMap map; std::memcpy(&map, &tiles, sizeof map);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(sm_count())); cfg.blockDim = dim3(kStepThreads); cfg.dynamicSmemBytes = StepSmem::kBytes; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;      // every CTA resident, or the launch fails
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_step_kernel, map, plan);
}

#ifdef TIB_TRACE
// Development builds: copies the timeline log out and clears it; returns the number of events.
extern "C" int ti_b200_trace_dump(unsigned long long* out, int capacity) {
  unsigned int n = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&n, g_trace_count, sizeof n);
  if (n > (1u << 16)) n = 1u << 16;
  if (int(n) > capacity) n = unsigned(capacity);
  cudaMemcpyFromSymbol(out, g_trace_buf, size_t(n) * sizeof(unsigned long long));
  if (capacity >= (1 << 16))      // the slot marks ride in the last 1024 words
    cudaMemcpyFromSymbol(out + (1 << 16) - 1024, g_trace_buf, 1024 * sizeof(unsigned long long), ((1 << 16) - 1024) * sizeof(unsigned long long));
  const unsigned int zero = 0;
  cudaMemcpyToSymbol(g_trace_count, &zero, sizeof zero);
  return int(n);
}
#endif

cudaError_t selftest_bounded_wait(cudaStream_t stream, unsigned int polls) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(polls);
  return cudaGetLastError();
}

cudaError_t device_status_address(unsigned int** address) {
  return cudaGetSymbolAddress(reinterpret_cast<void**>(address), g_device_status);
}

cudaError_t read_device_status(cudaStream_t stream, unsigned int* status) {
  cudaError_t st = cudaStreamSynchronize(stream);
  if (st != cudaSuccess) return st;
  st = cudaMemcpyFromSymbol(status, g_device_status, sizeof(unsigned int));
  if (st != cudaSuccess || *status == 0) return st;
  const unsigned int zero = 0;
  return cudaMemcpyToSymbol(g_device_status, &zero, sizeof zero);
}

}  // namespace tib
