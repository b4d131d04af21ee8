// Device-side building blocks shared by every kernel of the INT8-weight decode path:
// binary16 helpers, the int8 -> fp16 weight dequantisation with the reference's rounding,
// mbarrier / TMA (cp.async.bulk.tensor) wrappers for sm_100a, and bounded waits.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records a code in
// the library's device status word and returns false, and the caller falls through to the
// kernel's exit path instead of spinning.  The status word is read by the host runtime after
// it synchronises (tib::read_device_status).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace tib {

constexpr uint32_t kSpinLimit = 1u << 22;   // polls of ~20-40 ns each: far above any healthy TMA latency

enum DeviceStatus : unsigned int {
  kStatusOk = 0,
  kStatusTmaTimeout = 1,       // a weight tile never arrived
  kStatusMmaTimeout = 2,       // a tcgen05.commit never arrived
  kStatusPipeTimeout = 3,      // a consumer never released a stage
  kStatusFlagTimeout = 4,      // persistent decode step: a tagged word of another CTA never arrived
  kStatusNoToken = 5,          // greedy argmax found no comparable logit in a row (all NaN)
};

// One status word per device for the library (defined in kernels.cu, the only device translation unit).
#ifndef TIB_STATUS_DEFINED
extern __device__ unsigned int g_device_status;
#endif

__device__ __forceinline__ void report(unsigned int code) { atomicCAS(&g_device_status, 0u, code); }

// ------------------------------------------------------------------ binary16 helpers
__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }
__device__ __forceinline__ __half f2h(float f) { return __float2half_rn(f); }

// Weight used in every product: fp16_rn(float(q) * scale)  (reference load_stage,
// kernels/src/cuda/tc/gemm.cu:21-24 with dequantize_scalar).  Two at a time: the pair of fp32
// products is narrowed by one cvt.rn.f16x2.f32.
__device__ __forceinline__ __half2 dequant2(int q_lo, int q_hi, float s_lo, float s_hi) {
  return __floats2half2_rn(float(q_lo) * s_lo, float(q_hi) * s_hi);
}

// Four int8 weights of one 32-bit word at once, same values as dequant2 without integer-to-float conversions (which
// run on a narrow pipe and bound the tensor-core GEMM at decode sizes): byte b of (word ^ 0x80808080) is q + 128; placed
// under the exponent of 2^23 it is the float 8388608 + 128 + q exactly, one subtraction leaves float(q), one
// multiplication by the scale rounds once -- the product float(q) * scale of the reference -- and the pair is narrowed
// by cvt.rn.f16x2.f32.
__device__ __forceinline__ void dequant4(uint32_t word, float s0, float s1, float s2, float s3, __half2& lo, __half2& hi) {
  const uint32_t u = word ^ 0x80808080u;
  const float f0 = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7650)) - 8388736.f;
  const float f1 = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7651)) - 8388736.f;
  const float f2 = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7652)) - 8388736.f;
  const float f3 = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7653)) - 8388736.f;
  lo = __floats2half2_rn(f0 * s0, f1 * s1);
  hi = __floats2half2_rn(f2 * s2, f3 * s3);
}

// acc += float(a) * float(b), one rounding (the product of two binary16 values is exact in
// binary32).  Mixed-precision FMA of the sm_100 family.
__device__ __forceinline__ float fma_f16(float acc, __half a, __half b) {
  asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(__half_as_ushort(a)), "h"(__half_as_ushort(b)));
  return acc;
}

// tanh-GELU exactly as the reference writes it (kernels/src/cuda/tc/elementwise.cu:30-31).
__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------ shared-memory addresses
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Cluster-scope forms: an address of this CTA's shared memory as seen in CTA `rank` of the cluster, a store
// and an arrive (release) through such an address, and a wait that acquires what remote arrivers released.
__device__ __forceinline__ uint32_t cluster_addr(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// one 64-bit scalar store (single-copy atomic): both halves become visible together
__device__ __forceinline__ void st_cluster_b64(uint32_t addr, unsigned long long v) {
  asm volatile("st.shared::cluster.b64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait; false (and a recorded status) if the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int code) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
    if (mbar_try(bar, parity)) return true;
  report(code);
  return false;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, unsigned int code) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
    if (mbar_try_cluster(bar, parity)) return true;
  report(code);
  return false;
}

// ------------------------------------------------------------------ TMA (tensor tile loads, no multicast)
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2-D tile load: x is the fast (contiguous) coordinate and x * element_size must be a multiple
// of 16 bytes; out-of-range parts of the box are filled with zeros.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// Generic-proxy writes to shared memory made visible to the async proxy (TMA / tcgen05).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ programmatic dependent launch
// wait: block until the kernels this launch depends on have completed and flushed.
// launch_dependents: allow the next kernel in the stream to start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------ optional timeline (development builds only)
// With -DTIB_TRACE block (0,0,0) of every kernel records %globaltimer at entry (0), after its dependency
// wait (1) and at exit (2); tib::trace_dump copies the log out.  Without the macro nothing is compiled in.
#ifdef TIB_TRACE
__device__ unsigned long long g_trace_buf[1 << 16];   // this header is compiled into one device unit only
__device__ unsigned int g_trace_count = 0;
// any one thread of block (0,0,0): event `what` (< 256) of kernel `kernel`
__device__ __forceinline__ void trace_mark(int kernel, int what) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned int i = atomicAdd(&g_trace_count, 1u);
    if (i < (1u << 16) - 1024) g_trace_buf[i] = (unsigned long long)(kernel * 256 + what) << 48 | (t & ((1ull << 48) - 1));
  }
}
__device__ __forceinline__ void trace_event(int kernel, int what) { if (threadIdx.x == 0) trace_mark(kernel, what); }
// fire-and-forget variant for marks inside a pipeline: slot `what` of the last 1024 words, last writer wins
__device__ __forceinline__ void trace_slot(int what) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_trace_buf[(1 << 16) - 1024 + what] = t;
  }
}
#else
#define trace_event(kernel, what) ((void)0)
#define trace_mark(kernel, what) ((void)0)
#define trace_slot(what) ((void)0)
#endif
enum TraceKernel { kTrEmbed = 1, kTrLayerNorm, kTrGemmTc, kTrGemv, kTrAttnDecode, kTrAttnTile, kTrCombine, kTrArgmax, kTrAdvance };

// ------------------------------------------------------------------ argmax merge word
// (value, index) as one 64-bit word whose unsigned order is: larger value first, lower index among equal values.
__device__ __forceinline__ unsigned long long argmax_pack(float v, int index) {
  const uint32_t u = __float_as_uint(v + 0.f);                      // -0 -> +0: equal values must compare equal
  const uint32_t ordered = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return (unsigned long long)ordered << 32 | (0xffffffffu - uint32_t(index));
}

// ------------------------------------------------------------------ warp reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

}  // namespace tib
