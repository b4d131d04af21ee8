// ti_b200_attention_decode_static_f16: the split-history decode attention for callers that cannot
// allocate device memory.
//
// The regular entry point (ti_b200_attention_decode_f16) needs a scratch buffer for the partial
// results of the history chunks, and somebody has to cudaMalloc it.  Some callers cannot: a serving
// loop that was given a fixed memory budget up front and must never touch the allocator again (an
// allocation or free can block, or synchronise the whole device, in the middle of a token step); an
// operator plugged into a host program that owns every byte of device memory and hands out only
// tensors and a stream; a process whose memory limit is already spent on weights and KV pages.
// For them the scratch lives here, in a fixed array that is part of the library image.
//
// Limits and rules:
//   * the array holds kStaticScratchFloats floats (4 MiB).  Every GPU that loads the library keeps
//     that much memory until the process exits, whether or not this entry point is used.  A problem
//     whose partials need more (batch * heads * ceil(kv_len / chunk) * 66 floats) is rejected with
//     TI_V2_INVALID_ARGUMENT and a message that names both numbers;
//   * no cudaMalloc, cudaFree or allocating library call is made, on any path;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it; later calls only launch.  Make that first call during
//     start-up, before any stream capture begins on that device;
//   * all calls on one device share the one array.  Two calls whose kernels can overlap on the GPU
//     (different streams, no dependency) race on it and corrupt each other's results: serialise them.
//     The array keeps the previous call's contents; nothing in it needs to start at zero, because
//     every partial that a call reads was written earlier by that same call.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "launch.hpp"
#include "tinyinfer_b200_ext.h"
#include "tinyinfer_backend_v2.h"

namespace {

constexpr long long kStaticScratchFloats = 1ll << 20;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the symbol; the usable device address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

std::mutex g_setup_lock;
float* g_scratch_address[kMaxDevices] = {};

// Device address of the array on `device`, which must be the current device.
cudaError_t scratch_on(int device, float** out) {
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (!g_scratch_address[device]) {
    float* address = nullptr;
    const cudaError_t st = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_scratch);
    if (st != cudaSuccess) return st;
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return cudaSuccess;
}

}  // namespace

// Defined in backend_api.cpp: shared argument checks and error text of the operator ABI.
namespace tib_api {
int enter_call(int device);
int fail_call(int status, const char* text);
int cuda_call(cudaError_t st);
int check_decode_attention(const void* q, const void* k, const void* v, const void* y, const void* kv_lengths, int batch, int heads,
                           int kv_len, int head_dim, int chunk);
}

extern "C" long long ti_b200_attention_decode_static_capacity_floats(void) { return kStaticScratchFloats; }

extern "C" int ti_b200_attention_decode_static_f16(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* y,
                                                   const int32_t* kv_lengths, int batch, int heads, int kv_len, int head_dim,
                                                   int chunk, uintptr_t stream, int device) {
  int st = tib_api::enter_call(device);
  if (st) return st;
  st = tib_api::check_decode_attention(q, k, v, y, kv_lengths, batch, heads, kv_len, head_dim, chunk);
  if (st) return st;
  if (device >= kMaxDevices) return tib_api::fail_call(TI_V2_INVALID_ARGUMENT, "device index beyond the static-scratch table");
  const long long need = ti_b200_attention_decode_scratch_floats(batch, heads, kv_len, chunk);
  if (need > kStaticScratchFloats) {
    char text[200];
    std::snprintf(text, sizeof text, "decode attention needs %lld scratch floats but the built-in scratch holds %lld; "
                  "use ti_b200_attention_decode_f16 with caller memory, a larger chunk, or a smaller batch", need, kStaticScratchFloats);
    return tib_api::fail_call(TI_V2_INVALID_ARGUMENT, text);
  }
  float* scratch = nullptr;
  const cudaError_t found = scratch_on(device, &scratch);
  if (found != cudaSuccess) return tib_api::cuda_call(found);
  const long long acc_floats = (long long)batch * heads * tib::decode_chunks(kv_len, chunk) * 64;
  tib::LaunchOpts opts;
  opts.stream = reinterpret_cast<cudaStream_t>(stream);
  return tib_api::cuda_call(tib::attention_packed_decode(q, k, v, y, kv_lengths, batch, heads, kv_len, chunk, scratch,
                                                        scratch + acc_floats, opts));
}
