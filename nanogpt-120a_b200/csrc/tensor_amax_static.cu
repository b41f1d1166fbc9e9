// nvfp4_tensor_amax_f32_static_scratch: the tensor amax of an f32 tensor with the per-chunk
// scratch kept inside the library instead of in a caller buffer.
//
// Why it exists.  nvfp4_tensor_amax_f32 wants a scratch plane of one float per 1024 values
// from the caller.  Some callers have no way to produce one at the point of the call: a host
// program that handed the whole device to its own arena at start-up and sized that arena
// before it knew about this library, a step loop in which a device allocation would
// synchronise the device and stall every other stream, or a process whose GPU is already
// full.  For them this entry allocates nothing, on the host or on the device, and calls no
// routine that allocates: the scratch is a fixed array in the library's device image.
//
// Limits.  The array holds kStaticChunkCapacity chunk values (256 KiB), so one call covers at
// most 2^26 values; larger tensors are refused with an error, never truncated.  There is one
// array per device, shared by every stream and host thread: two calls that overlap in time on
// the same device race on it and either may return a wrong maximum.  Calls issued to one
// stream, or otherwise ordered, are safe.  The first call on a device looks the array's
// address up in the loaded image (cudaGetSymbolAddress, which may also load the image); that
// is set-up work, so make one call during initialisation, before any stream capture begins.
//
// Nothing in the array has to start at zero: a call reads only the slots it has just written.
//
// The reference has no counterpart; the result is the value nvfp4_tensor_amax_f32 writes to
// out[0] (same max.f32 semantics as utils/nvfp4/quant/kernels/row_amax.rs:67-101).
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace nvfp4 {
namespace {

constexpr uint32_t kStaticChunkCapacity = 1u << 16;  // chunks of 1024 values
constexpr uint64_t kStaticMaxElements = static_cast<uint64_t>(kStaticChunkCapacity) * 1024u;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_static_chunk_amax[kStaticChunkCapacity];

__device__ __forceinline__ float warp_max_f32(float m) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max_f32(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

// Warps stride over 1024-value chunks and write each chunk's amax to scratch[chunk].
__global__ void __launch_bounds__(256)
    tensor_amax_chunks_static_kernel(const float* __restrict__ x, float* __restrict__ scratch, uint64_t n) {
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t warps = static_cast<uint64_t>(gridDim.x) * 8;
  const uint64_t chunks = (n + 1023) / 1024;
  for (uint64_t chunk = static_cast<uint64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); chunk < chunks; chunk += warps) {
    const uint64_t base = chunk * 1024;
    const float* p = x + base;
    float m = 0.0f;
    if (base + 1024 <= n && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(p) + i * 32 + lane);
        m = max_f32(m, max_f32(max_f32(fabsf(t.x), fabsf(t.y)), max_f32(fabsf(t.z), fabsf(t.w))));
      }
    } else {
      const uint32_t count = static_cast<uint32_t>(min(static_cast<uint64_t>(1024), n - base));
      for (uint32_t i = lane; i < count; i += 32) m = max_f32(m, fabsf(__ldg(p + i)));
    }
    m = warp_max_f32(m);
    if (lane == 0) scratch[chunk] = m;
  }
}

// One CTA: out[0] = max of scratch[0 .. chunk_count) (0 for an empty tensor).
__global__ void __launch_bounds__(256)
    static_chunks_max_kernel(const float* __restrict__ scratch, float* __restrict__ out, uint32_t chunk_count) {
  __shared__ float partial[8];
  float m = 0.0f;
  for (uint32_t i = threadIdx.x; i < chunk_count; i += 256) m = max_f32(m, scratch[i]);
  m = warp_max_f32(m);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) r = max_f32(r, partial[i]);
    out[0] = r;
  }
}

// Address of the scratch array on the current device, looked up once per device.
int static_scratch_address(float** ptr_out) {
  static std::mutex lock;
  static float* cached[kMaxDevices] = {};
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (device < 0 || device >= kMaxDevices) {
    set_last_error("nvfp4_tensor_amax_f32_static_scratch: device ordinal out of range");
    return static_cast<int>(cudaErrorInvalidDevice);
  }
  std::lock_guard<std::mutex> guard(lock);
  if (cached[device] == nullptr) {
    float* ptr = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_chunk_amax);
    if (err != cudaSuccess) {
      set_last_error("nvfp4_tensor_amax_f32_static_scratch: cudaGetSymbolAddress failed");
      return static_cast<int>(err);
    }
    cached[device] = ptr;
  }
  *ptr_out = cached[device];
  return 0;
}

}  // namespace
}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_tensor_amax_f32_static_scratch(void* stream, const float* x, float* out,
                                                    uint64_t element_count) {
  if (out == nullptr || (x == nullptr && element_count != 0)) {
    set_last_error("nvfp4_tensor_amax_f32_static_scratch: null pointer");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (element_count > kStaticMaxElements) {
    set_last_error(
        "nvfp4_tensor_amax_f32_static_scratch: element_count exceeds the built-in scratch (67108864 values); "
        "use nvfp4_tensor_amax_f32 with a caller buffer");
    return static_cast<int>(cudaErrorInvalidValue);
  }
  float* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != 0) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t chunks = static_cast<uint32_t>((element_count + 1023) / 1024);
  if (chunks != 0) {
    const uint32_t grid = min((chunks + 7u) / 8u, 148u * 8u);
    tensor_amax_chunks_static_kernel<<<grid, 256, 0, s>>>(x, scratch, element_count);
    count_launch();
  }
  static_chunks_max_kernel<<<1, 256, 0, s>>>(scratch, out, chunks);
  count_launch();
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) set_last_error(cudaGetErrorString(err));
  return static_cast<int>(err);
}
