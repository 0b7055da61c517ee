// Shared device/host helpers for the sm_100a kernels in this directory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../../include/cuda_agent_b200.h"

namespace cab {

constexpr int kWarp = 32;
constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

__host__ __device__ inline bool aligned_to(const void* p, size_t bytes) {
  return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0;
}

// Status a launcher returns after enqueueing: catches bad launch configurations
// without synchronising the stream.
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? CAB_OK : CAB_ERR_LAUNCH; }

// Threads for a CTA that walks `chunks` equal pieces of a row, one piece per thread and pass: the largest
// multiple of 32 up to 256 that leaves no thread idle in the last pass (7168 bf16 columns in 16-byte pieces:
// 896 = 4 x 224), else 256.
inline int row_walk_threads(int chunks) {
  for (int t = 256; t >= 128; t -= 32)
    if (chunks % t == 0) return t;
  return 256;
}

// Opt-in to more than 48 KB of dynamic shared memory for `Kernel`. The attribute belongs to the
// (function, device) pair, so it is set once per device with that device current; one process may
// drive several GPUs and several host threads.
constexpr int kMaxDevices = 64;
template <auto Kernel>
inline bool ensure_dynamic_smem(int bytes) {
  static std::mutex mu;
  static bool done[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (!done[dev]) {
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    done[dev] = true;
  }
  return true;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, off));
  return x;
}

// bf16 bits -> fp32 is a 16-bit shift; exact.
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}

// Streaming 128-bit global accesses: data touched once, so it is marked
// evict-first in L1 and L2 instead of displacing anything reusable.
// The load is `asm volatile` so that it is issued exactly once, where it is
// written: a kernel that posts N loads before the first use keeps N in flight.
__device__ __forceinline__ float4 ld_stream(const float4* p) {
  float4 v;
  asm volatile("ld.global.cs.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(float4* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};"
               :
               : "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

}  // namespace cab
