// Shared helpers for the sm_100a block-sparse kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include <mutex>

#include "../../include/sparta_b200.h"

namespace sparta {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SPARTA_OK : static_cast<int>(e);
}

// A kernel's dynamic shared memory limit is an attribute of the (kernel, device) pair, so a process that
// drives several GPUs has to set it on each of them.  One instance per kernel instantiation; the table
// is filled under a mutex because launches may come from several host threads.
constexpr int kMaxDevices = 64;
struct SmemAttrOnce {
  std::mutex mu;
  bool done[kMaxDevices] = {};
  template <typename Kernel>
  cudaError_t ensure(Kernel kern, int bytes) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool tracked = dev >= 0 && dev < kMaxDevices;
    std::lock_guard<std::mutex> guard(mu);
    if (tracked && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && tracked) done[dev] = true;
    return e;
  }
};

inline bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

inline bool valid_bcs_block(int b) { return is_pow2(b) && b >= 4 && b <= 256; }

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace sparta
