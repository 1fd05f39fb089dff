// Shared helpers for the dynakv_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/dynakv_b200.h"

namespace dkv {

// ---- host-side error reporting -------------------------------------------
void set_error(const char* fmt, ...);

#define DKV_REQUIRE(cond, code, ...)  \
  do {                                \
    if (!(cond)) {                    \
      ::dkv::set_error(__VA_ARGS__);  \
      return (code);                  \
    }                                 \
  } while (0)

#define DKV_CHECK_LAUNCH()                                                        \
  do {                                                                            \
    cudaError_t e__ = cudaGetLastError();                                         \
    if (e__ != cudaSuccess) {                                                     \
      ::dkv::set_error("CUDA launch failed: %s (%s:%d)", cudaGetErrorString(e__), \
                       __FILE__, __LINE__);                                       \
      return DKV_E_CUDA;                                                          \
    }                                                                             \
  } while (0)

int sm_count();  // SM count of the current device (cached per device)

// ---- element type helpers ---------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

static inline size_t dtype_size(int dtype) { return dtype == DKV_F32 ? 4 : 2; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void set_status(int32_t* status, int32_t bit) {
  if (status != nullptr) atomicOr(status, bit);
}

}  // namespace dkv
