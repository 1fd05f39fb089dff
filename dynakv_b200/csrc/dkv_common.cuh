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

// Programmatic dependent launch.  The kernel after this one in the stream may be scheduled as soon as every CTA
// of this one has called launch_dependents (or exited); it must call wait before touching anything the kernel
// before it writes -- wait returns when that kernel has completed and its writes are visible.  Both are no-ops
// when the launch did not ask for programmatic serialization.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with the programmatic-serialization attribute: the kernel may start while its predecessor in the stream
// is still running, up to its pdl_wait().  Works under stream capture (the edge becomes a programmatic one).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// Device-side routing: true when batch row b (already mapped through batch_index) does not take part in this call.
__device__ __forceinline__ bool row_routed_out(const dkv_attn_args& p, int b) {
  if (p.route_min_tokens <= 0 && p.route_max_tokens <= 0) return false;
  int s = p.seq_len;
  if (p.seq_lens) s = min(s, max(p.seq_lens[b], 0));
  return s < p.route_min_tokens || (p.route_max_tokens > 0 && s >= p.route_max_tokens);
}

__device__ __forceinline__ void set_status(int32_t* status, int32_t bit) {
  if (status != nullptr) atomicOr(status, bit);
}

}  // namespace dkv
