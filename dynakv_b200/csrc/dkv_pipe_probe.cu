// Diagnostic: how long the tensor pipe is held by the three products of the decode kernel.
//
// One CTA per SM; one thread issues, back to back and without any other work on the SM, the tcgen05.mma chains of
// a 128-token tile exactly as the decode kernel shapes them -- (1) K = X Bk: 8 x (M=128, N=128, K=16), both operands
// in shared memory; (2) S = K' Q~^T: 8 x (M=128, N=16, K=16), A in tensor memory; (3) O^T += XV^T P: 8 x (M=128,
// N=16, K=16), both operands in shared memory, A MN-major -- over zero operands, commits once and waits (bounded).
// The result is clock cycles per tile: the floor the pipe itself puts under the kernel's time per tile.
// It has no counterpart in the reference and touches no cache state.
#include "dkv_common.cuh"

namespace dkv {

namespace {

constexpr uint32_t PROBE_SPIN = 1u << 22;
constexpr int PROBE_SMEM = 110592 + 128;

__device__ __forceinline__ uint32_t pp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t pp_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ void pp_mma_ss(uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void pp_mma_ts(uint32_t d, uint32_t a, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(d), "r"(a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}

__device__ __forceinline__ void pp_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int MASK>
__global__ void __launch_bounds__(128) pipe_probe_kernel(long long* cycles, int32_t* status, int tiles) {
  extern __shared__ __align__(1024) unsigned char pp_raw[];
  unsigned char* sA = pp_raw;             // K operand tile
  unsigned char* sB = pp_raw + 32768;     // basis
  unsigned char* sV = pp_raw + 65536;     // V operand tile
  unsigned char* sQ = pp_raw + 98304;     // rotated queries / P
  unsigned long long* bar = reinterpret_cast<unsigned long long*>(pp_raw + 110592);     // six barriers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pp_raw + 110592 + 64);
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int e = tid; e < 110592 / 16; e += blockDim.x) {
    // zero operands, or (mask bit 32) a non-trivial bit pattern: small bf16 values of both signs
    uint4 v = make_uint4(0, 0, 0, 0);
    if (MASK & 32) {
      const uint32_t h = (uint32_t)e * 2654435761u;
      v = make_uint4(0x3c003b00u ^ (h & 0x80ff80ffu), 0x3a803c80u ^ ((h >> 3) & 0x80ff80ffu), 0x3b403bc0u ^ ((h >> 7) & 0x80ff80ffu),
                     0x3c403a40u ^ ((h >> 11) & 0x80ff80ffu));
    }
    reinterpret_cast<uint4*>(pp_raw)[e] = v;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pp_smem(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pp_smem(bar)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pp_smem(bar + 1)));
    for (int i = 2; i < 6; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pp_smem(bar + i)));   // per-chain commits, never waited on
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = *tmem_slot;
  if (tid == 0) {
    const uint32_t id_k = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
    const uint32_t id_s = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
    const uint32_t id_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
    const long long t0 = clock64();
    for (int r = 0; r < tiles; ++r) {
      if (MASK & 1) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          pp_mma_ss(tb + 128 * (r % 3), pp_desc(pp_smem(sA) + ks * 4096, 2048, 128), pp_desc(pp_smem(sB) + ks * 4096, 2048, 128),
                    id_k, ks > 0);
        if (MASK & 16) pp_commit(pp_smem(bar + 2));
      }
      if (MASK & 2) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          pp_mma_ts(tb + 448 + 16 * (r & 1), tb + 128 * ((r + 1) % 3) + 32 * (ks >> 1) + 8 * (ks & 1),
                    pp_desc(pp_smem(sQ) + ks * 2 * 272, 272, 128), id_s, ks > 0);
        if (MASK & 16) pp_commit(pp_smem(bar + 3));
      }
      if (MASK & 4) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          pp_mma_ss(tb + 480, pp_desc(pp_smem(sV) + ks * 256, 128, 2048), pp_desc(pp_smem(sQ) + ks * 256, 128, 0), id_o, 1);
        if (MASK & 16) { pp_commit(pp_smem(bar + 4)); pp_commit(pp_smem(bar + 5)); }
      }
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pp_smem(bar)) : "memory");
    uint32_t ok = 0;
    for (uint32_t it = 0; it < PROBE_SPIN && !ok; ++it)
      asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0,1,0,p;\n}"
                   : "=r"(ok) : "r"(pp_smem(bar)), "r"(0u) : "memory");
    const long long t1 = clock64();
    if (!ok) set_status(status, DKV_ST_TIMEOUT);
    cycles[blockIdx.x] = t1 - t0;
  }
  if (tid == 32 && (MASK & 8)) {
    // product (3) from a second thread (another warp and SM sub-partition), as in the decode kernel
    const uint32_t id_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
    const long long t0 = clock64();
    for (int r = 0; r < tiles; ++r) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        pp_mma_ss(tb + 480, pp_desc(pp_smem(sV) + ks * 256, 128, 2048), pp_desc(pp_smem(sQ) + ks * 256, 128, 0), id_o, 1);
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pp_smem(bar + 1)) : "memory");
    uint32_t ok = 0;
    for (uint32_t it = 0; it < PROBE_SPIN && !ok; ++it)
      asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0,1,0,p;\n}"
                   : "=r"(ok) : "r"(pp_smem(bar + 1)), "r"(0u) : "memory");
    const long long t1 = clock64();
    if (!ok) set_status(status, DKV_ST_TIMEOUT);
    cycles[gridDim.x + blockIdx.x] = t1 - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(512));
  }
}

template <int MASK>
cudaError_t launch_probe(int n_cta, long long* cycles, int32_t* status, int tiles, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(pipe_probe_kernel<MASK>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM);
  if (e == cudaSuccess) pipe_probe_kernel<MASK><<<n_cta, 128, PROBE_SMEM, st>>>(cycles, status, tiles);
  return e;
}

}  // namespace

}  // namespace dkv

using namespace dkv;

extern "C" int dkv_probe_tensor_pipe(int32_t products, int32_t tiles, int32_t n_cta, int64_t* cycles, int32_t* status,
                                     void* stream) {
  DKV_REQUIRE(((products >= 1 && products <= 7) || products == 11 || products == 23 || products == 39 || products == 43) && tiles >= 1 && tiles <= 100000 && n_cta >= 1 &&
                  n_cta <= 1024,
              DKV_E_ARG, "dkv_probe_tensor_pipe: products is a mask of 1|2|4 (or 11 = 1|2 from one thread with product "
                         "(3) from a second), tiles in 1..100000, n_cta in 1..1024");
  DKV_REQUIRE(cycles != nullptr, DKV_E_ARG, "dkv_probe_tensor_pipe: null output");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  long long* out = reinterpret_cast<long long*>(cycles);
  cudaError_t e = cudaSuccess;
  switch (products) {
    case 1: e = launch_probe<1>(n_cta, out, status, tiles, st); break;
    case 2: e = launch_probe<2>(n_cta, out, status, tiles, st); break;
    case 3: e = launch_probe<3>(n_cta, out, status, tiles, st); break;
    case 4: e = launch_probe<4>(n_cta, out, status, tiles, st); break;
    case 5: e = launch_probe<5>(n_cta, out, status, tiles, st); break;
    case 6: e = launch_probe<6>(n_cta, out, status, tiles, st); break;
    case 11: e = launch_probe<11>(n_cta, out, status, tiles, st); break;
    case 23: e = launch_probe<23>(n_cta, out, status, tiles, st); break;   // 7 with a commit behind every chain
    case 39: e = launch_probe<39>(n_cta, out, status, tiles, st); break;   // 7 over non-zero operands
    case 43: e = launch_probe<43>(n_cta, out, status, tiles, st); break;   // 11 over non-zero operands
    default: e = launch_probe<7>(n_cta, out, status, tiles, st); break;
  }
  DKV_REQUIRE(e == cudaSuccess, DKV_E_CUDA, "dkv_probe_tensor_pipe: %s", cudaGetErrorString(e));
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}
