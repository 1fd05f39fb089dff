// Bulk (prefill) projection of pre-RoPE K or V rows onto the per-head spectral bases, on the 5th-generation
// tensor core:  coef[t, h, r] = sum_d x[t, h*128 + d] * basis[h, r, d].
//
// The reference folds this projection into the k_proj / v_proj weights once (k_proj.W <- k_down @ k_proj.W,
// src/dynakv/kernels/compressed_attention.py:267-275) so that the projection layers emit spectral coefficients; with
// per-head 128 x 128 bases the same product is a batched 128-wide GEMM over the token axis, done here directly on the
// projection output: one CTA per (128-token tile, head), A = the token tile (K-major: dims contiguous), B = the basis
// (K-major as stored: basis[r][d]).  Both tiles arrive by TMA (two 64-element x 128-row boxes each, 128-byte swizzle),
// one tcgen05.mma chain of 8 k-steps fills a 128-column tensor-memory accumulator, each thread reads back one token
// row, rounds it to the 16-bit type into the (now free) token tile in the same swizzled layout, and two TMA stores
// write the tile out; rows past the end are zero-filled on the way in and clipped on the way out by the tensor maps.
// The kernel moves 32 KB in (plus the basis, which stays in L2) and 32 KB out per 4.2 MFLOP, so it is bound by HBM
// bandwidth (64 flop/byte), not by the tensor core; three CTAs fit on an SM and overlap each other's phases.  Heads
// vary fastest over the grid, so that the CTAs running together touch whole rows of x and out.
#include <cuda.h>

#include <type_traits>

#include "dkv_common.cuh"

namespace dkv {

namespace {

constexpr int PJ_TOK = 128, PJ_D = 128;
constexpr int PJ_HALF_BYTES = PJ_TOK * 64 * 2;        // one 64-element half of a tile: 128 rows of 128 bytes
constexpr int PJ_TILE_BYTES = 2 * PJ_HALF_BYTES;
constexpr uint32_t PJ_SPIN = 1u << 22;

__device__ __forceinline__ uint32_t pj_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// K-major operand in the 128-byte swizzle: 8-row groups 1024 bytes apart; the k-step is taken on the start address
__device__ __forceinline__ uint64_t pj_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ bool pj_wait(unsigned long long* bar, uint32_t parity) {
  bool ok = false;
  for (uint32_t it = 0; it < PJ_SPIN && !ok; ++it) {
    uint32_t r;
    asm volatile("{\n.reg .pred q;\nmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\nselp.u32 %0, 1, 0, q;\n}"
                 : "=r"(r) : "r"(pj_smem(bar)), "r"(parity) : "memory");
    ok = r != 0;
  }
  return ok;
}
__device__ __forceinline__ void pj_tma_load(uint32_t dst, const CUtensorMap* map, int c0, int c1, unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(pj_smem(bar)) : "memory");
}
__device__ __forceinline__ void pj_tma_store(const CUtensorMap* map, int c0, int c1, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(c0), "r"(c1), "r"(src) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(128) project_bulk_kernel(const __grid_constant__ CUtensorMap map_x,
                                                           const __grid_constant__ CUtensorMap map_b,
                                                           const __grid_constant__ CUtensorMap map_o, int n_heads,
                                                           int32_t* status) {
  extern __shared__ unsigned char pj_raw[];
  // the swizzle pattern is taken on absolute shared-memory addresses: tiles start on 1024-byte boundaries
  unsigned char* a_tile = pj_raw + ((1024u - (pj_smem(pj_raw) & 1023u)) & 1023u);
  unsigned char* b_tile = a_tile + PJ_TILE_BYTES;
  __shared__ alignas(8) unsigned long long full_bar, done_bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int h = blockIdx.x % n_heads;
  const int t0 = (blockIdx.x / n_heads) * PJ_TOK;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pj_smem(&full_bar)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pj_smem(&done_bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pj_smem(&full_bar)), "r"(2 * PJ_TILE_BYTES) : "memory");
    pj_tma_load(pj_smem(a_tile), &map_x, h * PJ_D, t0, &full_bar);
    pj_tma_load(pj_smem(a_tile) + PJ_HALF_BYTES, &map_x, h * PJ_D + 64, t0, &full_bar);
    pj_tma_load(pj_smem(b_tile), &map_b, 0, h * PJ_D, &full_bar);
    pj_tma_load(pj_smem(b_tile) + PJ_HALF_BYTES, &map_b, 64, h * PJ_D, &full_bar);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pj_smem(&tmem_slot)), "r"(128));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    if (pj_wait(&full_bar, 0)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;   // 0 = f16, 1 = bf16
      // D fp32, A and B K-major, N = 128, M = 128
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t koff = (uint32_t)((ks >> 2) * PJ_HALF_BYTES + (ks & 3) * 32);
        asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, q;\n}"
                     ::"r"(tmem), "l"(pj_desc(pj_smem(a_tile) + koff)), "l"(pj_desc(pj_smem(b_tile) + koff)), "r"(idesc),
                       "r"(ks > 0 ? 1u : 0u)
                     : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pj_smem(&done_bar)) : "memory");
    } else {
      // the loads never landed: release the waiters, who then see the verdict below
      set_status(status, DKV_ST_TIMEOUT);
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pj_smem(&done_bar)) : "memory");
    }
  }
  // bounded wait for the products; one verdict for the block (the tensor-memory loads below are warp-collective)
  bool ok = pj_wait(&done_bar, 0);
  ok = __syncthreads_and(ok) != 0;
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok) {
    // thread = token row = tensor-memory lane, 16 coefficients per load, written as two 16-byte pieces at the
    // swizzled place of the row (piece index XOR row % 8), which also keeps the writes free of bank conflicts
    const uint32_t lane_addr = tmem + ((uint32_t)(32 * warp) << 16);
#pragma unroll
    for (int blk = 0; blk < 8; ++blk) {
      uint32_t r[16];
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
          "tcgen05.wait::ld.sync.aligned;"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
            "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
          : "r"(lane_addr + 16 * blk)
          : "memory");
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
        if (std::is_same<T, __nv_bfloat16>::value) {
          __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
          w[i] = *reinterpret_cast<uint32_t*>(&v);
        } else {
          __half2 v = __floats2half2_rn(lo, hi);
          w[i] = *reinterpret_cast<uint32_t*>(&v);
        }
      }
      uint4* srow = reinterpret_cast<uint4*>(a_tile + (blk >> 2) * PJ_HALF_BYTES + tid * 128);
      const int piece = (2 * blk) & 7;
      srow[piece ^ (tid & 7)] = make_uint4(w[0], w[1], w[2], w[3]);
      srow[(piece + 1) ^ (tid & 7)] = make_uint4(w[4], w[5], w[6], w[7]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (ok && tid == 0) {
    pj_tma_store(&map_o, h * PJ_D, t0, pj_smem(a_tile));
    pj_tma_store(&map_o, h * PJ_D + 64, t0, pj_smem(a_tile) + PJ_HALF_BYTES);
    asm volatile("cp.async.bulk.commit_group;\ncp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  if (!ok && tid == 0) set_status(status, DKV_ST_TIMEOUT);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128));
  }
}

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link against the driver
typedef CUresult (*pj_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
pj_encode_fn pj_encoder() {
  static pj_encode_fn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<pj_encode_fn>(f);
  }();
  return fn;
}
// [rows, cols] 16-bit matrix with a row pitch in elements, boxes of 64 columns x 128 rows in the 128-byte swizzle
bool pj_map(CUtensorMap* m, int dtype, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch) {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)PJ_TOK};
  const cuuint32_t estr[2] = {1, 1};
  return pj_encoder()(m, dtype == DKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                      const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

}  // namespace dkv

using namespace dkv;

extern "C" int dkv_project_bulk(const dkv_project_args* a) {
  DKV_REQUIRE(a != nullptr, DKV_E_ARG, "dkv_project_bulk: null args");
  DKV_REQUIRE(a->dtype == DKV_F16 || a->dtype == DKV_BF16, DKV_E_ARG, "dkv_project_bulk: 16-bit element types only");
  DKV_REQUIRE(a->n_tokens >= 0 && a->n_heads >= 1 && a->n_heads <= 4096, DKV_E_ARG, "dkv_project_bulk: bad sizes");
  DKV_REQUIRE(a->x && a->basis && a->out, DKV_E_ARG, "dkv_project_bulk: null input");
  DKV_REQUIRE(a->x_stride >= (int64_t)a->n_heads * 128 && a->out_stride >= (int64_t)a->n_heads * 128, DKV_E_ARG,
              "dkv_project_bulk: row strides must cover n_heads * 128 elements");
  DKV_REQUIRE((((uintptr_t)a->x | (uintptr_t)a->basis | (uintptr_t)a->out) & 15) == 0 && (a->x_stride % 8) == 0 &&
                  (a->out_stride % 8) == 0,
              DKV_E_ALIGN, "dkv_project_bulk: pointers must be 16-byte aligned and row strides multiples of 8 elements");
  if (a->n_tokens == 0) return DKV_OK;
  const long long tiles = ((long long)a->n_tokens + PJ_TOK - 1) / PJ_TOK;
  DKV_REQUIRE(tiles * a->n_heads <= 2147483647LL, DKV_E_LIMIT, "dkv_project_bulk: too many tokens");
  DKV_REQUIRE(pj_encoder() != nullptr, DKV_E_CUDA, "dkv_project_bulk: the driver does not export cuTensorMapEncodeTiled");
  CUtensorMap mx, mb, mo;
  const uint64_t cols = (uint64_t)a->n_heads * 128;
  DKV_REQUIRE(pj_map(&mx, a->dtype, a->x, (uint64_t)a->n_tokens, cols, (uint64_t)a->x_stride) &&
                  pj_map(&mb, a->dtype, a->basis, cols, 128, 128) &&
                  pj_map(&mo, a->dtype, a->out, (uint64_t)a->n_tokens, cols, (uint64_t)a->out_stride),
              DKV_E_CUDA, "dkv_project_bulk: tensor map encoding failed");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  const unsigned grid = (unsigned)(tiles * a->n_heads);
  const size_t smem = 2 * PJ_TILE_BYTES + 1024;
  cudaError_t e;
  if (a->dtype == DKV_BF16) {
    e = cudaFuncSetAttribute(project_bulk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) project_bulk_kernel<__nv_bfloat16><<<grid, 128, smem, st>>>(mx, mb, mo, a->n_heads, a->status);
  } else {
    e = cudaFuncSetAttribute(project_bulk_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) project_bulk_kernel<__half><<<grid, 128, smem, st>>>(mx, mb, mo, a->n_heads, a->status);
  }
  DKV_REQUIRE(e == cudaSuccess, DKV_E_CUDA, "dkv_project_bulk: %s", cudaGetErrorString(e));
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}
