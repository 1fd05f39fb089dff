// Tensor-core decode attention over per-KV-head ragged arenas (bf16 / fp16, D = 128, R <= 128,
// lengths multiples of 8, gap-free prefix-sum packed rows).  One kernel template serves
//   * the short-cache fused path: one CTA per (batch row, KV head), result projected in-kernel;
//   * the long-cache split path: a persistent grid that partitions each KV head's token space
//     evenly over CTAs and writes (m, l, latent accumulator) partials, merged by a combine kernel.
//
// Per CTA 16 warps work on 128-token stages:
//   4 gather warps : copy each token's ragged coefficient row (16-byte cp.async, zero fill past the row's
//                    length) into a K-major, unswizzled operand tile in shared memory;
//   1 MMA warp     : K[128 x 128] = X[128 x 128] . Bk with eight tcgen05.mma (M=128, N=128, K=16), the
//                    accumulator in tensor memory (two 128-column buffers), completion by tcgen05.commit;
//   1 V loader     : the stage's V bytes are one contiguous range (rows are gap-free): cp.async.bulk into
//                    a shared-memory ring, mbarrier transaction completion;
//   1 rotator      : q~ = scale . R(-s0) q per 64-token sub-stage, so consumers rotate K only locally;
//   8 consumers    : one 16-token group each per stage.  tcgen05.ld.16x256b brings the group's K rows into
//                    registers in the mma.sync accumulator layout; RoPE in fp32 (pairs (j, j+64) sit in
//                    one thread); S = K'.q~^T with mma.sync reusing the fragments as A operand; online
//                    softmax (exp2, shuffles); O^T[r x heads] += XV^T . P with mma.sync, XV read by
//                    ldmatrix.trans straight from the ragged V bytes.
//
// Reference math: src/dynakv/kernels/fused.py:28-142 (fused), two_stage.py:52-157,211-281 (two-stage;
// the latent-space V accumulation with one up-projection at the end is two_stage.py:261-277).
#include <math.h>

#include <type_traits>

#include "dkv_common.cuh"

namespace dkv {

constexpr int D = 128;
constexpr int NCW = 8;                 // consumer warps (warp w owns TMEM lanes 32(w&3)+16(w>>2) .. +15)
constexpr int W_ROT = 8;               // query rotator
constexpr int W_VLOAD = 9;             // V loader
constexpr int W_GATHER0 = 10;          // gather warps 10..13 (32 tokens of the stage each)
constexpr int N_GATHER = 4;
constexpr int W_MMA = 14;              // tcgen05.mma issuer, owns the tensor-memory allocation
constexpr int NTHREADS = 16 * 32;      // 4 warps per SM sub-partition, 128 registers per thread
constexpr int ST_TOK = 128;            // tokens per stage = rows of one UMMA
constexpr int QSUB = 64;               // tokens per query-rotation sub-stage (extent of the local RoPE table)
constexpr int GRP_PER_STAGE = ST_TOK / 16;  // 16-token groups, one per consumer warp
constexpr int NSLOT = 4;               // stages in flight (metadata, rotated queries, V bytes)
constexpr int PD = 4;                  // prefetch distance for the stage metadata (stages)
constexpr int MSLOT = NSLOT + PD;      // metadata staging slots
constexpr int NBUF = 2;                // K operand tiles in shared memory = accumulator buffers in tensor memory
constexpr int A_TILE_BYTES = ST_TOK * 128 * 2;   // 128 tokens x 128 coefficients, chunk-major (see gather)
constexpr int TMEM_COLS = NBUF * 128;  // fp32 accumulator columns
constexpr int Q_PITCH = 272;
constexpr int HP = 4;                  // query heads per KV head supported by this kernel
constexpr int RING_BYTES = 36 * 1024;  // V ring; >= one worst-case stage (128 tokens x 256 B)
constexpr int MAX_BATCH = 1024;
constexpr int PART_STRIDE = 2 + 128;   // floats per (head) partial record: m, l, latent[128]
constexpr uint32_t SPIN_LIMIT = 1u << 22;

struct __align__(16) StageHdr {   // V side of one stage
  uint32_t base;    // shared-memory byte address of the stage's bytes
  int32_t n_tok;
  int32_t start;    // arena element offset of the stage's first coefficient
  int32_t elems;    // elements copied for the stage (0 when the stage was rejected)
};

struct StageMeta {   // raw slices of one side's cache metadata for one stage, copied asynchronously
  alignas(16) int lens[ST_TOK];
  alignas(16) int offs[ST_TOK];
};

struct SmemLayout {
  alignas(1024) unsigned char a_tile[NBUF][A_TILE_BYTES];   // chunk c (8 coefficients) of token t at c*2048 + t*16
  alignas(1024) unsigned char basis[128 * 256];             // Bk[r][d] at (r/8)*2048 + (d/8)*128 + (r%8)*16 + (d%8)*2
  alignas(128) unsigned char ring[RING_BYTES];
  alignas(16) float4 trig[QSUB * 64 / 2];            // [t][nt ^ (t&7)][q] -> {c_j, c_j+1, s_j, s_j+1}
  alignas(16) unsigned char qrot[NSLOT][ST_TOK / QSUB][HP * Q_PITCH];
  alignas(16) StageMeta meta[2][MSLOT];              // [0] K side, [1] V side
  alignas(16) StageHdr hdr[NSLOT];
  alignas(16) float merge[NCW][HP][PART_STRIDE];
  alignas(16) float knorm_w[D];
  alignas(16) unsigned char zero_chunk[16];
  alignas(8) unsigned long long full_k[NSLOT];    // K metadata (4 gather warps) + rotated queries (rotator)
  alignas(8) unsigned long long full_v[NSLOT];    // V bytes (loader arrive + transaction bytes)
  alignas(8) unsigned long long empty_bar[NSLOT]; // 8 consumer groups done with the stage
  alignas(8) unsigned long long a_full[NBUF];     // operand tile written (4 gather warps)
  alignas(8) unsigned long long a_free[NBUF];     // operand tile consumed by the tensor core (commit)
  alignas(8) unsigned long long t_ready[NBUF];    // accumulator buffer written (commit)
  alignas(8) unsigned long long t_free[NBUF];     // accumulator buffer read out (8 consumer warps)
  int prefix[MAX_BATCH + 1];
  int ring_start[NSLOT];
  int abort_flag;
  uint32_t tmem_base;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait for a whole warp: returns false (and raises the CTA's abort flag) instead of spinning forever.
// Only lane 0 polls the barrier -- hundreds of threads polling would compete with the async copies for the
// shared-memory barrier unit -- and the result (with lane 0's acquire) is handed to the warp by the shuffle.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 0;
  if ((threadIdx.x & 31) == 0) {
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
      if (mbar_test(bar, parity)) { ok = 1; break; }
      if ((it & 1023u) == 1023u && *abort_flag) break;
      if (it + 1 == SPIN_LIMIT) *abort_flag = 1;
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// tcgen05 (5th generation tensor core) helpers ---------------------------------------------------------
// Shared-memory matrix descriptor, no swizzle: start address, leading and stride byte offsets in 16-byte
// units, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Two 16-row x 32-column fp32 blocks of tensor memory in the mma.sync accumulator layout:
// v[i][0..3] = n-tile i {(row g, col 2q), (g, 2q+1), (g+8, 2q), (g+8, 2q+1)}, g = lane/4, q = lane%4;
// v[0..3] from addr_lo, v[4..7] from addr_hi.  The wait is part of the same statement, so no register of
// the result can be touched before the loads have landed.
__device__ __forceinline__ void tmem_ld_2x_16x32(float (&v)[8][4], uint32_t addr_lo, uint32_t addr_hi) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%32];\n"
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%33];\n"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr_lo), "r"(addr_hi)
      : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) v[i][j] = __uint_as_float(r[4 * i + j]);
}

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// Loads of data that does not change after the prologue barrier (the basis) carry no ordering
// constraint, so the compiler is free to hoist and batch them.
__device__ __forceinline__ void ldsm_x4_t_const(uint32_t (&r)[4], uint32_t addr) {
  asm("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
      : "r"(addr));
}

// 8x8 transpose of 16-bit elements across the warp: lane (g, q) gives row g, columns 2q,2q+1 and
// receives row g, columns 2q,2q+1 of the transposed matrix.
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t x) {
  uint32_t y;
  asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

template <typename T>
struct Mma;
template <>
struct Mma<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ void run0(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {   // c = a.b (no accumulator input)
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <>
struct Mma<__half> {
  static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ void run0(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// --------------------------------------------------------------- work partition
// Token space of one KV head: batch rows back to back, each rounded up to whole 64-token units.
__device__ __forceinline__ int row_tokens(const dkv_attn_args& p, int i) {
  const int b = p.batch_index ? p.batch_index[i] : i;
  int s = p.seq_len;
  if (p.seq_lens) s = min(s, max(p.seq_lens[b], 0));
  return s;
}
__host__ __device__ __forceinline__ int unit_begin(int k, int n, int total_units) {
  return (int)(((long long)k * (long long)total_units) / (long long)n);
}

struct WsHeader {  // start of the split workspace, written by the split kernel, read by the combine kernel
  int total_units;
  int n_cta;
  int prefix[MAX_BATCH + 1];
};
__host__ __device__ constexpr size_t ws_header_bytes() { return (sizeof(WsHeader) + 255) / 256 * 256; }

// ------------------------------------------------------------------ the kernel
template <typename T, bool FUSED, bool KNORM>
__global__ void __launch_bounds__(NTHREADS, 1) mma_decode_kernel(dkv_attn_args p, float log_theta, int n_cta, int meta16) {
  extern __shared__ unsigned char smem_raw[];
  SmemLayout& sm = *reinterpret_cast<SmemLayout*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.y;                        // KV head == basis group == arena within the batch row
  const int G = p.n_q_heads / p.n_basis_groups;    // query heads sharing this KV head (<= HP)
  const int R = p.rank;
  volatile int* abort_flag = &sm.abort_flag;

  // ---- prologue A: partition table and barriers --------------------------------------------------
  if (warp == 0) {
    // inclusive scan of the per-row unit counts, 32 rows at a time
    int carry = 0;
    for (int base = 0; base < p.batch; base += 32) {
      const int i = base + lane;
      int v = (i < p.batch) ? (row_tokens(p, i) + ST_TOK - 1) / ST_TOK : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
      }
      if (i < p.batch) sm.prefix[i + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) {
      sm.prefix[0] = 0;
      sm.abort_flag = 0;
      for (int s = 0; s < NSLOT; ++s) {
        mbar_init(smem_u32(&sm.full_k[s]), N_GATHER + 1);      // gather warps (metadata) + rotator
        mbar_init(smem_u32(&sm.full_v[s]), 1);                 // V loader (with tx bytes)
        mbar_init(smem_u32(&sm.empty_bar[s]), GRP_PER_STAGE);  // one arrival per 16-token group
      }
      for (int s = 0; s < NBUF; ++s) {
        mbar_init(smem_u32(&sm.a_full[s]), N_GATHER);
        mbar_init(smem_u32(&sm.a_free[s]), 1);
        mbar_init(smem_u32(&sm.t_ready[s]), 1);
        mbar_init(smem_u32(&sm.t_free[s]), NCW);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
  }
  if (tid < 4) reinterpret_cast<uint32_t*>(sm.zero_chunk)[tid] = 0u;
  __syncthreads();

  const int total_units = sm.prefix[p.batch];
  int u_begin, u_end;
  if (FUSED) {
    u_begin = sm.prefix[blockIdx.x];
    u_end = sm.prefix[blockIdx.x + 1];
  } else {
    u_begin = unit_begin(blockIdx.x, n_cta, total_units);
    u_end = unit_begin(blockIdx.x + 1, n_cta, total_units);
    if (blockIdx.x == 0 && g == 0 && p.workspace) {
      WsHeader* wh = reinterpret_cast<WsHeader*>(p.workspace);
      for (int i = tid; i <= p.batch; i += NTHREADS) wh->prefix[i] = sm.prefix[i];
      if (tid == 0) { wh->total_units = total_units; wh->n_cta = n_cta; }
    }
  }
  const int n_stages = u_end - u_begin;

  if (FUSED && n_stages <= 0) {
    // row without tokens: zeros, flagged
    for (int e = tid; e < G * D; e += NTHREADS) {
      const int b = p.batch_index ? p.batch_index[blockIdx.x] : blockIdx.x;
      T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)(g * G + e / D) * p.out_stride_h;
      op[e % D] = from_f32<T>(0.f);
    }
    if (tid == 0) set_status(p.status, DKV_ST_EMPTY_ROW);
    return;
  }
  if (n_stages <= 0) return;

  // ---- prologue B: basis and local-rotation table (only CTAs that have work) ---------------------
  {
    // basis rows [R][128] -> the MN-major unswizzled operand layout of the tensor core: 8x8 core matrices,
    // element (r, d) at (r/8)*2048 + (d/8)*128 + (r%8)*16 + (d%8)*2; rows >= R are zero
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.k_up) + (size_t)g * R * D);
    for (int e = tid; e < 128 * 16; e += NTHREADS) {
      const int r = e >> 4, c = e & 15;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < R) v = src[r * 16 + c];
      *reinterpret_cast<uint4*>(sm.basis + (r >> 3) * 2048 + c * 128 + (r & 7) * 16) = v;
    }
    if (warp == W_MMA) {   // tensor-memory columns for the two accumulator buffers
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                   "r"(TMEM_COLS));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // local rotation table for offsets t = 0..63: angle = t * f_j, f_j = exp(-(2j/D) ln theta).
    // NTHREADS is a multiple of 64, so a thread keeps one j and steps t by NTHREADS/64: one exact
    // sincos for its first t, then a fixed-angle rotation per step (error ~1e-7 per step, <= 11 steps).
    static_assert(NTHREADS % 64 == 0, "trig table fill assumes a fixed j per thread");
    constexpr int TSTEP = NTHREADS / 64;
    float* tr = reinterpret_cast<float*>(sm.trig);
    const int j = tid & 63;
    const float f = expf(-((float)(2 * j) / (float)D) * log_theta);
    float sn, cs, ds, dc;
    sincosf((float)(tid >> 6) * f, &sn, &cs);
    sincosf((float)TSTEP * f, &ds, &dc);
    const int nt = j >> 3, q = (j & 7) >> 1;
    for (int t = tid >> 6; t < QSUB; t += TSTEP) {
      const int idx = ((t * 8 + (nt ^ (t & 7))) * 4 + q) * 4 + (j & 1);
      tr[idx] = cs;
      tr[idx + 2] = sn;
      const float c2 = cs * dc - sn * ds, s2 = sn * dc + cs * ds;
      cs = c2; sn = s2;
    }
    if (KNORM && tid < D) sm.knorm_w[tid] = p.k_norm_weight[tid];
  }
  proxy_fence_async();     // the basis was written with ordinary stores and is read by the tensor core
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  // first batch row touched by this CTA
  int row0 = 0;
  {
    int lo = 0, hi = p.batch;  // largest i with prefix[i] <= u_begin
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (sm.prefix[mid] <= u_begin) lo = mid; else hi = mid;
    }
    row0 = FUSED ? (int)blockIdx.x : lo;
  }

  if (warp == W_ROT) {
    // =========================== query rotator warp ===========================
    // For every 64-token sub-stage with base position s0 it publishes q~ = scale * R(-s0) q for the
    // group's heads, so that q~ . R(t) k = q . R(s0 + t) k with the local offset t = 0..63.
    const float f_lo = expf(-((float)(2 * lane) / (float)D) * log_theta);
    const float f_hi = expf(-((float)(2 * (lane + 32)) / (float)D) * log_theta);
    float cda, sda, cdb, sdb;
    sincosf((float)QSUB * f_lo, &sda, &cda);
    sincosf((float)QSUB * f_hi, &sdb, &cdb);
    const float qscale = rsqrtf((float)D) * 1.4426950408889634f;  // softmax scale and log2(e) folded into q
    float qa0[HP], qa1[HP], qb0[HP], qb1[HP];                      // dims lane, lane+64 | lane+32, lane+96
    int row = row0;
    for (int c = 0; c < n_stages; ++c) {
      const int slot = c % NSLOT;
      if (c >= NSLOT &&
          !mbar_wait(smem_u32(&sm.empty_bar[slot]), (uint32_t)(((c / NSLOT) - 1) & 1), abort_flag))
        break;
      const int u = u_begin + c;
      while (u >= sm.prefix[row + 1]) ++row;
      const bool row_start = (c == 0) || (u == sm.prefix[row]);
      const int b = p.batch_index ? p.batch_index[row] : row;
      const int s0 = (u - sm.prefix[row]) * ST_TOK;
#pragma unroll
      for (int sub = 0; sub < ST_TOK / QSUB; ++sub) {
        if (row_start && sub == 0) {
          float sa, ca, sb, cb;
          sincosf((float)s0 * f_lo, &sa, &ca);
          sincosf((float)s0 * f_hi, &sb, &cb);
#pragma unroll
          for (int h = 0; h < HP; ++h) {
            float x0 = 0.f, x1 = 0.f, y0 = 0.f, y1 = 0.f;
            if (h < G) {
              const T* qp = reinterpret_cast<const T*>(p.q) + (size_t)b * p.q_stride_b + (size_t)(g * G + h) * p.q_stride_h;
              x0 = to_f32(qp[lane]) * qscale; x1 = to_f32(qp[lane + 64]) * qscale;
              y0 = to_f32(qp[lane + 32]) * qscale; y1 = to_f32(qp[lane + 96]) * qscale;
            }
            qa0[h] = x0 * ca + x1 * sa; qa1[h] = x1 * ca - x0 * sa;
            qb0[h] = y0 * cb + y1 * sb; qb1[h] = y1 * cb - y0 * sb;
          }
        } else {
#pragma unroll
          for (int h = 0; h < HP; ++h) {
            const float x0 = qa0[h], x1 = qa1[h], y0 = qb0[h], y1 = qb1[h];
            qa0[h] = x0 * cda + x1 * sda; qa1[h] = x1 * cda - x0 * sda;
            qb0[h] = y0 * cdb + y1 * sdb; qb1[h] = y1 * cdb - y0 * sdb;
          }
        }
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          T* qd = reinterpret_cast<T*>(sm.qrot[slot][sub] + h * Q_PITCH);
          qd[lane] = from_f32<T>(qa0[h]); qd[lane + 64] = from_f32<T>(qa1[h]);
          qd[lane + 32] = from_f32<T>(qb0[h]); qd[lane + 96] = from_f32<T>(qb1[h]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.full_k[slot]));
    }
  }

  else if (warp == W_VLOAD) {
    // =========================== V loader warp ===========================
    // Per stage: copy the V side's raw lens/offs slices into a staging slot (cp.async, PD stages ahead), read
    // the stage's first and one-past-last arena offsets from them (rows are gap-free, so the stage is one
    // contiguous byte range), take ring space, and issue the bulk copy in two halves from two lanes.
    const dkv_side& sd = p.v;
    unsigned char* const ring = sm.ring;
    // per-row facts are cached and refreshed only when the stage sequence enters another batch row
    struct RowInfo { int row, arena, tokens, first_unit; };
    auto enter_row = [&](RowInfo& ri, int u) {
      while (u >= sm.prefix[ri.row + 1]) ++ri.row;
      const int b = p.batch_index ? p.batch_index[ri.row] : ri.row;
      ri.arena = b * p.arenas_per_batch + g;
      ri.tokens = row_tokens(p, ri.row);
      ri.first_unit = sm.prefix[ri.row];
    };
    RowInfo pre{row0, 0, 0, 0}, cur{row0, 0, 0, 0};
    int pre_end = -1, cur_end = -1;   // first unit past the cached row
    auto prefetch = [&](int c) {
      if (c < n_stages) {
        const int u = u_begin + c;
        if (u >= pre_end) { enter_row(pre, u); pre_end = sm.prefix[pre.row + 1]; }
        const int s0 = (u - pre.first_unit) * ST_TOK;
        StageMeta& dst = sm.meta[1][c % MSLOT];
        const int32_t* ls = sd.lens + (size_t)pre.arena * sd.lens_stride_a + s0;
        const int32_t* os = sd.offs + (size_t)pre.arena * sd.offs_stride_a + s0;
        const int left = pre.tokens - s0;                 // tokens of the row from s0 on (> 0)
        if (meta16) {
          // 16-byte copies with zero fill past the row's last token (never reads beyond it)
          const int t = lane * 4;
          const int nbytes = min(max(left - t, 0), 4) * 4;
          cp_async16_zfill(smem_u32(&dst.lens[t]), nbytes ? (const void*)(ls + t) : (const void*)ls, nbytes);
          cp_async16_zfill(smem_u32(&dst.offs[t]), nbytes ? (const void*)(os + t) : (const void*)os, nbytes);
        } else {
#pragma unroll
          for (int hh = 0; hh < ST_TOK / 32; ++hh) {
            const int t = lane + 32 * hh;
            if (t < left) {
              cp_async4(smem_u32(&dst.lens[t]), ls + t);
              cp_async4(smem_u32(&dst.offs[t]), os + t);
            } else {
              dst.lens[t] = 0; dst.offs[t] = 0;
            }
          }
        }
      }
      cp_async_commit();
    };
    for (int c = 0; c < PD; ++c) prefetch(c);

    int head = 0;         // ring allocation cursor (state is kept identical on all lanes)
    int oldest = 0;       // oldest stage whose ring bytes are still owned by consumers
    bool wrapped = false;
    bool ok = true;
    auto release_oldest = [&](int c) -> bool {
      const bool done = mbar_wait(smem_u32(&sm.empty_bar[oldest % NSLOT]), (uint32_t)((oldest / NSLOT) & 1), abort_flag);
      if (!done) return false;
      const int old_start = sm.ring_start[oldest % NSLOT];
      ++oldest;
      if (oldest < c) {
        const int new_start = sm.ring_start[oldest % NSLOT];
        if (new_start < old_start) wrapped = false;
      } else {
        head = 0;
        wrapped = false;
      }
      return true;
    };
    for (int c = 0; c < n_stages && ok; ++c) {
      const int slot = c % NSLOT;
      // the stage that last used this slot (and the staging slot the next prefetch overwrites) must be done
      while (ok && oldest <= c - NSLOT) ok = release_oldest(c);
      if (!ok) break;
      prefetch(c + PD);
      cp_async_wait<PD>();
      __syncwarp();
      const int u = u_begin + c;
      if (u >= cur_end) { enter_row(cur, u); cur_end = sm.prefix[cur.row + 1]; }
      const int s0 = (u - cur.first_unit) * ST_TOK;
      const int n_tok = min(ST_TOK, cur.tokens - s0);
      const StageMeta& mt = sm.meta[1][c % MSLOT];
      const int start_el = mt.offs[0];
      const int end_el = mt.offs[n_tok - 1] + mt.lens[n_tok - 1];
      int tot = end_el - start_el;
      // the byte range must be 16-byte aligned, inside the arena row and no larger than a full stage
      const bool bad = ((start_el | end_el) & 7) != 0 || start_el < 0 || tot < 0 || tot > ST_TOK * 128 ||
                       (int64_t)end_el > sd.flat_stride;
      if (bad) {
        if (lane == 0) set_status(p.status, DKV_ST_BAD_LENGTH);
        tot = 0;     // consumers see an empty stage and skip its tokens
      }
      const int need = tot * 2;

      int start = 0;
      while (ok) {
        if (oldest == c) { start = 0; head = 0; wrapped = false; break; }
        const int tail = sm.ring_start[oldest % NSLOT];
        if (!wrapped) {
          if (head + need <= RING_BYTES) { start = head; break; }
          if (need <= tail) { start = 0; wrapped = true; break; }
        } else {
          if (head + need <= tail) { start = head; break; }
        }
        ok = release_oldest(c);
      }
      if (!ok) break;
      head = start + need;
      __syncwarp();
      const uint32_t bar = smem_u32(&sm.full_v[slot]);
      const uint32_t base = smem_u32(ring + start);
      if (lane == 2) {
        sm.ring_start[slot] = start;
        StageHdr h;
        h.base = base; h.n_tok = n_tok; h.start = start_el; h.elems = tot;
        sm.hdr[slot] = h;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)need);
      // a thread sustains only a few bulk copies per microsecond: the range is cut in two 16-byte aligned
      // halves issued by two lanes; both complete on the same barrier
      if (lane < 2) {
        const int first = (need / 2) & ~15;
        const int off = lane ? first : 0, len = lane ? need - first : first;
        const unsigned char* src = reinterpret_cast<const unsigned char*>(
            reinterpret_cast<const T*>(sd.flat) + (size_t)cur.arena * sd.flat_stride + start_el);
        if (len > 0) bulk_g2s(base + (uint32_t)off, src + off, (uint32_t)len, bar);
      }
    }
    cp_async_wait<0>();
    if (!ok && lane == 0) set_status(p.status, DKV_ST_OVERFLOW);
  }

  else if (warp >= W_GATHER0 && warp < W_GATHER0 + N_GATHER) {
    // =========================== gather warps ===========================
    // Lane l of gather warp j owns token 32j + l of every stage: it stages the token's length and offset
    // (cp.async, PD stages ahead) and copies the token's coefficient row into the operand tile, one 16-byte
    // chunk per cp.async, chunk c of token t at c*2048 + t*16; chunks past the row's length are zero-filled
    // (source size 0), so the tensor core always multiplies a full 128 x 128 tile.
    const int t = (warp - W_GATHER0) * 32 + lane;
    const dkv_side& sd = p.k;
    struct RowInfo { int row, arena, tokens, first_unit; };
    auto enter_row = [&](RowInfo& ri, int u) {
      while (u >= sm.prefix[ri.row + 1]) ++ri.row;
      const int b = p.batch_index ? p.batch_index[ri.row] : ri.row;
      ri.arena = b * p.arenas_per_batch + g;
      ri.tokens = row_tokens(p, ri.row);
      ri.first_unit = sm.prefix[ri.row];
    };
    RowInfo pre{row0, 0, 0, 0}, cur{row0, 0, 0, 0};
    int pre_end = -1, cur_end = -1;
    auto prefetch_meta = [&](int c) {   // no commit: the caller groups it with the stage's data copies
      if (c < n_stages) {
        const int u = u_begin + c;
        if (u >= pre_end) { enter_row(pre, u); pre_end = sm.prefix[pre.row + 1]; }
        const int s0 = (u - pre.first_unit) * ST_TOK;
        StageMeta& dst = sm.meta[0][c % MSLOT];
        if (s0 + t < pre.tokens) {
          cp_async4(smem_u32(&dst.lens[t]), sd.lens + (size_t)pre.arena * sd.lens_stride_a + s0 + t);
          cp_async4(smem_u32(&dst.offs[t]), sd.offs + (size_t)pre.arena * sd.offs_stride_a + s0 + t);
        } else {
          dst.lens[t] = 0; dst.offs[t] = 0;
        }
      }
    };
    for (int c = 0; c < PD; ++c) { prefetch_meta(c); cp_async_commit(); }   // groups 0..PD-1
    auto publish = [&](int c) {   // the copies of stage c have landed: hand tile and metadata over
      proxy_fence_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&sm.a_full[c % NBUF]));
        mbar_arrive(smem_u32(&sm.full_k[c % NSLOT]));
      }
    };
    bool ok = true;
    int c = 0;
    for (; c < n_stages; ++c) {
      const int slot = c % NSLOT, buf = c % NBUF;
      // metadata slot (c+PD) % MSLOT was last used by stage c - NSLOT
      if (c >= NSLOT && !mbar_wait(smem_u32(&sm.empty_bar[slot]), (uint32_t)(((c / NSLOT) - 1) & 1), abort_flag)) { ok = false; break; }
      cp_async_wait<PD - 1>();   // group c (this stage's metadata) is complete
      const int u = u_begin + c;
      if (u >= cur_end) { enter_row(cur, u); cur_end = sm.prefix[cur.row + 1]; }
      StageMeta& mt = sm.meta[0][c % MSLOT];
      int len = mt.lens[t];
      const int off = mt.offs[t];
      if (((len | off) & 7) != 0 || len < 0 || len > R || off < 0 || (int64_t)off + len > sd.flat_stride) {
        set_status(p.status, DKV_ST_BAD_LENGTH);   // breaks the layout contract: token dropped, call flagged
        len = 0;
        mt.lens[t] = 0;
      }
      // the tensor core must be done with the tile that was in this buffer two stages ago
      if (c >= NBUF && !mbar_wait(smem_u32(&sm.a_free[buf]), (uint32_t)(((c / NBUF) - 1) & 1), abort_flag)) { ok = false; break; }
      const unsigned char* row_src = reinterpret_cast<const unsigned char*>(
          reinterpret_cast<const T*>(sd.flat) + (size_t)cur.arena * sd.flat_stride + (len > 0 ? off : 0));
      const uint32_t dst = smem_u32(sm.a_tile[buf]) + t * 16;
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const bool in = ch * 8 < len;
        cp_async16_zfill(dst + ch * 2048, in ? row_src + ch * 16 : row_src, in ? 16 : 0);
      }
      prefetch_meta(c + PD);
      cp_async_commit();                       // group PD + c
      if (c >= 1) { cp_async_wait<1>(); publish(c - 1); }   // groups up to PD + c - 1 are complete
    }
    cp_async_wait<0>();
    if (ok && n_stages > 0) publish(n_stages - 1);
  }
  else if (warp == W_MMA) {
    // =========================== tensor-core issuer ===========================
    // K tile = X[128 x 128] . Bk[128 x 128]: eight M=128, N=128, K=16 instructions per stage, fp32
    // accumulator in tensor-memory buffer c % 2.  Two commits: accumulator ready (consumers) and operand
    // tile free (gather warps).
    const uint32_t fmt = (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) ? 1u : 0u;   // 0 = f16, 1 = bf16
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
    const uint32_t basis_addr = smem_u32(sm.basis);
    for (int c = 0; c < n_stages; ++c) {
      const int buf = c % NBUF;
      const uint32_t ph = (uint32_t)((c / NBUF) & 1);
      if (!mbar_wait(smem_u32(&sm.a_full[buf]), ph, abort_flag)) break;
      if (c >= NBUF && !mbar_wait(smem_u32(&sm.t_free[buf]), ph ^ 1u, abort_flag)) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(sm.a_tile[buf]);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // A: K-major, 8-row core matrices 128 B apart (SBO), the two 8-coefficient chunks 2048 B apart (LBO)
          // B: MN-major, 8-column core matrices 128 B apart (SBO), the two 8-row groups 2048 B apart (LBO)
          umma_f16(tmem_base + buf * 128, umma_desc(a_addr + ks * 4096, 2048, 128),
                   umma_desc(basis_addr + ks * 4096, 2048, 128), idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&sm.t_ready[buf]));
        umma_commit(smem_u32(&sm.a_free[buf]));
      }
      __syncwarp();
    }
  }
  else if (warp < NCW) {
  // ============================= consumer warps =============================
  // Consumer warp w owns the 16-token group gi = 2*(w&3) + (w>>2) of every stage: those are the tensor-memory
  // lanes 32*(w&3) + 16*(w>>2) .. +15, the only ones a warp in SM sub-partition w&3 may read.
  const int gi = 2 * (warp & 3) + (warp >> 2);
  const uint32_t tmem_lane = (uint32_t)(16 * gi) << 16;
  const int gq = lane >> 2, qq = lane & 3;
  const uint32_t zero_addr = smem_u32(sm.zero_chunk);
  const float4* trig4 = sm.trig;

  int row = row0;
  int c = 0;                  // next stage
  while (row < p.batch && sm.prefix[row] < u_end) {
    const int c_hi = min(sm.prefix[row + 1], u_end) - u_begin;   // stages of this row: [.., c_hi)
    float m_run0 = -INFINITY, m_run1 = -INFINITY, l_part0 = 0.f, l_part1 = 0.f;   // heads 2qq, 2qq+1
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }

    for (; c < c_hi; ++c) {
      const int slot = c % NSLOT, buf = c % NBUF;
      if (*abort_flag) continue;
      const uint32_t phase = (uint32_t)((c / NSLOT) & 1);
      if (!mbar_wait(smem_u32(&sm.full_k[slot]), phase, abort_flag)) continue;
      // lengths as the gather warps left them (0 = token absent or rejected)
      const int klen = sm.meta[0][c % MSLOT].lens[gi * 16 + (lane & 15)];   // lanes 16..31 mirror lanes 0..15
      const uint32_t valid = __ballot_sync(0xffffffffu, klen > 0) & 0xffffu;
      // the stage's K tile in tensor memory
      if (!mbar_wait(smem_u32(&sm.t_ready[buf]), (uint32_t)((c / NBUF) & 1), abort_flag)) continue;
      tc_fence_after();
      const uint32_t tmem_tile = tmem_base + tmem_lane + buf * 128;
      if (valid == 0u) {
        tc_fence_before();
        if (lane == 0) mbar_arrive(smem_u32(&sm.t_free[buf]));
      }
      if (valid != 0u) {
        // ---------------- K from tensor memory, RoPE, S = K' . Q~^T : two passes over half of the head dims ----------------
        // Pass h handles dims [32h, 32h+32) and their rotation partners [64+32h, 64+32h+32): only 32 accumulator
        // registers are live at a time (this is what lets 16 warps fit on the SM).
        const uint32_t qbase = smem_u32(sm.qrot[slot][gi / (QSUB / 16)]);
        const int qr = lane & 7;   // ldmatrix rows 0..HP-1 = heads, the other rows read the zero chunk
        const uint32_t qaddr = (qr < HP) ? qbase + qr * Q_PITCH + (lane >> 3) * 16 : zero_addr;
        const int tA = (gi & (QSUB / 16 - 1)) * 16 + gq, tB = tA + 8;   // offsets inside the 64-token sub-stage
        float sacc[4] = {0.f, 0.f, 0.f, 0.f}, sacc2[4] = {0.f, 0.f, 0.f, 0.f};   // two chains: low dims / partners
        float ss0 = 0.f, ss1 = 0.f;     // sum of squares of the two token rows (K-RMSNorm)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          // this group's K rows, dims [32hf, 32hf+32) and their rotation partners [64+32hf, ..): acc[0..3] =
          // n-tiles 4hf+i (dims j), acc[4..7] = n-tiles 8+4hf+i (dims j+64), in the mma.sync accumulator layout
          float acc[8][4];
          tmem_ld_2x_16x32(acc, tmem_tile + 32 * hf, tmem_tile + 64 + 32 * hf);
          if (hf == 1) {   // both halves are in registers: the accumulator buffer may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.t_free[buf]));
          }
          if (KNORM) {
            // RMSNorm of K (Qwen3): the weight is applied here, the per-token 1/rms scales the score at the end
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              ss0 = fmaf(acc[i][0], acc[i][0], fmaf(acc[i][1], acc[i][1], ss0));
              ss1 = fmaf(acc[i][2], acc[i][2], fmaf(acc[i][3], acc[i][3], ss1));
              const int nt = (i >> 2) * 8 + 4 * hf + (i & 3);
              const float2 w = *reinterpret_cast<const float2*>(&sm.knorm_w[8 * nt + 2 * qq]);
              acc[i][0] *= w.x; acc[i][1] *= w.y; acc[i][2] *= w.x; acc[i][3] *= w.y;
            }
          }
          // local RoPE on packed fp32 pairs, packed to 16-bit A fragments
          uint32_t kl[4][2], kh[4][2];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int nt = 4 * hf + i;
            const float4 ta = trig4[(tA * 8 + (nt ^ (tA & 7))) * 4 + qq];   // {c_j, c_j+1, s_j, s_j+1}
            const float4 tb = trig4[(tB * 8 + (nt ^ (tB & 7))) * 4 + qq];
            {
              const float2 lo = make_float2(acc[i][0], acc[i][1]), hi = make_float2(acc[4 + i][0], acc[4 + i][1]);
              const float2 C = make_float2(ta.x, ta.y), S = make_float2(ta.z, ta.w);
              const float2 u = __fmul2_rn(hi, S);
              const float2 lo2 = __ffma2_rn(lo, C, make_float2(-u.x, -u.y));
              const float2 hi2 = __ffma2_rn(lo, S, __fmul2_rn(hi, C));
              kl[i][0] = Mma<T>::pack(lo2.x, lo2.y);
              kh[i][0] = Mma<T>::pack(hi2.x, hi2.y);
            }
            {
              const float2 lo = make_float2(acc[i][2], acc[i][3]), hi = make_float2(acc[4 + i][2], acc[4 + i][3]);
              const float2 C = make_float2(tb.x, tb.y), S = make_float2(tb.z, tb.w);
              const float2 u = __fmul2_rn(hi, S);
              const float2 lo2 = __ffma2_rn(lo, C, make_float2(-u.x, -u.y));
              const float2 hi2 = __ffma2_rn(lo, S, __fmul2_rn(hi, C));
              kl[i][1] = Mma<T>::pack(lo2.x, lo2.y);
              kh[i][1] = Mma<T>::pack(hi2.x, hi2.y);
            }
          }
          // S[tokens x heads] += K'[:, these dims] . Q~^T : the rotated fragments are the A operand, the rotated
          // queries the B operand.  16-dim steps 2hf, 2hf+1 (low dims) and 4+2hf, 4+2hf+1 (partners).
          uint32_t ql[4], qh[4];
          ldsm_x4(ql, (qr < HP) ? qaddr + hf * 64 : zero_addr);         // {step 2hf: dims 0-7, 8-15 ; step 2hf+1: ...}
          ldsm_x4(qh, (qr < HP) ? qaddr + (2 + hf) * 64 : zero_addr);
          Mma<T>::run(sacc, kl[0][0], kl[0][1], kl[1][0], kl[1][1], ql[0], ql[1]);
          Mma<T>::run(sacc, kl[2][0], kl[2][1], kl[3][0], kl[3][1], ql[2], ql[3]);
          Mma<T>::run(sacc2, kh[0][0], kh[0][1], kh[1][0], kh[1][1], qh[0], qh[1]);
          Mma<T>::run(sacc2, kh[2][0], kh[2][1], kh[3][0], kh[3][1], qh[2], qh[3]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) sacc[i] += sacc2[i];
        if (KNORM) {
          ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
          ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
          const float rs0 = rsqrtf(ss0 * (1.0f / D) + p.k_norm_eps), rs1 = rsqrtf(ss1 * (1.0f / D) + p.k_norm_eps);
          sacc[0] *= rs0; sacc[1] *= rs0; sacc[2] *= rs1; sacc[3] *= rs1;
        }
        // ---------------- V fragments: fetched now, used after the softmax ----------------
        const bool v_ok = mbar_wait(smem_u32(&sm.full_v[slot]), phase, abort_flag);
        uint32_t va[8][4];
        int vmax = 0;
        if (v_ok) {
          const StageHdr hv = sm.hdr[slot];
          const StageMeta& mv = sm.meta[1][c % MSLOT];
          const int tv = gi * 16 + (lane & 7) + 8 * (lane >> 4);   // token whose row this lane addresses
          int vlen_t = 0;
          uint32_t vrow = zero_addr;
          if (tv < hv.n_tok) {
            vlen_t = mv.lens[tv];
            const int vo = mv.offs[tv] - hv.start;
            if (((vlen_t | vo) & 7) != 0 || vlen_t < 0 || vlen_t > R || vo < 0 || vo + vlen_t > hv.elems) {
              set_status(p.status, DKV_ST_BAD_LENGTH);
              vlen_t = 0;
            }
            vrow = hv.base + ((uint32_t)vo >> 3) * 16u;
          }
          vmax = __reduce_max_sync(0xffffffffu, vlen_t);
          const int cpar = (lane >> 3) & 1;
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            if (mt * 16 < vmax) {
              const int chunk = 2 * mt + cpar;
              ldsm_x4_t(va[mt], (chunk * 8 < vlen_t) ? vrow + chunk * 16 : zero_addr);
            }
          }
        }
        // ---------------- online softmax (base 2) ----------------
        // this lane: tokens gq and gq+8, heads 2qq and 2qq+1; head maxima are reduced over the 8 token lanes
        float sc0 = sacc[0], sc1 = sacc[1], sc2 = sacc[2], sc3 = sacc[3];
        if (!((valid >> gq) & 1u)) { sc0 = -INFINITY; sc1 = -INFINITY; }
        if (!((valid >> (gq + 8)) & 1u)) { sc2 = -INFINITY; sc3 = -INFINITY; }
        float mx0 = fmaxf(sc0, sc2), mx1 = fmaxf(sc1, sc3);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
        }
        const float mn0 = fmaxf(m_run0, mx0), mn1 = fmaxf(m_run1, mx1);
        const float al0 = exp2f(m_run0 - mn0), al1 = exp2f(m_run1 - mn1);
        const float p0 = exp2f(sc0 - mn0), p1 = exp2f(sc1 - mn1), p2 = exp2f(sc2 - mn0), p3 = exp2f(sc3 - mn1);
        l_part0 = l_part0 * al0 + (p0 + p2);
        l_part1 = l_part1 * al1 + (p1 + p3);
        m_run0 = mn0; m_run1 = mn1;
        // P[tokens x heads] -> B operand [token pairs x head] by an 8x8 transpose per token half
        const uint32_t pb0 = movmatrix_t(Mma<T>::pack(p0, p1)), pb1 = movmatrix_t(Mma<T>::pack(p2, p3));
        if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { oacc[i][0] *= al0; oacc[i][1] *= al1; oacc[i][2] *= al0; oacc[i][3] *= al1; }
        }
        // ---------------- O^T[r x heads] += XV^T . P ----------------
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          if (mt * 16 < vmax) Mma<T>::run(oacc[mt], va[mt][0], va[mt][1], va[mt][2], va[mt][3], pb0, pb1);
        }
      } else {
        // nothing to do for this group, but its V bytes must have landed before the slot is handed back
        mbar_wait(smem_u32(&sm.full_v[slot]), phase, abort_flag);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.empty_bar[slot]));
    }

    // ---------------- row flush: merge the consumer warps' partial states ----------------
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l_part0 += __shfl_xor_sync(0xffffffffu, l_part0, o);
      l_part1 += __shfl_xor_sync(0xffffffffu, l_part1, o);
    }
    if (gq == 0) {
      if (2 * qq < HP) { sm.merge[warp][2 * qq][0] = m_run0; sm.merge[warp][2 * qq][1] = l_part0; }
      if (2 * qq + 1 < HP) { sm.merge[warp][2 * qq + 1][0] = m_run1; sm.merge[warp][2 * qq + 1][1] = l_part1; }
    }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const int r = 16 * mt + gq;
      if (2 * qq < HP) { sm.merge[warp][2 * qq][2 + r] = oacc[mt][0]; sm.merge[warp][2 * qq][2 + r + 8] = oacc[mt][2]; }
      if (2 * qq + 1 < HP) { sm.merge[warp][2 * qq + 1][2 + r] = oacc[mt][1]; sm.merge[warp][2 * qq + 1][2 + r + 8] = oacc[mt][3]; }
    }
    consumer_bar();
    const int b = p.batch_index ? p.batch_index[row] : row;
    const int ctid = tid;  // consumer threads come first in the block
    constexpr int N_ITEMS = HP * 128, N_IT = (N_ITEMS + NCW * 32 - 1) / (NCW * 32);
    float outv[N_IT], L_tot[N_IT], M_tot[N_IT];
#pragma unroll
    for (int it = 0; it < N_IT; ++it) {
      const int item = ctid + it * (NCW * 32);   // (head, r)
      outv[it] = 0.f; L_tot[it] = 0.f; M_tot[it] = -INFINITY;
      if (item >= N_ITEMS) continue;
      const int h = item >> 7, r = item & 127;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NCW; ++w) M = fmaxf(M, sm.merge[w][h][0]);
      float v = 0.f, L = 0.f;
#pragma unroll
      for (int w = 0; w < NCW; ++w) {
        const float mw = sm.merge[w][h][0];
        const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        v = fmaf(sm.merge[w][h][2 + r], wgt, v);
        L = fmaf(sm.merge[w][h][1], wgt, L);
      }
      outv[it] = v; L_tot[it] = L; M_tot[it] = M;
    }
    if (!FUSED) {
      // partial record (row, cta) -> entry row + blockIdx.x of this KV head
      float* ws = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p.workspace) + ws_header_bytes());
      const size_t entries_per_group = (size_t)p.batch + n_cta;
      float* rec = ws + (((size_t)g * entries_per_group + (size_t)row + blockIdx.x) * HP) * PART_STRIDE;
#pragma unroll
      for (int it = 0; it < N_IT; ++it) {
        const int item = ctid + it * (NCW * 32);
        if (item >= N_ITEMS) continue;
        const int h = item >> 7, r = item & 127;
        rec[h * PART_STRIDE + 2 + r] = outv[it];
        if (r == 0) { rec[h * PART_STRIDE] = M_tot[it]; rec[h * PART_STRIDE + 1] = L_tot[it]; }
      }
      consumer_bar();
    } else {
      consumer_bar();   // all reads of merge[] done; reuse merge[0] as the normalised latent [HP][128]
      float* lat = &sm.merge[0][0][0];
#pragma unroll
      for (int it = 0; it < N_IT; ++it) {
        const int item = ctid + it * (NCW * 32);
        if (item >= N_ITEMS) continue;
        const float L = L_tot[it];
        lat[item] = L > 0.f ? outv[it] / L : 0.f;
        if (L <= 0.f && (item & 127) == 0 && (item >> 7) < G) set_status(p.status, DKV_ST_EMPTY_ROW);
      }
      consumer_bar();
      const T* vup = reinterpret_cast<const T*>(p.v_up) + (size_t)g * R * D;
#pragma unroll
      for (int it = 0; it < N_IT; ++it) {
        const int item = ctid + it * (NCW * 32);
        const int h = item >> 7, d = item & 127;
        if (item < N_ITEMS && h < G) {
          float o = 0.f;
          for (int r = 0; r < R; ++r) o = fmaf(lat[h * 128 + r], to_f32(vup[(size_t)r * D + d]), o);
          T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)(g * G + h) * p.out_stride_h;
          op[d] = from_f32<T>(o);
        }
      }
      consumer_bar();
    }
    ++row;
  }
  }   // consumer warps

  // ---- epilogue: every warp arrives here; the tensor memory is returned by the warp that allocated it ----
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
  if (*abort_flag && tid == 0) set_status(p.status, DKV_ST_OVERFLOW);
}

// Merge the split partials of one (batch row, query head) and project through Bv.
// 128 threads; the partial records of the row are read with independent loads (weights first, then the
// latent vectors 8 records at a time) so the kernel is not a chain of dependent L2 round trips.
constexpr int COMBINE_MAX_PART = 160;   // >= CTAs per KV head (at most the SM count)
template <typename T>
__global__ void __launch_bounds__(128) split_combine_kernel(dkv_attn_args p) {
  __shared__ float lat_s[128];
  __shared__ float wgt_s[COMBINE_MAX_PART];
  __shared__ float red_s[4][128];
  const WsHeader* wh = reinterpret_cast<const WsHeader*>(p.workspace);
  const float* ws = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(p.workspace) + ws_header_bytes());
  const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.n_q_heads / p.n_basis_groups, g = h / G, hl = h - g * G, R = p.rank;
  const int n_cta = wh->n_cta, total_units = wh->total_units;
  const int u_lo = wh->prefix[i], u_hi = wh->prefix[i + 1];
  const size_t entries_per_group = (size_t)p.batch + n_cta;
  // CTA k of this KV head covered units [unit_begin(k), unit_begin(k+1)); those that overlap this row's
  // units [u_lo, u_hi) each left one partial record at entry (row + k).
  int k_lo = 0, k_hi = -1;
  if (u_hi > u_lo && total_units > 0) {
    k_lo = (int)(((long long)u_lo * n_cta) / total_units);
    while (k_lo > 0 && unit_begin(k_lo, n_cta, total_units) > u_lo) --k_lo;
    k_hi = min(n_cta - 1, (int)(((long long)u_hi * n_cta + total_units - 1) / total_units));
  }
  const float* rec0 = ws + (((size_t)g * entries_per_group + (size_t)i) * HP + hl) * PART_STRIDE;
  const size_t rec_step = (size_t)HP * PART_STRIDE;   // record k sits at rec0 + k * rec_step
  // pass 1: thread t looks at candidate CTA k_lo + t (the range never exceeds the block in practice; loop anyway)
  float m_mine = -INFINITY, l_mine = 0.f;
  float M = -INFINITY;
  for (int base = k_lo; base <= k_hi; base += 128) {
    const int k = base + tid;
    float mk = -INFINITY;
    if (k <= k_hi) {
      const int ub = unit_begin(k, n_cta, total_units), ue = unit_begin(k + 1, n_cta, total_units);
      if (ue > ub && ub < u_hi && ue > u_lo) { mk = rec0[k * rec_step]; l_mine = rec0[k * rec_step + 1]; m_mine = mk; }
    }
    M = fmaxf(M, mk);
  }
  M = warp_max(M);
  if (lane == 0) red_s[0][warp] = M;
  __syncthreads();
  M = fmaxf(fmaxf(red_s[0][0], red_s[0][1]), fmaxf(red_s[0][2], red_s[0][3]));
  __syncthreads();
  // weights (k_hi - k_lo < 128 whenever the grid has at most 128 CTAs per head per row; larger ranges fall
  // back to recomputing weights below)
  const int span = k_hi - k_lo + 1;
  const bool fits = span <= 128 && span <= COMBINE_MAX_PART;
  float w_mine = (m_mine == -INFINITY) ? 0.f : exp2f(m_mine - M);
  if (fits && tid < span) wgt_s[tid] = w_mine;
  float L = warp_sum(w_mine * l_mine);
  if (lane == 0) red_s[1][warp] = L;
  __syncthreads();
  L = red_s[1][0] + red_s[1][1] + red_s[1][2] + red_s[1][3];
  // pass 2: latent vector, thread = latent index
  float v = 0.f;
  if (fits) {
    int kk = 0;
    for (; kk + 8 <= span; kk += 8) {
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = wgt_s[kk + j] != 0.f ? rec0[(size_t)(k_lo + kk + j) * rec_step + 2 + tid] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v = fmaf(x[j], wgt_s[kk + j], v);
    }
    for (; kk < span; ++kk)
      if (wgt_s[kk] != 0.f) v = fmaf(rec0[(size_t)(k_lo + kk) * rec_step + 2 + tid], wgt_s[kk], v);
  } else {
    L = 0.f;
    for (int k = k_lo; k <= k_hi; ++k) {
      const int ub = unit_begin(k, n_cta, total_units), ue = unit_begin(k + 1, n_cta, total_units);
      if (!(ue > ub && ub < u_hi && ue > u_lo)) continue;
      const float mw = rec0[k * rec_step];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      v = fmaf(rec0[k * rec_step + 2 + tid], wgt, v);
      L = fmaf(rec0[k * rec_step + 1], wgt, L);
    }
  }
  lat_s[tid] = L > 0.f ? v / L : 0.f;
  if (L <= 0.f && tid == 0) set_status(p.status, DKV_ST_EMPTY_ROW);
  __syncthreads();
  // projection: warp w takes latent rows w, w+4, ...; lane covers 4 output dims; partial sums merged in smem
  const T* vup = reinterpret_cast<const T*>(p.v_up) + (size_t)g * R * D;
  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll 4
  for (int r = warp; r < R; r += 4) {
    const float lr = lat_s[r];
    const T* row = vup + (size_t)r * D + lane * 4;
    o0 = fmaf(lr, to_f32(row[0]), o0); o1 = fmaf(lr, to_f32(row[1]), o1);
    o2 = fmaf(lr, to_f32(row[2]), o2); o3 = fmaf(lr, to_f32(row[3]), o3);
  }
  red_s[warp][lane * 4 + 0] = o0; red_s[warp][lane * 4 + 1] = o1;
  red_s[warp][lane * 4 + 2] = o2; red_s[warp][lane * 4 + 3] = o3;
  __syncthreads();
  const float o = red_s[0][tid] + red_s[1][tid] + red_s[2][tid] + red_s[3][tid];
  const int b = p.batch_index ? p.batch_index[i] : i;
  T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)h * p.out_stride_h;
  op[tid] = from_f32<T>(o);
}

// ------------------------------------------------------------------ host side
static size_t smem_bytes() { return sizeof(SmemLayout) + 1024; }

bool mma_path_ok(const dkv_attn_args* a) {
  if (a->dtype != DKV_F16 && a->dtype != DKV_BF16) return false;
  if (a->head_dim != D || a->rank > 128 || a->rank < 8 || (a->rank & 7)) return false;
  if (a->len_multiple < 8 || (a->len_multiple & 7)) return false;
  if (a->arenas_per_batch != a->n_basis_groups) return false;
  if (a->n_q_heads / a->n_basis_groups > HP) return false;
  if (a->batch > MAX_BATCH || a->n_basis_groups > 65535) return false;
  if (a->k.lens_stride_s != 1 || a->v.lens_stride_s != 1) return false;
  if (a->k.offs_stride_s != 1 || a->v.offs_stride_s != 1) return false;
  if (((uintptr_t)a->k.flat & 15) || ((uintptr_t)a->v.flat & 15) || ((uintptr_t)a->k_up & 15)) return false;
  if ((a->k.flat_stride & 7) || (a->v.flat_stride & 7)) return false;
  return true;
}

static int split_grid_x(const dkv_attn_args* a) {
  const int n_sm = a->n_sm > 0 ? a->n_sm : sm_count();
  int n = n_sm / a->n_basis_groups;
  return n < 1 ? 1 : n;
}

size_t mma_split_workspace_bytes(const dkv_attn_args* a) {
  const size_t entries = (size_t)a->n_basis_groups * ((size_t)a->batch + split_grid_x(a));
  return ws_header_bytes() + entries * HP * PART_STRIDE * sizeof(float);
}

template <typename T, bool FUSED>
static int launch_mma(const dkv_attn_args* a, int n_cta) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  const float log_theta = (float)log((double)a->theta);
  const size_t smem = smem_bytes();
  dim3 grid(FUSED ? a->batch : n_cta, a->n_basis_groups);
  // metadata rows that start on 16-byte boundaries are staged with 16-byte async copies
  auto al16 = [](const dkv_side& s) {
    return (((uintptr_t)s.lens | (uintptr_t)s.offs) & 15) == 0 && (s.lens_stride_a & 3) == 0 && (s.offs_stride_a & 3) == 0;
  };
  const int meta16 = al16(a->k) && al16(a->v) ? 1 : 0;
  cudaError_t e;
  if (a->k_norm_weight) {
    auto kern = mma_decode_kernel<T, FUSED, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, NTHREADS, smem, st>>>(*a, log_theta, n_cta, meta16);
  } else {
    auto kern = mma_decode_kernel<T, FUSED, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, NTHREADS, smem, st>>>(*a, log_theta, n_cta, meta16);
  }
  DKV_REQUIRE(e == cudaSuccess, DKV_E_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}

int mma_fused(const dkv_attn_args* a) {
  if (a->batch == 0) return DKV_OK;
  return a->dtype == DKV_BF16 ? launch_mma<__nv_bfloat16, true>(a, 1) : launch_mma<__half, true>(a, 1);
}

int mma_split(const dkv_attn_args* a) {
  if (a->batch == 0) return DKV_OK;
  DKV_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= mma_split_workspace_bytes(a), DKV_E_WORKSPACE,
              "split workspace too small: need %zu bytes, got %zu", mma_split_workspace_bytes(a), a->workspace_bytes);
  DKV_REQUIRE(((uintptr_t)a->workspace & 15) == 0, DKV_E_ALIGN, "split workspace must be 16-byte aligned");
  const int n = split_grid_x(a);
  return a->dtype == DKV_BF16 ? launch_mma<__nv_bfloat16, false>(a, n) : launch_mma<__half, false>(a, n);
}

int mma_combine(const dkv_attn_args* a) {
  if (a->batch == 0) return DKV_OK;
  DKV_REQUIRE(a->workspace != nullptr, DKV_E_WORKSPACE, "combine needs the split workspace");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  dim3 grid(a->batch, a->n_q_heads);
  if (a->dtype == DKV_BF16) split_combine_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(*a);
  else split_combine_kernel<__half><<<grid, 128, 0, st>>>(*a);
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}

// ---------------------------------------------------------------- entry point that allocates nothing
// Some hosts of this library may not create device allocations at all: a serving process that has handed
// every byte of HBM to its own pool at start-up, a plugin that runs inside someone else's captured or
// real-time section, or a sandbox that forbids cudaMalloc after initialisation.  For them the split path's
// partial-result scratch lives in this fixed array, which is part of the loaded module: every GPU that
// loads the library holds these 2 MiB until the process exits.
constexpr size_t NOALLOC_SCRATCH_BYTES = 2u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a stand-in symbol, not a device address: the address is asked
// from the runtime once per device, with that device current, and kept here.
static void* g_noalloc_ptr[64];

static int noalloc_scratch(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  DKV_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, DKV_E_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    DKV_REQUIRE(e == cudaSuccess && ptr != nullptr, DKV_E_CUDA, "cudaGetSymbolAddress(scratch) failed: %s",
                cudaGetErrorString(e));
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return DKV_OK;
}

int mma_two_stage_noalloc(const dkv_attn_args* a) {
  DKV_REQUIRE(mma_path_ok(a), DKV_E_ARG,
              "dkv_two_stage_decode_noalloc: only the split tensor-core path uses scratch; the cache must have "
              "16-bit elements, per-KV-head arenas, rank <= 128 and lengths declared as multiples of 8");
  const size_t need = mma_split_workspace_bytes(a);
  DKV_REQUIRE(need <= NOALLOC_SCRATCH_BYTES, DKV_E_LIMIT,
              "dkv_two_stage_decode_noalloc: this call needs %zu bytes of scratch, the built-in array holds %zu "
              "(reduce the batch per call or use dkv_two_stage_decode with a caller workspace)",
              need, (size_t)NOALLOC_SCRATCH_BYTES);
  dkv_attn_args b = *a;
  void* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  b.workspace = scratch;
  b.workspace_bytes = NOALLOC_SCRATCH_BYTES;
  if (int rc = mma_split(&b)) return rc;
  return mma_combine(&b);
}

}  // namespace dkv
