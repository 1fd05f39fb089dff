// Tensor-core decode attention over per-KV-head ragged arenas (bf16 / fp16, D = 128, R <= 128,
// lengths multiples of 8, gap-free prefix-sum packed rows).  One kernel template serves
//   * the short-cache fused path: one CTA per (batch row, KV head), result projected in-kernel;
//   * the long-cache split path: a persistent grid that partitions each KV head's token space
//     evenly over CTAs and writes (m, l, latent accumulator) partials, merged by a combine kernel.
//
// A CTA works on 128-token tiles.  Per tile:
//   K gather (4 warps)  : each lane copies its token's ragged K coefficient row (16-byte cp.async, zero fill past
//                         the row's length) into a K-major 128 x 128 operand tile in shared memory;
//   service warp        : one lane issues the K reconstruction  K = X . Bk  (tcgen05.mma, M = 128 tokens, N = 128,
//                         K = 128, accumulator in tensor memory); the warp then publishes the rotated queries
//                         Q~ = scale . R(-s0) q for the tile's base position s0 as mma.sync A fragments, so K is
//                         rotated only by the in-tile offset 0..127;
//   V gather (4 warps)  : each lane copies its token's V coefficient row into a row-major tile (one token per
//                         272-byte row), zero-filled only up to the longest row of its 16-token group;
//   compute (8 warps)   : warp w owns tokens 16w'..16w'+15 of every tile.  It reads their K rows from tensor
//                         memory in the mma.sync fragment layout (tcgen05.ld.16x256b), applies [RMSNorm and] RoPE
//                         in fp32 registers (the cos/sin of its in-tile offsets stay in registers), and feeds K'
//                         straight into mma.sync as the B operand of  S^T = Q~ . K'^T  (no round trip through
//                         tensor or shared memory).  Online softmax is private to the warp (own running maximum,
//                         own sum); P^T is the A operand of  O += P^T . XV  (mma.sync, B via ldmatrix.trans from the
//                         V tile, only as many latent columns as the group's longest V row), with O[4 heads x 128
//                         latent] in registers.  At the end of a batch row the eight warps merge their partials.
// The compute warps raise their register allowance (setmaxnreg) from what the gather and service warps release.
//
// Reference math: src/dynakv/kernels/fused.py:28-142 (fused), two_stage.py:52-157,211-281 (two-stage;
// the latent-space V accumulation with one up-projection at the end is two_stage.py:261-277).
#include <math.h>

#include <type_traits>

#include "dkv_common.cuh"

namespace dkv {

constexpr int D = 128;
constexpr int N_CW = 8;                // compute warps 0..7 (warpgroups 0 and 1)
constexpr int W_KG0 = 8;               // K gather warps 8..11 (warpgroup 2)
constexpr int W_VG0 = 12;              // V gather warps 12..15 (warpgroup 3)
constexpr int NTHREADS = 16 * 32;
constexpr int REGS_COMPUTE = 200;      // per-thread register allowances after the roles split (setmaxnreg):
constexpr int REGS_OTHER = 56;         // 8 x 32 x 200 + 8 x 32 x 56 = 64 K registers
constexpr int ST_TOK = 128;            // tokens per tile = rows of one UMMA
constexpr int NRING = 3;               // K operand tiles = K accumulators = rotated-query slots (one ring)
constexpr int NBUF_V = 2;              // V tiles
constexpr int PD = 2;                  // prefetch distance of the gather warps' metadata (tiles)
constexpr int MSLOT = PD + 1;          // metadata staging slots (private to the lane that fetched them)
// Token-validity masks: the K gather writes tile c's mask after product (1) of tile c - NRING has completed, which
// needs the accumulator of tile c - 2 NRING released, i.e. every compute warp has started (not finished) tile
// c - 2 NRING.  So masks of tiles c - 2 NRING .. c are live at once.
constexpr int KV_RING = 8;
static_assert(KV_RING > 2 * NRING, "validity-mask ring must cover the K gather's lead over the compute warps");
constexpr int TILE_BYTES = ST_TOK * 128 * 2;   // K operand tile: 128 tokens x 128 coefficients, chunk-major
constexpr int V_PITCH = 272;                   // bytes between token rows of a V tile (256 + 16: ldmatrix bank spread)
constexpr int V_TILE_BYTES = ST_TOK * V_PITCH;
constexpr int HP = 4;                  // query heads per KV head supported by this kernel
constexpr int MAX_BATCH = 1024;
constexpr int PART_STRIDE = 2 + 128;   // floats per (head) partial record: m, l, latent[128]
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr float M_SLACK = 8.f;         // a tile may exceed a warp's running maximum by 2^8 before O is rescaled
constexpr uint32_t TMEM_COLS = 512;    // three 128-column K accumulators (allocation sizes are powers of two)

struct SmemLayout {
  alignas(1024) unsigned char a_tile[NRING][TILE_BYTES];    // chunk c (8 coefficients) of token t at c*2048 + t*16
  alignas(1024) unsigned char basis[128 * 256];             // Bk[r][d] at (r/8)*2048 + (d/8)*128 + (r%8)*16 + (d%8)*2
  alignas(128) unsigned char v_tile[NBUF_V][V_TILE_BYTES];  // latent chunk c of token t at t*272 + c*16
  alignas(16) uint32_t qfrag[NRING][4][32][4];              // [slot][i][lane]{a0a1(ks=i), a4a5(ks=i), a0a1(ks=4+i), a4a5(ks=4+i)}
  alignas(16) float part_o[N_CW / 2][HP][128];              // row end: latent accumulators of a warp pair (w, w + 4)
  alignas(16) float part_m[N_CW / 2][HP];
  alignas(16) float part_l[N_CW / 2][HP];
  alignas(16) int meta[2][MSLOT][2][ST_TOK];                // [K|V][slot][lens|offs][token]
  alignas(16) float lat[HP][128];                           // fused path: normalised latent result of a row
  alignas(16) float knorm_w[D];
  uint32_t kvalid[KV_RING][4];                              // bit l of word w: token 32w + l of the tile has a K row
  int vfill[NBUF_V][8];                                     // 16-latent column pairs filled for each 16-token group
  alignas(8) unsigned long long a_full[NRING];     // K operand tile written (128 copy arrivals + 4 warp arrivals)
  alignas(8) unsigned long long t_ready[NRING];    // K accumulator written, operand tile free (commit)
  alignas(8) unsigned long long acc_free[NRING];   // accumulator and rotated-query slot read out (8 compute warps)
  alignas(8) unsigned long long q_full[NRING];     // rotated queries written (4 V gather warps, one head each)
  alignas(8) unsigned long long v_full[NBUF_V];    // V tile written (128 copy arrivals + 4 warp arrivals)
  alignas(8) unsigned long long v_free[NBUF_V];    // V tile read (8 compute warps)
  alignas(8) unsigned long long row_sync;          // row-end rendezvous of the 8 compute warps
  int prefix[MAX_BATCH + 1];
  int abort_flag;
  uint32_t tmem_base;
};
static_assert(sizeof(SmemLayout) <= 227 * 1024, "shared memory budget");
static_assert(ST_TOK * 64 * 8 <= NRING * TILE_BYTES, "RoPE staging table must fit in the K operand tiles");

#ifdef DKV_TRACE
// Debug builds only: per-role clock stamps of the first tiles of CTA (0, 0).
constexpr int TR_TILES = 96, TR_ROLES = 6, TR_PTS = 6;
__device__ long long g_trace[TR_ROLES][TR_TILES][TR_PTS];
__device__ unsigned int g_qdbg[2][64][32][4];
__device__ float g_pdbg[64][9][4][2];   // [cta][warp 0..7 | 8 = merged][head]{m, l}
#define PDBG(w, h, m, l) do { const int cta__ = blockIdx.y * gridDim.x + blockIdx.x; if (cta__ < 64) { g_pdbg[cta__][w][h][0] = (m); g_pdbg[cta__][w][h][1] = (l); } } while (0)
#define QDBG(which, c, h, val) do { const int cta__ = blockIdx.y * gridDim.x + blockIdx.x; if (cta__ < 64 && (c) < 32) g_qdbg[which][cta__][c][h] = (val); } while (0)
#define TRACE(role, c, pt) do { if (blockIdx.x == 1 && blockIdx.y == 0 && (c) < TR_TILES && (threadIdx.x & 31) == 0) g_trace[role][c][pt] = clock64(); } while (0)
#else
#define TRACE(role, c, pt) do { } while (0)
#define QDBG(which, c, h, val) do { } while (0)
#define PDBG(w, h, m, l) do { } while (0)
#endif

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(bar) : "memory");
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
// shared-memory barrier unit.  Once it has seen the phase complete, every lane tests the barrier once itself:
// the acquire of lane 0 orders nothing for the other lanes, and without one of their own their later
// shared-memory loads may be scheduled ahead of the wait.
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
  if (ok) (void)mbar_test(bar, parity);
  __syncwarp();
  return ok != 0;
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// The barrier receives one arrival from this thread once all of its earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive_when_landed(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void set_max_regs_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void set_max_regs_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
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

// Tensor-memory load in the mma.sync accumulator layout (16 lanes x 256 bits, twice = 16 columns): thread
// (g = lane / 4, t = lane % 4) receives, for each 8-column block k = 0, 1,
//   r[4k + 0], r[4k + 1] = lane (base + g),     columns 8k + 2t, 8k + 2t + 1
//   r[4k + 2], r[4k + 3] = lane (base + g + 8), columns 8k + 2t, 8k + 2t + 1.
// Two such loads (a 16-column block and its rotation partners 64 columns up) and the wait share one statement,
// so no result register can be touched before the data has landed.
__device__ __forceinline__ void tmem_ld_frag2(float (&lo)[8], float (&hi)[8], uint32_t a_lo, uint32_t a_hi) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%16];\n"
      "tcgen05.ld.sync.aligned.16x256b.x2.b32 {%8,%9,%10,%11,%12,%13,%14,%15}, [%17];\n"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(a_lo), "r"(a_hi)
      : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) { lo[i] = __uint_as_float(r[i]); hi[i] = __uint_as_float(r[8 + i]); }
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
struct Pack;
template <>
struct Pack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t two(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <>
struct Pack<__half> {
  static __device__ __forceinline__ uint32_t two(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// mma.sync m16n8k16 with fp32 accumulation.  Only rows 0..7 of A are ever non-zero here (rows = query heads,
// four of them real), so a1 = a3 = 0 and the accumulator rows 8..15 (d2, d3) are discarded.
template <typename T>
__device__ __forceinline__ void mma_rows8(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  float x2, x3;
  if (std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                 : "+f"(d0), "+f"(d1), "=f"(x2), "=f"(x3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                 : "+f"(d0), "+f"(d1), "=f"(x2), "=f"(x3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
  }
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}

// --------------------------------------------------------------- work partition
// Token space of one KV head: batch rows back to back, each rounded up to whole 128-token tiles.
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

// RoPE of four (dim j, dim j + 64) pairs of two tokens, then the score products that consume them.
//   lo / hi : a 16-column block of the K accumulator (column blocks cb = 2 I, 2 I + 1 of the 16 blocks of 8) and
//             its partners 64 columns up, in the tcgen05.ld.16x256b layout above
//   ct / st : cos and sin of (token offset) * f_j for this thread's two tokens and its 16 pairs
// K' goes straight into mma.sync B fragments: the k-step of dims 16 I .. 16 I + 15 takes block 2 I (b0) and
// 2 I + 1 (b1), and the partners form k-step 4 + I.  sa / sb accumulate the low / high half of the dot product
// for token block e (0: lanes g, 1: lanes g + 8).
template <typename T, bool KNORM, int I>
__device__ __forceinline__ void rope_scores(const float (&lo)[8], const float (&hi)[8], const float2 (&ct)[2][8],
                                            const float2 (&st)[2][8], const uint32_t* qf_lane, const float* knorm_w,
                                            int t, float (&ss)[2], float (&sa)[2][2], float (&sb)[2][2]) {
  uint32_t blo[2][2], bhi[2][2];       // [token block e][b0 | b1]
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int cb = 2 * I + k;
    float2 wl = make_float2(1.f, 1.f), wh = make_float2(1.f, 1.f);
    if (KNORM) {
      wl = *reinterpret_cast<const float2*>(knorm_w + 8 * cb + 2 * t);
      wh = *reinterpret_cast<const float2*>(knorm_w + 64 + 8 * cb + 2 * t);
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float2 L = make_float2(lo[4 * k + 2 * e], lo[4 * k + 2 * e + 1]);
      float2 H = make_float2(hi[4 * k + 2 * e], hi[4 * k + 2 * e + 1]);
      if (KNORM) {
        ss[e] = fmaf(L.x, L.x, fmaf(L.y, L.y, fmaf(H.x, H.x, fmaf(H.y, H.y, ss[e]))));
        L = __fmul2_rn(L, wl);
        H = __fmul2_rn(H, wh);
      }
      const float2 C = ct[e][cb], S = st[e][cb];
      const float2 nH = make_float2(-H.x, -H.y);
      const float2 lo2 = __ffma2_rn(nH, S, __fmul2_rn(L, C));
      const float2 hi2 = __ffma2_rn(L, S, __fmul2_rn(H, C));
      blo[e][k] = Pack<T>::two(lo2.x, lo2.y);
      bhi[e][k] = Pack<T>::two(hi2.x, hi2.y);
    }
  }
  const uint4 qa = *reinterpret_cast<const uint4*>(qf_lane + I * 32 * 4);
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    mma_rows8<T>(sa[e][0], sa[e][1], qa.x, qa.y, blo[e][0], blo[e][1]);
    mma_rows8<T>(sb[e][0], sb[e][1], qa.z, qa.w, bhi[e][0], bhi[e][1]);
  }
}

// ------------------------------------------------------------------ the kernel
template <typename T, bool FUSED, bool KNORM>
__global__ void __launch_bounds__(NTHREADS, 1) mma_decode_kernel(dkv_attn_args p, float log_theta, int n_cta) {
  // The dynamic shared memory is used from its (aligned) start, so that every shared-memory address -- and with
  // it every operand descriptor the tensor-core issuer builds -- is a link-time constant, not a run-time value.
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  SmemLayout& sm = *reinterpret_cast<SmemLayout*>(smem_raw);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.y;                        // KV head == basis group == arena within the batch row
  const int G = p.n_q_heads / p.n_basis_groups;    // query heads sharing this KV head (<= HP)
  const int R = p.rank;
  volatile int* abort_flag = &sm.abort_flag;

  // ---- prologue A: everything that does not depend on the kernel before this one -----------------------
  // (programmatic dependent launch: this part overlaps the tail of the preceding kernel in the stream, which
  // may still be appending this step's token; only the bases and the K-norm weight are read here)
  if (tid == 0) {
    sm.prefix[0] = 0;
    sm.abort_flag = 0;
    for (int s = 0; s < NRING; ++s) {
      mbar_init(smem_u32(&sm.a_full[s]), ST_TOK + 4);   // one arrival per gather lane's copies + one per gather warp
      mbar_init(smem_u32(&sm.t_ready[s]), 1);
      mbar_init(smem_u32(&sm.acc_free[s]), N_CW);
      mbar_init(smem_u32(&sm.q_full[s]), 4);
    }
    for (int s = 0; s < NBUF_V; ++s) { mbar_init(smem_u32(&sm.v_full[s]), ST_TOK + 4); mbar_init(smem_u32(&sm.v_free[s]), N_CW); }
    mbar_init(smem_u32(&sm.row_sync), N_CW);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
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
    if (warp == W_KG0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                   "r"(TMEM_COLS));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // RoPE table for the in-tile offsets t = 0..127: angle = t * f_j, f_j = exp(-(2j/D) ln theta), staged in the
    // (not yet used) K operand tiles as fp32 cos[t][j] and, 32 KB further, sin[t][j].  NTHREADS is a multiple of
    // 64, so a thread keeps one j and steps t by NTHREADS/64: one exact sincos, then a fixed-angle rotation per step.
    static_assert(NTHREADS % 64 == 0, "trig table fill assumes a fixed j per thread");
    constexpr int TSTEP = NTHREADS / 64;
    float* tc = reinterpret_cast<float*>(sm.a_tile[0]);
    float* ts = tc + ST_TOK * 64;
    const int j = tid & 63;
    const float f = expf(-((float)(2 * j) / (float)D) * log_theta);
    float sn, cs, ds, dc;
    sincosf((float)(tid >> 6) * f, &sn, &cs);
    sincosf((float)TSTEP * f, &ds, &dc);
    for (int t = tid >> 6; t < ST_TOK; t += TSTEP) {
      tc[t * 64 + j] = cs;
      ts[t * 64 + j] = sn;
      const float c2 = cs * dc - sn * ds, s2 = sn * dc + cs * ds;
      cs = c2; sn = s2;
    }
    if (KNORM && tid < D) sm.knorm_w[tid] = p.k_norm_weight[tid];
    for (int e = tid; e < NRING * 4 * 32 * 4; e += NTHREADS) (&sm.qfrag[0][0][0][0])[e] = 0u;   // rows no V warp ever writes
  }

  // ---- prologue B: partition table (cache lengths: written by the kernel before this one) ----------------
  pdl_wait();
  if (warp == 0) {
    // inclusive scan of the per-row tile counts, 32 rows at a time
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
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  const int cq = warp & 3, chf = (warp >> 2) & 1;          // tensor-memory lane quarter / 16-lane half of a compute warp
  const int fg = lane >> 2, ft = lane & 3;                 // mma.sync fragment coordinates
  const int tok0 = 32 * cq + 16 * chf;                     // first of a compute warp's 16 tokens in every tile

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
  bool project = FUSED;   // fused path: the block projects its row at the end

  if (FUSED && n_stages <= 0) {
    // row without tokens: zeros, flagged
    for (int e = tid; e < G * D; e += NTHREADS) {
      const int b = p.batch_index ? p.batch_index[blockIdx.x] : blockIdx.x;
      T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)(g * G + e / D) * p.out_stride_h;
      op[e % D] = from_f32<T>(0.f);
    }
    if (tid == 0) set_status(p.status, DKV_ST_EMPTY_ROW);
    project = false;
  }

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
  // ---- the roles split; registers move from the gather / service warpgroups to the compute warpgroups ----
  // (each side finishes the set-up inside its own branch, so that nothing the compute warps keep in their
  // enlarged register file is live in code the other warps share)
  if (warp < N_CW) {
    float2 ct[2][8], st[2][8];
    set_max_regs_inc<REGS_COMPUTE>();
    // cos / sin of this thread's two in-tile token offsets (tensor-memory lanes tok0 + g and tok0 + g + 8) times
    // its sixteen frequencies j = 8 cb + 2 t, + 1 (cb = 0..7), kept in registers for the whole kernel
    const float* tc = reinterpret_cast<const float*>(sm.a_tile[0]);
    const float* ts = tc + ST_TOK * 64;
#pragma unroll
    for (int e = 0; e < 2; ++e)
#pragma unroll
      for (int cb = 0; cb < 8; ++cb) {
        ct[e][cb] = *reinterpret_cast<const float2*>(tc + (tok0 + fg + 8 * e) * 64 + 8 * cb + 2 * ft);
        st[e][cb] = *reinterpret_cast<const float2*>(ts + (tok0 + fg + 8 * e) * 64 + 8 * cb + 2 * ft);
      }
    proxy_fence_async();     // every thread wrote part of the basis with ordinary stores; the tensor core reads it
    tc_fence_before();
    __syncthreads();         // the staging table has been read: the gather may now overwrite the K operand tiles
    tc_fence_after();
    if (n_stages > 0) {
    // ============================= compute warps =============================
    const uint32_t lane_addr = tmem_base + ((uint32_t)tok0 << 16);
    const uint32_t* const qf_lane = &sm.qfrag[0][0][lane][0];
    const uint32_t v_lane = smem_u32(sm.v_tile[0]) + (uint32_t)(tok0 + ((lane >> 3) & 1) * 8 + (lane & 7)) * V_PITCH + (lane >> 4) * 16;
    const int vgrp = 2 * cq + chf;               // this warp's 16-token group
    const bool head_lane = fg < HP;              // lanes 0..15 hold the four real heads' scores
    uint32_t row_phase = 0;

    int row = row0;
    bool dead = false;
    while (row < p.batch && sm.prefix[row] < u_end) {
      const int c_lo = max(sm.prefix[row], u_begin) - u_begin;     // tiles of this row in this CTA: [c_lo, c_hi)
      const int c_hi = min(sm.prefix[row + 1], u_end) - u_begin;
      float m_run = -INFINITY, l_run = 0.f;      // of head fg (lanes 0..15), over this warp's tokens
      float o[16][2];                            // O[head fg][latent 8 nb + 2 ft, + 1]
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) { o[nb][0] = 0.f; o[nb][1] = 0.f; }

      for (int c = c_lo; c < c_hi; ++c) {
        if (dead || *abort_flag) { dead = true; continue; }
        const int slot = c % NRING;
        const uint32_t par = (uint32_t)((c / NRING) & 1);
        const int vb = c % NBUF_V;
        const int trole = warp == 0 ? 0 : (warp == 5 ? 1 : -1);
        if (trole >= 0) TRACE(trole, c, 0);
        if (!mbar_wait(smem_u32(&sm.q_full[slot]), par, abort_flag)) { dead = true; continue; }
        if (!mbar_wait(smem_u32(&sm.t_ready[slot]), par, abort_flag)) { dead = true; continue; }
        tc_fence_after();
        if (trole >= 0) TRACE(trole, c, 1);
        // ---------------- K rows from tensor memory: [RMSNorm,] RoPE, scores by mma.sync ----------------
        const uint32_t k_addr = lane_addr + slot * 128;
        const uint32_t* const qf = qf_lane + slot * (4 * 32 * 4);
        if (warp == 0 && (lane & 3) == 0 && lane < 16) QDBG(1, c, lane >> 2, qf[0]);
        float ss[2] = {0.f, 0.f};
        float sa[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, sb[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
        {
          float lo[8], hi[8];
          tmem_ld_frag2(lo, hi, k_addr, k_addr + 64);
          rope_scores<T, KNORM, 0>(lo, hi, ct, st, qf, sm.knorm_w, ft, ss, sa, sb);
          tmem_ld_frag2(lo, hi, k_addr + 16, k_addr + 80);
          rope_scores<T, KNORM, 1>(lo, hi, ct, st, qf, sm.knorm_w, ft, ss, sa, sb);
          tmem_ld_frag2(lo, hi, k_addr + 32, k_addr + 96);
          rope_scores<T, KNORM, 2>(lo, hi, ct, st, qf, sm.knorm_w, ft, ss, sa, sb);
          tmem_ld_frag2(lo, hi, k_addr + 48, k_addr + 112);
          // accumulator and query slot are released once the last read of each has been issued
          tc_fence_before();
          rope_scores<T, KNORM, 3>(lo, hi, ct, st, qf, sm.knorm_w, ft, ss, sa, sb);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.acc_free[slot]));
        if (trole >= 0) TRACE(trole, c, 2);

        // ---------------- softmax weights of this warp's 16 tokens (private running maximum) ----------------
        float s[2][2];
#pragma unroll
        for (int e = 0; e < 2; ++e) { s[e][0] = sa[e][0] + sb[e][0]; s[e][1] = sa[e][1] + sb[e][1]; }
        if (KNORM) {
          // 1/rms of the tokens: ss[e] holds a quarter of the squares of token (g + 8e); the scores of this thread
          // belong to tokens 8e + 2t, 8e + 2t + 1, whose sums sit in the lanes with g = 2t, 2t + 1
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 1);
            ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 2);
            const float rs = rsqrtf(ss[e] * (1.0f / D) + p.k_norm_eps);
            s[e][0] *= __shfl_sync(0xffffffffu, rs, 8 * ft);
            s[e][1] *= __shfl_sync(0xffffffffu, rs, 8 * ft + 4);
          }
        }
        const uint32_t vbits = sm.kvalid[c % KV_RING][cq] >> (16 * chf);
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const bool valid = head_lane && ((vbits >> (8 * e + 2 * ft + x)) & 1u);
            if (!valid) s[e][x] = -INFINITY;
            mx = fmaxf(mx, s[e][x]);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const bool grow = mx > m_run + M_SLACK;        // also the first tile with a token: -inf + slack = -inf
        if (__any_sync(0xffffffffu, grow)) {
          const float factor = grow ? ex2(m_run - mx) : 1.f;   // 0 when there was no maximum yet
          if (grow) m_run = mx;
          l_run *= factor;
#pragma unroll
          for (int nb = 0; nb < 16; ++nb) { o[nb][0] *= factor; o[nb][1] *= factor; }
        }
        const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
        float pr[2][2];
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            pr[e][x] = ex2(s[e][x] - m_use);
            l_run += pr[e][x];
          }
        const uint32_t pa0 = Pack<T>::two(pr[0][0], pr[0][1]);   // tokens 2t, 2t+1      (k = 2t, 2t+1)
        const uint32_t pa2 = Pack<T>::two(pr[1][0], pr[1][1]);   // tokens 8+2t, 8+2t+1  (k = 2t+8, 2t+9)

        // ---------------- O += P^T . XV over the group's filled latent columns ----------------
        if (trole >= 0) TRACE(trole, c, 3);
        if (!mbar_wait(smem_u32(&sm.v_full[vb]), (uint32_t)((c / NBUF_V) & 1), abort_flag)) { dead = true; continue; }
        if (trole >= 0) TRACE(trole, c, 4);
        const int npair = sm.vfill[vb][vgrp];
        const uint32_t v_addr = v_lane + vb * V_TILE_BYTES;
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          if (np < npair) {
            uint32_t bm[4];
            ldmatrix_x4_trans(bm, v_addr + np * 32);
            mma_rows8<T>(o[2 * np][0], o[2 * np][1], pa0, pa2, bm[0], bm[1]);
            mma_rows8<T>(o[2 * np + 1][0], o[2 * np + 1][1], pa0, pa2, bm[2], bm[3]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.v_free[vb]));
        if (trole >= 0) TRACE(trole, c, 5);
      }

      // ---------------- row end: the eight warps merge their partials ----------------
      // Warps 4..7 hand theirs to warps 0..3 (same fragment layout, so thread to thread), which merge and publish;
      // then all 256 threads merge the four pair results, two (head, latent index) values each.
      l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
      l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
      if (dead) m_run = -INFINITY;
      const int pw = warp & 3;
      if (head_lane && ft == 0) PDBG(warp, fg, m_run, l_run);
      if (warp >= 4 && head_lane) {
#pragma unroll
        for (int nb = 0; nb < 16; ++nb)
          *reinterpret_cast<float2*>(&sm.part_o[pw][fg][8 * nb + 2 * ft]) = make_float2(o[nb][0], o[nb][1]);
        if (ft == 0) { sm.part_m[pw][fg] = m_run; sm.part_l[pw][fg] = l_run; }
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.row_sync));
      if (!mbar_wait(smem_u32(&sm.row_sync), row_phase, abort_flag)) dead = true;
      row_phase ^= 1u;
      if (warp < 4 && head_lane) {
        const float pm = sm.part_m[pw][fg], pl = sm.part_l[pw][fg];
        const float M = fmaxf(m_run, pm);
        const float f1 = (m_run == -INFINITY) ? 0.f : ex2(m_run - M);
        const float f2 = (pm == -INFINITY) ? 0.f : ex2(pm - M);
#pragma unroll
        for (int nb = 0; nb < 16; ++nb) {
          float2* cell = reinterpret_cast<float2*>(&sm.part_o[pw][fg][8 * nb + 2 * ft]);
          const float2 po = *cell;
          *cell = make_float2(fmaf(o[nb][0], f1, po.x * f2), fmaf(o[nb][1], f1, po.y * f2));
        }
        if (ft == 0) { sm.part_m[pw][fg] = M; sm.part_l[pw][fg] = fmaf(l_run, f1, pl * f2); }
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.row_sync));
      if (!mbar_wait(smem_u32(&sm.row_sync), row_phase, abort_flag)) dead = true;
      row_phase ^= 1u;
      {
        float* rec = nullptr;
        if (!FUSED) {
          // partial record (row, cta) -> entry row + blockIdx.x of this KV head
          float* ws = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p.workspace) + ws_header_bytes());
          const size_t entries_per_group = (size_t)p.batch + n_cta;
          rec = ws + (((size_t)g * entries_per_group + (size_t)row + blockIdx.x) * HP) * PART_STRIDE;
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int e = tid + 256 * k, h = e >> 7, r = e & 127;
          float M = -INFINITY;
#pragma unroll
          for (int w = 0; w < N_CW / 2; ++w) M = fmaxf(M, sm.part_m[w][h]);
          float acc = 0.f, L = 0.f;
#pragma unroll
          for (int w = 0; w < N_CW / 2; ++w) {
            const float mw = sm.part_m[w][h];
            const float wt = (mw == -INFINITY) ? 0.f : ex2(mw - M);
            acc = fmaf(sm.part_o[w][h][r], wt, acc);
            L = fmaf(sm.part_l[w][h], wt, L);
          }
          if (!FUSED) {
            rec[h * PART_STRIDE + 2 + r] = acc;
            if (r == 0) { rec[h * PART_STRIDE] = M; rec[h * PART_STRIDE + 1] = L; }
          } else {
            if (r == 0) PDBG(8, h, M, L);
            sm.lat[h][r] = L > 0.f ? acc / L : 0.f;
            if (L <= 0.f && r == 0 && h < G) set_status(p.status, DKV_ST_EMPTY_ROW);
            // the up-projection is done by the whole block after the pipeline has drained (a fused CTA has one row)
          }
        }
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.row_sync));     // the partial buffers may be rewritten after this
      if (!mbar_wait(smem_u32(&sm.row_sync), row_phase, abort_flag)) dead = true;
      row_phase ^= 1u;
      ++row;
    }
    }   // compute warps
  } else {
    set_max_regs_dec<REGS_OTHER>();
    proxy_fence_async();     // the basis was written with ordinary stores and is read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (n_stages <= 0) {
      // nothing to do for this CTA (fewer tiles than CTAs, or an empty row): straight to the epilogue
    } else {
      // =========================== gather warps ===========================
      // Lane l of gather warp j owns token 32j + l of every tile: it stages the token's length and offset (cp.async,
      // PD tiles ahead, slots private to the lane) and copies the coefficient row, one 16-byte chunk per cp.async.
      //   K: chunk c of token t at c*2048 + t*16 (the tensor core's K-major operand layout); chunks past the row's
      //      length are zero-filled (source size 0), so the tensor core always sees a full 128 x 128 tile.
      //      The first K warp also issues the K reconstruction of the tile before (one lane, tcgen05.mma).
      //   V: chunk c of token t at t*272 + c*16; zero-filled only up to the longest row of the token's 16-token
      //      group, rounded to 16 latent columns -- the compute warp that owns the group reads no further.
      //      V warp h also publishes the tile's rotated query of head h.
      const bool is_v = warp >= W_VG0;
      const int gw = (warp - W_KG0) & 3;
      const dkv_side& sd = is_v ? p.v : p.k;
      const int side = is_v ? 1 : 0;
      const int t = 32 * gw + lane;
      // the batch row a tile belongs to, tracked separately for the metadata prefetch (PD tiles ahead) and the copies
      int pre_row = row0, pre_end = -1, pre_first = 0, pre_tokens = 0, pre_arena = 0;
      int cur_row = row0, cur_end = -1, cur_arena = 0;
      auto prefetch_meta = [&](int c) {   // no commit: the caller groups it with the tile's data copies
        if (c < n_stages) {
          const int u = u_begin + c;
          if (u >= pre_end) {
            while (u >= sm.prefix[pre_row + 1]) ++pre_row;
            pre_arena = (p.batch_index ? p.batch_index[pre_row] : pre_row) * p.arenas_per_batch + g;
            pre_tokens = row_tokens(p, pre_row);
            pre_first = sm.prefix[pre_row];
            pre_end = sm.prefix[pre_row + 1];
          }
          const int s0 = (u - pre_first) * ST_TOK;
          int(*dst)[ST_TOK] = sm.meta[side][c % MSLOT];
          if (s0 + t < pre_tokens) {
            cp_async4(smem_u32(&dst[0][t]), sd.lens + (size_t)pre_arena * sd.lens_stride_a + s0 + t);
            cp_async4(smem_u32(&dst[1][t]), sd.offs + (size_t)pre_arena * sd.offs_stride_a + s0 + t);
          } else {
            dst[0][t] = 0; dst[1][t] = 0;
          }
        }
      };
      // this tile's row of the token: validated length and source address
      auto token_row = [&](int c, int& len) -> const unsigned char* {
        const int u = u_begin + c;
        if (u >= cur_end) {
          while (u >= sm.prefix[cur_row + 1]) ++cur_row;
          cur_arena = (p.batch_index ? p.batch_index[cur_row] : cur_row) * p.arenas_per_batch + g;
          cur_end = sm.prefix[cur_row + 1];
        }
        int(*mt)[ST_TOK] = sm.meta[side][c % MSLOT];
        len = mt[0][t];
        const int off = mt[1][t];
        if (((len | off) & 7) != 0 || len < 0 || len > R || off < 0 || (int64_t)off + len > sd.flat_stride) {
          set_status(p.status, DKV_ST_BAD_LENGTH);   // breaks the layout contract: token dropped, call flagged
          len = 0;
        }
        return reinterpret_cast<const unsigned char*>(reinterpret_cast<const T*>(sd.flat) + (size_t)cur_arena * sd.flat_stride +
                                                      (len > 0 ? off : 0));
      };
      for (int c = 0; c < PD; ++c) { prefetch_meta(c); cp_async_commit(); }   // groups 0..PD-1

      if (!is_v) {
        // ---------------------------------- K side ----------------------------------
        const bool issuer = warp == W_KG0;
        const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;   // 0 = f16, 1 = bf16
        const uint32_t idesc_k = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
        // product (1) of tile j: K = X . Bk into accumulator j % NRING, once the operand tile has landed and the
        // compute warps have read the accumulator's previous contents (tile j - NRING)
        auto issue = [&](int j) -> bool {
          const int slot = j % NRING;
          const uint32_t par = (uint32_t)((j / NRING) & 1);
          TRACE(2, j, 0);
          if (j >= NRING && !mbar_wait(smem_u32(&sm.acc_free[slot]), par ^ 1u, abort_flag)) return false;
          TRACE(2, j, 1);
          if (!mbar_wait(smem_u32(&sm.a_full[slot]), par, abort_flag)) return false;
          TRACE(2, j, 2);
          if (lane == 0) {
            proxy_fence_async();   // the tile was written by cp.async (generic proxy), the tensor core reads it through the async proxy
            tc_fence_after();
            const uint32_t a_addr = smem_u32(sm.a_tile[0]) + slot * TILE_BYTES;
            const uint32_t basis_addr = smem_u32(sm.basis);
            const uint32_t d_addr = tmem_base + slot * 128;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              // A: K-major, 8-row core matrices 128 B apart (SBO), the two 8-coefficient chunks 2048 B apart (LBO)
              // B: MN-major, 8-column core matrices 128 B apart (SBO), the two 8-row groups 2048 B apart (LBO)
              umma_f16(d_addr, umma_desc(a_addr + ks * 4096, 2048, 128), umma_desc(basis_addr + ks * 4096, 2048, 128),
                       idesc_k, ks > 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&sm.t_ready[slot]));   // also frees the operand tile (the K gather warps wait on it)
          }
          __syncwarp();
          TRACE(2, j, 3);
          return true;
        };
        bool ok = true;
        for (int c = 0; c < n_stages && ok; ++c) {
          const int buf = c % NRING;
          if (issuer) TRACE(3, c, 0);
          cp_async_wait<PD - 1>();   // group c (this tile's metadata) is complete
          int len;
          const unsigned char* row_src = token_row(c, len);
          // product (1) of tile c - NRING must be done with this buffer: its completion is t_ready
          if (c >= NRING && !mbar_wait(smem_u32(&sm.t_ready[buf]), (uint32_t)(((c / NRING) - 1) & 1), abort_flag)) break;
          if (issuer) TRACE(3, c, 1);
          const uint32_t m = __ballot_sync(0xffffffffu, len > 0);
          if (lane == 0) sm.kvalid[c % KV_RING][gw] = m;
          const uint32_t dst = smem_u32(sm.a_tile[buf]) + t * 16;
#pragma unroll
          for (int ch = 0; ch < 16; ++ch) {
            // past the row's length the source size is 0: nothing is read from the (then meaningless) address
            cp_async16_zfill(dst + ch * 2048, row_src + ch * 16, ch * 8 < len ? 16 : 0);
          }
          // The tile is handed over by the copy engine itself: each lane's arrival on the tile's barrier fires when
          // its copies have landed.  One ordinary arrival per warp carries the warp's plain store (validity mask).
          cp_async_arrive_when_landed(smem_u32(&sm.a_full[buf]));
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sm.a_full[buf]));
          prefetch_meta(c + PD);
          cp_async_commit();                       // group PD + c
          if (issuer) TRACE(3, c, 2);
          if (issuer && c >= 1) ok = issue(c - 1);   // one tile behind the copies, so the wait for them is short
        }
        if (issuer && ok) issue(n_stages - 1);
      } else {
        // ---------------------------------- V side ----------------------------------
        // Rotated query of head hv: Q~ = scale * R(-s0) q for the tile's base position s0, written as mma.sync A
        // fragments (row hv), so that q~ . R(t) k = q . R(s0 + t) k with the in-tile offset t = 0..127 (the rotation
        // the compute warps apply).  Lane l owns the pairs j = 2l, 2l+1.
        const int hv = gw;
        const float f0 = expf(-((float)(4 * lane) / (float)D) * log_theta);
        const float f1 = expf(-((float)(4 * lane + 2) / (float)D) * log_theta);
        float cd0, sd0, cd1, sd1;     // rotation by one tile
        sincosf((float)ST_TOK * f0, &sd0, &cd0);
        sincosf((float)ST_TOK * f1, &sd1, &cd1);
        const float qscale = rsqrtf((float)D) * 1.4426950408889634f;  // softmax scale and log2(e) folded into q
        float a0 = 0.f, b0 = 0.f, a1 = 0.f, b1 = 0.f;   // (q~_j, q~_{j+64}) for j = 2l and j = 2l+1
        // fragment cell of this lane's dims (2l, 2l+1): k-step pair i = l / 8, register a0a1 or a4a5, thread 4 hv + l % 4
        uint32_t* const qf_w = &sm.qfrag[0][lane >> 3][4 * hv + (lane & 3)][(lane & 7) >> 2];
        int qrow = row0;
        for (int c = 0; c < n_stages; ++c) {
          const int buf = c % NBUF_V, slot = c % NRING;
          if (warp == W_VG0) TRACE(4, c, 0);
          // ---- rotated query (slot last read by the compute warps in tile c - NRING) ----
          if (c >= NRING && !mbar_wait(smem_u32(&sm.acc_free[slot]), (uint32_t)(((c / NRING) - 1) & 1), abort_flag)) break;
          {
            const int u = u_begin + c;
            while (u >= sm.prefix[qrow + 1]) ++qrow;
            if (c == 0 || u == sm.prefix[qrow]) {
              const int b = p.batch_index ? p.batch_index[qrow] : qrow;
              const int s0 = (u - sm.prefix[qrow]) * ST_TOK;
              float sa, ca, sb, cb;
              sincosf((float)s0 * f0, &sa, &ca);
              sincosf((float)s0 * f1, &sb, &cb);
              float x0 = 0.f, x1 = 0.f, y0 = 0.f, y1 = 0.f;
              if (hv < G) {
                const T* qp = reinterpret_cast<const T*>(p.q) + (size_t)b * p.q_stride_b + (size_t)(g * G + hv) * p.q_stride_h;
                x0 = to_f32(qp[2 * lane]) * qscale; x1 = to_f32(qp[2 * lane + 64]) * qscale;
                y0 = to_f32(qp[2 * lane + 1]) * qscale; y1 = to_f32(qp[2 * lane + 65]) * qscale;
              }
              a0 = x0 * ca + x1 * sa; b0 = x1 * ca - x0 * sa;
              a1 = y0 * cb + y1 * sb; b1 = y1 * cb - y0 * sb;
            } else {
              const float x0 = a0, x1 = b0, y0 = a1, y1 = b1;
              a0 = x0 * cd0 + x1 * sd0; b0 = x1 * cd0 - x0 * sd0;
              a1 = y0 * cd1 + y1 * sd1; b1 = y1 * cd1 - y0 * sd1;
            }
            uint32_t* const w0 = qf_w + slot * (4 * 32 * 4);
            w0[0] = Pack<T>::two(a0, a1);          // dims 2l, 2l+1     -> k-step i
            if (lane == 0) QDBG(0, c, hv, Pack<T>::two(a0, a1));
            w0[2] = Pack<T>::two(b0, b1);          // dims 2l+64, 2l+65 -> k-step 4 + i
            __threadfence_block();   // every lane's stores must be performed before lane 0 announces them
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.q_full[slot]));
          }
          if (warp == W_VG0) TRACE(4, c, 1);
          // ---- V rows ----
          cp_async_wait<PD - 1>();   // group c (this tile's metadata) is complete
          int len;
          const unsigned char* row_src = token_row(c, len);
          // the 8 compute warps must be done with the tile that was in this buffer NBUF_V tiles ago
          if (c >= NBUF_V && !mbar_wait(smem_u32(&sm.v_free[buf]), (uint32_t)(((c / NBUF_V) - 1) & 1), abort_flag)) break;
          if (warp == W_VG0) TRACE(4, c, 2);
          int gmax = len;   // longest row of this lane's 16-token group
#pragma unroll
          for (int o = 1; o < 16; o <<= 1) gmax = max(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
          const int npair = (gmax + 15) >> 4;                      // 16-column pairs this group needs
          const int wpair = max(npair, __shfl_xor_sync(0xffffffffu, npair, 16));
          if ((lane & 15) == 0) sm.vfill[buf][2 * gw + (lane >> 4)] = npair;
          const uint32_t dst = smem_u32(sm.v_tile[buf]) + t * V_PITCH;
#pragma unroll
          for (int ch = 0; ch < 16; ++ch) {
            if (ch < 2 * wpair) {            // warp-uniform
              if (ch < 2 * npair) cp_async16_zfill(dst + ch * 16, row_src + ch * 16, ch * 8 < len ? 16 : 0);
            }
          }
          cp_async_arrive_when_landed(smem_u32(&sm.v_full[buf]));
          __threadfence_block();   // lanes 0 and 16 stored the fill widths
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sm.v_full[buf]));   // carries the plain store of the fill width
          prefetch_meta(c + PD);
          cp_async_commit();                       // group PD + c
          if (warp == W_VG0) TRACE(4, c, 3);
        }
      }
      cp_async_wait<0>();
    }
  }

  // ---- epilogue: every warp arrives here; the tensor memory is returned by the warp that allocated it ----
  tc_fence_before();
  __syncthreads();
  if (project) {
    // out[head][d] = sum_r latent[head][r] * Bv[r][d]: one output element per thread
    const int h = tid >> 7, d = tid & 127;
    if (h < HP && h < G) {
      const int b = p.batch_index ? p.batch_index[blockIdx.x] : blockIdx.x;
      const T* vup = reinterpret_cast<const T*>(p.v_up) + (size_t)g * R * D + d;
      float acc0 = 0.f, acc1 = 0.f;
      int r = 0;
      for (; r + 1 < R; r += 2) {
        acc0 = fmaf(sm.lat[h][r], to_f32(vup[(size_t)r * D]), acc0);
        acc1 = fmaf(sm.lat[h][r + 1], to_f32(vup[(size_t)(r + 1) * D]), acc1);
      }
      if (r < R) acc0 = fmaf(sm.lat[h][r], to_f32(vup[(size_t)r * D]), acc0);
      T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)(g * G + h) * p.out_stride_h;
      op[d] = from_f32<T>(acc0 + acc1);
    }
  }
  if (warp == W_KG0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
  if (*abort_flag && tid == 0) set_status(p.status, DKV_ST_TIMEOUT);
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
static size_t smem_bytes() { return sizeof(SmemLayout); }

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
  cudaError_t e;
  if (a->k_norm_weight) {
    auto kern = mma_decode_kernel<T, FUSED, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = launch_pdl(kern, grid, dim3(NTHREADS), smem, st, *a, log_theta, n_cta);
  } else {
    auto kern = mma_decode_kernel<T, FUSED, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = launch_pdl(kern, grid, dim3(NTHREADS), smem, st, *a, log_theta, n_cta);
  }
  DKV_REQUIRE(e == cudaSuccess, DKV_E_CUDA, "launch of the decode kernel failed: %s", cudaGetErrorString(e));
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
  // launched the ordinary way: measured, an early (programmatic) launch of the combine or of the next append
  // costs more than it hides -- their CTAs wait on the SMs the decode kernel is using
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

#ifdef DKV_TRACE
extern "C" int dkv_debug_p(float* host, size_t bytes) {
  if (bytes > sizeof(dkv::g_pdbg)) bytes = sizeof(dkv::g_pdbg);
  return (int)cudaMemcpyFromSymbol(host, dkv::g_pdbg, bytes);
}
extern "C" int dkv_debug_q(unsigned int* host, size_t bytes) {
  if (bytes > sizeof(dkv::g_qdbg)) bytes = sizeof(dkv::g_qdbg);
  return (int)cudaMemcpyFromSymbol(host, dkv::g_qdbg, bytes);
}
extern "C" int dkv_debug_trace(long long* host, size_t bytes) {
  if (bytes > sizeof(dkv::g_trace)) bytes = sizeof(dkv::g_trace);
  return (int)cudaMemcpyFromSymbol(host, dkv::g_trace, bytes);
}
#endif
