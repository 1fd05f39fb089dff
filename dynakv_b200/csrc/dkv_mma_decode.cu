// Tensor-core decode attention over per-KV-head ragged arenas (bf16 / fp16, D = 128, R <= 128,
// lengths multiples of 8, gap-free prefix-sum packed rows).  One kernel template serves
//   * the short-cache fused path: one CTA per (batch row, KV head), result projected in-kernel;
//   * the long-cache split path: a persistent grid that partitions each KV head's token space
//     evenly over CTAs and writes (m, l, latent accumulator) partials, merged by a combine kernel.
//
// A CTA works on 128-token tiles; all three matrix products of a tile run on the 5th-generation tensor
// core (tcgen05.mma, accumulators in tensor memory), and a token row of the tile belongs to one thread
// (tensor-memory lane = token), so neither RoPE nor the softmax weights need a shuffle.  The tile pipeline:
//   4+4 gather warps : copy each token's ragged K / V coefficient row (16-byte cp.async, zero fill past the
//                      row's length) into K-major, unswizzled 128 x 128 operand tiles in shared memory; the
//                      copy engine itself signals the tile's barrier when a lane's copies have landed;
//   2 MMA threads    : per tile  (1) K = X . Bk          M=128 tokens, N=128, K=128 (A, B from shared memory)
//                                (2) S = K' . Q~^T       M=128 tokens, N=16,  K=128 (A = K' in tensor memory)
//                                (3) O^T += XV^T . P     M=128 latent, N=16,  K=128 tokens (accumulates per row);
//                      one thread issues (1) and (2) from an event loop over barrier probes, another issues (3);
//                      completion of each product is signalled by tcgen05.commit on mbarriers;
//   1 rotator warp   : Q~ = scale . R(-s0) q for the tile's base position s0 (the B operand of (2)), so K is
//                      rotated only by the in-tile offset 0..127;
//   4 RoPE warps     : a thread reads its token's K row from one of three accumulator buffers (tcgen05.ld.32x32b),
//                      applies [RMSNorm and] RoPE in fp32 with its 64 (cos, sin) pairs, which also live in tensor
//                      memory (fp16 pairs; they depend on the lane only), and writes K' back in place as packed
//                      16-bit pairs (tcgen05.st) for product (2);
//   4 softmax warps  : a thread reads its token's four scores, takes p = exp2(s - m_ref) against a reference
//                      maximum shared by the four warps, which is only raised (with a rescale of O in tensor
//                      memory) when a tile exceeds it by more than 2^8, and stores P for product (3); these
//                      warps follow the batch rows and write each row's partial (split) or projected (fused)
//                      result.
//
// Reference math: src/dynakv/kernels/fused.py:28-142 (fused), two_stage.py:52-157,211-281 (two-stage;
// the latent-space V accumulation with one up-projection at the end is two_stage.py:261-277).
#include <math.h>

#include <type_traits>

#include "dkv_common.cuh"

namespace dkv {

constexpr int D = 128;
constexpr int NGROUP = 2;              // score tiles / P tiles in flight (tile parity)
constexpr int NCW = 8;                 // warps 0-3: RoPE stage, warps 4-7: softmax stage
// Service warps.  Warp w runs on SM sub-partition w % 4, next to RoPE warp w % 4 and softmax warp 4 + w % 4; the roles are
// placed so that the sub-partitions of the two issuer threads do not also hold the (large) gather code: the
// instruction caches are small and the issuers' instruction stream is the serial part of the pipeline.
constexpr int W_KG0 = 8;               // K gather warps 8, 12 (32 tokens of the tile each; two more below)
constexpr int W_VG0 = 9;               // V gather warps 9, 13
constexpr int W_MMA = 10;              // tcgen05.mma issuer for products (1), (2); owns the tensor-memory allocation
constexpr int W_ROT = 14;              // query rotator
constexpr int W_MMA2 = 11;             // tcgen05.mma issuer for product (3)
constexpr int W_G2 = 16;               // gather warps 16, 17 (K) and 18, 19 (V): the second half of each side's four
constexpr int W_ROPE2 = 20;            // RoPE warps 20-23: the second half of each token's pairs (sub-partition w % 4 again)
constexpr int NTHREADS = 24 * 32;      // at most 85 registers per thread
constexpr int ST_TOK = 128;            // tokens per tile = rows of one UMMA
constexpr int NBUF_A = 3;              // K operand tiles in shared memory (on the critical ring: three in flight)
constexpr int NBUF_T = 3;              // K accumulator buffers in tensor memory (held from product (1) to product (2))
constexpr int NBUF_V = 2;              // V operand tiles
constexpr int NQ = 2;                  // rotated-query tiles
constexpr int PD = 2;                  // prefetch distance of the gather warps' metadata (tiles)
constexpr int MSLOT = PD + 1;          // metadata staging slots (private to the lane that fetched them)
constexpr int KV_RING = 8;             // tiles of token-validity masks kept
// 1/rms ring: a RoPE write for tile c only implies that the softmax warps have finished tile c-5 (product (1) of c
// needs product (2) of c-3 issued, which needs the P tile of c-5), so tiles c-4 .. c may be unread
constexpr int RS_RING = 5;
static_assert(RS_RING >= 5, "1/rms ring must cover the RoPE warps' lead over the softmax warps");
constexpr int TILE_BYTES = ST_TOK * 128 * 2;   // 128 tokens x 128 coefficients, chunk-major
constexpr int Q_LBO = 272;             // byte distance of the 8-dim chunks of the rotated-query tile (bank spread)
constexpr int Q_TILE_BYTES = 16 * Q_LBO;
constexpr int HP = 4;                  // query heads per KV head supported by this kernel
constexpr int MAX_BATCH = 1024;
constexpr int PART_STRIDE = 2 + 128;   // floats per (head) partial record: m, l, latent[128]
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr float M_SLACK = 8.f;         // a tile may exceed the reference maximum by 2^8 before O is rescaled
// tensor-memory columns (32-bit cells): three K accumulators, the RoPE table (fp16 pairs), two score tiles, one O
// accumulator
constexpr uint32_t TM_K = 0, TM_TRIG = 384, TM_S = 448, TM_O = 480, TMEM_COLS = 512;

struct SmemLayout {
  alignas(1024) unsigned char a_tile[NBUF_A][TILE_BYTES];   // chunk c (8 coefficients) of token t at c*2048 + t*16
  alignas(1024) unsigned char v_tile[NBUF_V][TILE_BYTES];   // same layout; [NBUF_V-1] stages the RoPE table in the prologue
  alignas(1024) unsigned char basis[128 * 256];             // Bk[r][d] at (r/8)*2048 + (d/8)*128 + (r%8)*16 + (d%8)*2
  alignas(128) unsigned char qrot[NQ][Q_TILE_BYTES];        // Q~[n][d] at (d/8)*272 + (n/8)*128 + (n%8)*16 + (d%8)*2
  alignas(128) unsigned char p_tile[NGROUP][ST_TOK * 16];   // P[t][n < 8] at t*16
  alignas(16) int meta[2][MSLOT][2][ST_TOK];                // [K|V][slot][lens|offs][token]
  alignas(16) float lat[HP][128];                           // fused path: normalised latent result of a row
  alignas(16) float tmax[2][4][4];                          // [tile parity][warp][head]
  alignas(16) float lsum[4][4];                             // [warp][head]
  alignas(16) float rs_buf[RS_RING][2][ST_TOK];             // K-RMSNorm: sum of squares of each half of the tokens' K rows, last tiles
  alignas(16) float knorm_w[D];
  uint32_t kvalid[KV_RING][4];                              // bit l of word w: token 32w + l of the tile has a K row
  alignas(8) unsigned long long a_full[NBUF_A];    // K operand tile written (128 gather lanes)
  alignas(8) unsigned long long v_full[NBUF_V];    // V operand tile written (128 gather lanes)
  alignas(8) unsigned long long v_free[NBUF_V];    // product (3) done with it (commit)
  alignas(8) unsigned long long q_full[NQ];        // rotated queries written (rotator)
  alignas(8) unsigned long long t_ready[NBUF_T];   // K accumulator written (commit)
  alignas(8) unsigned long long kp_ready[NBUF_T];  // K' written back to tensor memory (8 RoPE warps)
  alignas(8) unsigned long long s_ready[NGROUP];   // scores written (commit)
  alignas(8) unsigned long long p_ready[NGROUP];   // P tile written (4 token warps)
  alignas(8) unsigned long long pv_done[NGROUP];   // product (3) done: O updated, P tile free (commit)
  alignas(8) unsigned long long grp_sync;          // per-tile rendezvous of the 4 softmax warps (tile maxima)
  int prefix[MAX_BATCH + 1];
  int abort_flag;
  uint32_t tmem_base;
};
static_assert(sizeof(SmemLayout) <= 227 * 1024, "shared memory budget");
static_assert(ST_TOK * 65 * 4 <= NBUF_V * TILE_BYTES, "RoPE staging table must fit in the V tiles");

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
// Every lane tests the barrier itself (one instruction for the warp), so each has its own acquire: with a single
// polling lane the other lanes' later shared-memory loads are not ordered behind the wait and can be scheduled
// ahead of it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
    if (mbar_test(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// Non-blocking probe of a barrier phase.
__device__ __forceinline__ bool mbar_probe(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same for a single thread (the tensor-core issuers run on one lane).
__device__ __forceinline__ bool mbar_wait_thread(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
    if (mbar_test(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
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
// tcgen05 (5th generation tensor core) helpers ---------------------------------------------------------
// Shared-memory matrix descriptors are unswizzled: start address, leading and stride byte offsets in 16-byte
// units, descriptor version 1.
// tcgen05.mma with the shared-memory operand descriptors passed as two 32-bit words (low = (address >> 4) |
// (LBO >> 4) << 16, high = (SBO >> 4) | version bit 46): the issuer threads keep the words of each ring slot ready
// and add the (compile-time) k-step offset to the low word, so that nothing but that add stands between two
// tcgen05.mma of a product.  Building the 64-bit descriptor with shifts, masks and ors per step (~15 dependent
// instructions on a lone thread) was what an issue block waited on.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo) { return ((addr >> 4) & 0x3FFFu) | (((lbo >> 4) & 0x3FFFu) << 16); }
__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo) { return ((sbo >> 4) & 0x3FFFu) | (1u << 14); }
__device__ __forceinline__ void umma_f16_w(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\nsetp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}"
      ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (16-bit pairs packed in 32-bit cells, lane = row)
__device__ __forceinline__ void umma_f16_ta_w(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n.reg .b64 db;\n.reg .pred p;\nmov.b64 db, {%2, %3};\nsetp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Thread-per-lane tensor-memory access (32x32b shapes): thread i of the warp addresses lane (base lane + i),
// register k holds column (base column + k).  Every load carries its wait in the same statement, so no
// result register can be touched before the data has landed.
// One RoPE chunk: 8 K values of dims j0..j0+7, their rotation partners (dims +64) and the 8 table cells (fp16 pairs).
__device__ __forceinline__ void tmem_ld_rope_chunk(float (&lo)[8], float (&hi)[8], uint32_t (&tg)[8], uint32_t a_lo,
                                                   uint32_t a_hi, uint32_t a_tg) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%24];\n"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%8,%9,%10,%11,%12,%13,%14,%15}, [%25];\n"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%16,%17,%18,%19,%20,%21,%22,%23}, [%26];\n"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(tg[0]), "=r"(tg[1]), "=r"(tg[2]), "=r"(tg[3]), "=r"(tg[4]), "=r"(tg[5]), "=r"(tg[6]), "=r"(tg[7])
      : "r"(a_lo), "r"(a_hi), "r"(a_tg)
      : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) { lo[i] = __uint_as_float(r[i]); hi[i] = __uint_as_float(r[8 + i]); }
}
__device__ __forceinline__ void tmem_ld4(float (&v)[4], uint32_t addr) {
  uint32_t r[4];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];\ntcgen05.wait::ld.sync.aligned;"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const float (&v)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                 "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
                 "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
                 "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
                 "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
               : "memory");
}

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(4 * 32) : "memory"); }   // the 4 softmax warps

// order-preserving map float -> int (and back: the map is its own inverse), for redux.sync
__device__ __forceinline__ int float_key(float f) {
  const int i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }
__device__ __forceinline__ float warp_max_redux(float v) { return key_float(__reduce_max_sync(0xffffffffu, float_key(v))); }

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

// --------------------------------------------------------------- work partition
// Token space of one KV head: batch rows back to back, each rounded up to whole 128-token tiles.
__device__ __forceinline__ int row_tokens(const dkv_attn_args& p, int i) {
  const int b = p.batch_index ? p.batch_index[i] : i;
  if (row_routed_out(p, b)) return 0;   // a row routed to the other kernel contributes no tiles
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

// per-row facts cached by the warps that walk the tile sequence
struct RowInfo { int row, arena, tokens, first_unit; };

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
  // may still be appending this step's token; only the K basis is read here)
  if (tid == 0) {
    sm.prefix[0] = 0;
    sm.abort_flag = 0;
    for (int s = 0; s < NBUF_A; ++s) mbar_init(smem_u32(&sm.a_full[s]), ST_TOK);   // one arrival per gather lane
    for (int s = 0; s < NBUF_V; ++s) { mbar_init(smem_u32(&sm.v_full[s]), ST_TOK); mbar_init(smem_u32(&sm.v_free[s]), 1); }
    for (int s = 0; s < NQ; ++s) mbar_init(smem_u32(&sm.q_full[s]), 1);
    for (int s = 0; s < NGROUP; ++s) {
      mbar_init(smem_u32(&sm.s_ready[s]), 1);
      mbar_init(smem_u32(&sm.p_ready[s]), 4);
      mbar_init(smem_u32(&sm.pv_done[s]), 1);
    }
    for (int s = 0; s < NBUF_T; ++s) { mbar_init(smem_u32(&sm.t_ready[s]), 1); mbar_init(smem_u32(&sm.kp_ready[s]), 8); }
    mbar_init(smem_u32(&sm.grp_sync), 4);
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
    if (warp == W_MMA) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                   "r"(TMEM_COLS));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // RoPE table for the in-tile offsets t = 0..127: angle = t * f_j, f_j = exp(-(2j/D) ln theta), staged as
    // 16-bit cells tr[t][4*(j/2) + (j&1)] = cos, [.. + 2] = sin (row pitch 130 cells = 65 words): per two pairs one
    // word of cosines and one of sines, kept in fp16 (2^-11 absolute, below the 16-bit rounding of K').
    // NTHREADS is a multiple of 64, so a thread keeps one j and steps t by NTHREADS/64: one exact sincos, then a
    // fixed-angle rotation per step.
    static_assert(NTHREADS % 64 == 0, "trig table fill assumes a fixed j per thread");
    constexpr int TSTEP = NTHREADS / 64;
    __half* tr = reinterpret_cast<__half*>(sm.v_tile[0]);   // spans the (contiguous) V tiles until the pipeline starts
    const int j = tid & 63;
    const float f = expf(-((float)(2 * j) / (float)D) * log_theta);
    float sn, cs, ds, dc;
    sincosf((float)(tid >> 6) * f, &sn, &cs);
    sincosf((float)TSTEP * f, &ds, &dc);
    for (int t = tid >> 6; t < ST_TOK; t += TSTEP) {
      const int idx = t * 130 + 4 * (j >> 1) + (j & 1);
      tr[idx] = __float2half_rn(cs);
      tr[idx + 2] = __float2half_rn(sn);
      const float c2 = cs * dc - sn * ds, s2 = sn * dc + cs * ds;
      cs = c2; sn = s2;
    }
    for (int e = tid; e < NQ * Q_TILE_BYTES / 4; e += NTHREADS) reinterpret_cast<uint32_t*>(sm.qrot)[e] = 0u;   // rows the rotator never writes
  }

  // ---- prologue B: partition table (cache lengths: written by the kernel before this one) ----------------
  pdl_wait();
  if (KNORM && tid >= 128 && tid < 128 + D) sm.knorm_w[tid - 128] = p.k_norm_weight[tid - 128];   // may be produced by the kernel before
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
  if (warp < 4) {
    // the table row of this thread's in-tile offset goes to its tensor-memory lane
    const float* tr = reinterpret_cast<const float*>(sm.v_tile[0]) + tid * 65;   // 64 packed words of this row
    const uint32_t dst = tmem_base + ((uint32_t)(32 * warp) << 16) + TM_TRIG;
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = tr[16 * blk + i];
      tmem_st16(dst + 16 * blk, v);
    }
    tmem_wait_st();
  }
  proxy_fence_async();     // the basis was written with ordinary stores and is read by the tensor core
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

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

  if (FUSED && n_stages <= 0 && row_routed_out(p, p.batch_index ? p.batch_index[blockIdx.x] : (int)blockIdx.x)) {
    project = false;   // this row belongs to the other kernel: nothing is written
  } else if (FUSED && n_stages <= 0) {
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
  auto enter_row = [&](RowInfo& ri, int u) {
    while (u >= sm.prefix[ri.row + 1]) ++ri.row;
    const int b = p.batch_index ? p.batch_index[ri.row] : ri.row;
    ri.arena = b * p.arenas_per_batch + g;
    ri.tokens = row_tokens(p, ri.row);
    ri.first_unit = sm.prefix[ri.row];
  };

  if (n_stages <= 0) {
    // nothing to do for this CTA (fewer tiles than CTAs, or an empty row): straight to the epilogue
  }
  else if (warp == W_ROT) {
    // =========================== query rotator warp ===========================
    // For every tile (base position s0) it publishes Q~ = scale * R(-s0) q for the group's heads as rows 0..3 of
    // the B operand of product (2), so that q~ . R(t) k = q . R(s0 + t) k with the in-tile offset t = 0..127
    // (the rotation the token threads apply).  Rows 4..15 stay zero.  Lane l owns the pairs j = 2l, 2l+1.
    const float f0 = expf(-((float)(4 * lane) / (float)D) * log_theta);
    const float f1 = expf(-((float)(4 * lane + 2) / (float)D) * log_theta);
    float cd0, sd0, cd1, sd1;     // rotation by one tile
    sincosf((float)ST_TOK * f0, &sd0, &cd0);
    sincosf((float)ST_TOK * f1, &sd1, &cd1);
    const float qscale = rsqrtf((float)D) * 1.4426950408889634f;  // softmax scale and log2(e) folded into q
    float a0[HP], b0[HP], a1[HP], b1[HP];   // (q~_j, q~_{j+64}) for j = 2l and j = 2l+1
    int row = row0;
    for (int c = 0; c < n_stages; ++c) {
      const int slot = c % NQ;
      // the slot was read by product (2) of tile c-2, whose completion is s_ready of that tile
      if (c >= NQ && !mbar_wait(smem_u32(&sm.s_ready[slot]), (uint32_t)(((c / NQ) - 1) & 1), abort_flag)) break;
      const int u = u_begin + c;
      while (u >= sm.prefix[row + 1]) ++row;
      const bool row_start = (c == 0) || (u == sm.prefix[row]);
      if (row_start) {
        const int b = p.batch_index ? p.batch_index[row] : row;
        const int s0 = (u - sm.prefix[row]) * ST_TOK;
        float sa, ca, sb, cb;
        sincosf((float)s0 * f0, &sa, &ca);
        sincosf((float)s0 * f1, &sb, &cb);
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          float x0 = 0.f, x1 = 0.f, y0 = 0.f, y1 = 0.f;
          if (h < G) {
            const T* qp = reinterpret_cast<const T*>(p.q) + (size_t)b * p.q_stride_b + (size_t)(g * G + h) * p.q_stride_h;
            x0 = to_f32(qp[2 * lane]) * qscale; x1 = to_f32(qp[2 * lane + 64]) * qscale;
            y0 = to_f32(qp[2 * lane + 1]) * qscale; y1 = to_f32(qp[2 * lane + 65]) * qscale;
          }
          a0[h] = x0 * ca + x1 * sa; b0[h] = x1 * ca - x0 * sa;
          a1[h] = y0 * cb + y1 * sb; b1[h] = y1 * cb - y0 * sb;
        }
      } else {
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          const float x0 = a0[h], x1 = b0[h], y0 = a1[h], y1 = b1[h];
          a0[h] = x0 * cd0 + x1 * sd0; b0[h] = x1 * cd0 - x0 * sd0;
          a1[h] = y0 * cd1 + y1 * sd1; b1[h] = y1 * cd1 - y0 * sd1;
        }
      }
      unsigned char* const w0 = sm.qrot[slot] + (lane >> 2) * Q_LBO + (lane & 3) * 4;
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        *reinterpret_cast<uint32_t*>(w0 + h * 16) = Pack<T>::two(a0[h], a1[h]);                 // dims 2l, 2l+1
        *reinterpret_cast<uint32_t*>(w0 + h * 16 + 8 * Q_LBO) = Pack<T>::two(b0[h], b1[h]);     // dims 2l+64, 2l+65
      }
      proxy_fence_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.q_full[slot]));
    }
  }

  else if (warp == W_KG0 || warp == W_KG0 + 4 || warp == W_VG0 || warp == W_VG0 + 4 || (warp >= W_G2 && warp < W_ROPE2)) {
    // =========================== gather warps ===========================
    // Four warps per side; lane l of gather warp j owns token 32j + l of every tile: it stages the token's length
    // and offset (cp.async, PD tiles ahead, slots private to the lane) and copies the coefficient row into the
    // operand tile, one 16-byte chunk per cp.async, chunk c of token t at c*2048 + t*16; chunks past the row's
    // length are zero-filled (source size 0), so the tensor core always sees a full 128 x 128 tile.
    const bool is_v = warp >= W_G2 ? warp >= W_G2 + 2 : (warp & 3) == (W_VG0 & 3);
    const int gw = warp >= W_G2 ? 2 + ((warp - W_G2) & 1) : (warp >> 2) & 1;
    const dkv_side& sd = is_v ? p.v : p.k;
    const int side = is_v ? 1 : 0;
    const int NB = is_v ? NBUF_V : NBUF_A;
    const int t = 32 * gw + lane;
    RowInfo pre{row0, 0, 0, 0}, cur{row0, 0, 0, 0};
    int pre_end = -1, cur_end = -1;
    auto prefetch_meta = [&](int c) {   // no commit: the caller groups it with the tile's data copies
      if (c < n_stages) {
        const int u = u_begin + c;
        if (u >= pre_end) { enter_row(pre, u); pre_end = sm.prefix[pre.row + 1]; }
        const int s0 = (u - pre.first_unit) * ST_TOK;
        int(*dst)[ST_TOK] = sm.meta[side][c % MSLOT];
        if (s0 + t < pre.tokens) {
          cp_async4(smem_u32(&dst[0][t]), sd.lens + (size_t)pre.arena * sd.lens_stride_a + s0 + t);
          cp_async4(smem_u32(&dst[1][t]), sd.offs + (size_t)pre.arena * sd.offs_stride_a + s0 + t);
        } else {
          dst[0][t] = 0; dst[1][t] = 0;
        }
      }
    };
    for (int c = 0; c < PD; ++c) { prefetch_meta(c); cp_async_commit(); }   // groups 0..PD-1
    for (int c = 0; c < n_stages; ++c) {
      const int buf = c % NB;
      cp_async_wait<PD - 1>();   // group c (this tile's metadata) is complete
      const int u = u_begin + c;
      if (u >= cur_end) { enter_row(cur, u); cur_end = sm.prefix[cur.row + 1]; }
      int(*mt)[ST_TOK] = sm.meta[side][c % MSLOT];
      int len = mt[0][t];
      const int off = mt[1][t];
      if (((len | off) & 7) != 0 || len < 0 || len > R || off < 0 || (int64_t)off + len > sd.flat_stride) {
        set_status(p.status, DKV_ST_BAD_LENGTH);   // breaks the layout contract: token dropped, call flagged
        len = 0;
      }
      const unsigned char* row_src = reinterpret_cast<const unsigned char*>(
          reinterpret_cast<const T*>(sd.flat) + (size_t)cur.arena * sd.flat_stride + (len > 0 ? off : 0));
      // the tensor core must be done with the tile that was in this buffer NB tiles ago
      // (K: product (1) of tile c-2 read this buffer; its completion is t_ready of that tile, ring of NBUF_T)
      if (c >= NB) {
        const uint32_t bar = is_v ? smem_u32(&sm.v_free[buf]) : smem_u32(&sm.t_ready[(c - NBUF_A) % NBUF_T]);
        const uint32_t par = is_v ? (uint32_t)(((c / NBUF_V) - 1) & 1) : (uint32_t)(((c - NBUF_A) / NBUF_T) & 1);
        if (!mbar_wait(bar, par, abort_flag)) break;
      }
      if (!is_v) {
        // written after the wait: product (1) of tile c-3 is complete, so product (2) of tile c-6 has been issued,
        // which needed the P tile of tile c-8 written -- the softmax warps are past the mask of tile c-8 (same slot)
        const uint32_t m = __ballot_sync(0xffffffffu, len > 0);
        if (lane == 0) sm.kvalid[c % KV_RING][gw] = m;
      }
      const uint32_t dst = smem_u32(is_v ? sm.v_tile[buf] : sm.a_tile[buf]) + t * 16;
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        // past the row's length the source size is 0: nothing is read from the (then meaningless) address
        cp_async16_zfill(dst + ch * 2048, row_src + ch * 16, ch * 8 < len ? 16 : 0);
      }
      // The tile is handed over by the copy engine itself: each lane's arrival on the tile's barrier fires when
      // its copies have landed, so the warp neither waits for the data nor delays the hand-over until it comes
      // round again (which would put the next tile's wait for a free buffer into the serial loop
      // buffer free -> copies -> product (1) -> buffer free).  The consumer issues the proxy fence.
      cp_async_arrive_when_landed(smem_u32(is_v ? &sm.v_full[buf] : &sm.a_full[buf]));
      prefetch_meta(c + PD);
      cp_async_commit();                       // group PD + c
    }
    cp_async_wait<0>();
  }

  else if (warp == W_MMA) {
    // =========================== tensor-core issuer A: products (1) and (2) ===========================
    // One lane issues both products.  It never blocks on one barrier: it probes whether the next product (1) or
    // (2) has its operands in place and issues what is ready, so that one group's RoPE pass does not hold back
    // the other group's products.  The tensor core executes one thread's instructions in issue order, which also
    // orders the re-use of the accumulator buffers: product (1) of tile i+3 is only issued after product (2) of
    // tile i, which reads K' from the same buffer.  This thread is the serial part of the pipeline, so its code
    // is kept short: fully unrolled issue loops over constant descriptors, probes issued back to back.
    if (lane == 0) {
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;   // 0 = f16, 1 = bf16
      const uint32_t idesc_k = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
      // descriptor words: low = (address >> 4) | (LBO >> 4) << 16, high = (SBO >> 4) | version bit
      const uint32_t a_lo0 = desc_lo(smem_u32(sm.a_tile[0]), 2048), b_lo0 = desc_lo(smem_u32(sm.basis), 2048);
      const uint32_t q_lo0 = desc_lo(smem_u32(sm.qrot[0]), Q_LBO), hi_128 = desc_hi(128);
      static_assert(TILE_BYTES % 16 == 0 && Q_TILE_BYTES % 16 == 0 && (2 * Q_LBO) % 16 == 0, "descriptor steps are whole 16-byte units");
      int ri = 0, qi = 0;     // next tile of products (1), (2)
      int rt = 0, qt = 0;     // their accumulator buffers ri % 3, qi % 3 ...
      uint32_t rtp = 0, qtp = 0;   // ... and phases (ri / 3) & 1, (qi / 3) & 1
      uint32_t idle = 0;
      while (qi < n_stages) {
        static_assert(NBUF_A == NBUF_T, "the K operand tiles and the K accumulators share ring index and phase");
        const int rb = rt, qg = qi & 1;
        const bool r_ok = mbar_probe(smem_u32(&sm.a_full[rb]), rtp);
        const bool k_ok = mbar_probe(smem_u32(&sm.kp_ready[qt]), qtp);
        const bool q_ok = mbar_probe(smem_u32(&sm.q_full[qg]), (uint32_t)((qi >> 1) & 1)) &&
                          (qi < 2 || mbar_probe(smem_u32(&sm.p_ready[qg]), (uint32_t)(((qi >> 1) - 1) & 1)));   // score tile read out
        bool progress = false;
        if (ri < n_stages && ri - qi < NBUF_T && r_ok) {
          proxy_fence_async();   // the tile was written by cp.async (generic proxy), the tensor core reads it through the async proxy
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + (uint32_t)rb * (TILE_BYTES >> 4), d_k = tmem_base + TM_K + rt * 128;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            // A: K-major, 8-row core matrices 128 B apart (SBO), the two 8-coefficient chunks 2048 B apart (LBO)
            // B: MN-major, 8-column core matrices 128 B apart (SBO), the two 8-row groups 2048 B apart (LBO)
            // a k-step is 4096 B further in both tiles
            umma_f16_w(d_k, a_lo + ks * 256, hi_128, b_lo0 + ks * 256, hi_128, idesc_k, ks > 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&sm.t_ready[rt]));   // also frees the operand tile (the K gather warps wait on it too)
          ++ri;
          if (++rt == NBUF_T) { rt = 0; rtp ^= 1u; }
          progress = true;
        }
        if (qi < ri && k_ok && q_ok && !(progress && qi + 1 == ri)) {
          tc_fence_after();
          const uint32_t q_lo = q_lo0 + (uint32_t)qg * (Q_TILE_BYTES >> 4), d_s = tmem_base + TM_S + 16 * qg;
          const uint32_t kp = tmem_base + TM_K + qt * 128;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            // A: K' of the tile, dims 16ks..16ks+15 = 8 packed columns; each 32-dim quarter of the row starts its
            // 16 packed columns at the quarter's own first column (0, 32, 64, 96)
            // B: K-major, head rows 16 B apart inside a core matrix, 8-row groups 128 B (SBO), dim chunks Q_LBO apart
            umma_f16_ta_w(d_s, kp + 32 * (ks >> 1) + 8 * (ks & 1), q_lo + ks * ((2 * Q_LBO) >> 4), hi_128, idesc_s,
                          ks > 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&sm.s_ready[qg]));   // also frees the rotated queries (the rotator waits on it too)
          ++qi;
          if (++qt == NBUF_T) { qt = 0; qtp ^= 1u; }
          progress = true;
        }
        if (progress) {
          idle = 0;
        } else {
          ++idle;
          if ((idle & 1023u) == 0u && *abort_flag) break;
          if (idle >= SPIN_LIMIT) { *abort_flag = 1; break; }
        }
      }
    }
  }

  else if (warp == W_MMA2) {
    // =========================== tensor-core issuer B: product (3) ===========================
    // A thread of its own (on another SM sub-partition), so that product (3) costs issuer A no time.
    if (lane == 0) {
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t v_lo0 = desc_lo(smem_u32(sm.v_tile[0]), 128), p_lo0 = desc_lo(smem_u32(sm.p_tile[0]), 128);
      const uint32_t hi_2048 = desc_hi(2048), hi_0 = desc_hi(0), d_o = tmem_base + TM_O;
      int row_pv = row0;
      int c_row_lo = 0, c_row_hi = 0;   // tiles of the current batch row in this CTA: [c_row_lo, c_row_hi)
      for (int c = 0; c < n_stages; ++c) {
        const int grp = c & 1, vb = c % NBUF_V;
        if (c >= c_row_hi) {
          const int u = u_begin + c;
          while (u >= sm.prefix[row_pv + 1]) ++row_pv;
          c_row_lo = max(sm.prefix[row_pv], u_begin) - u_begin;
          c_row_hi = sm.prefix[row_pv + 1] - u_begin;
        }
        const bool first = c == c_row_lo;   // the first tile of a row starts a new sum
        if (!mbar_wait_thread(smem_u32(&sm.v_full[vb]), (uint32_t)((c / NBUF_V) & 1), abort_flag)) break;
        if (!mbar_wait_thread(smem_u32(&sm.p_ready[grp]), (uint32_t)((c >> 1) & 1), abort_flag)) break;
        proxy_fence_async();   // V tile written by cp.async
        tc_fence_after();
        const uint32_t v_lo = v_lo0 + (uint32_t)vb * (TILE_BYTES >> 4), p_lo = p_lo0 + (uint32_t)grp * ((ST_TOK * 16) >> 4);
        const uint32_t acc0 = first ? 0u : 1u;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // A = XV^T: MN-major, 16 tokens per step (256 B), token groups of 8 are 128 B apart (LBO), latent
          //     chunks 2048 B apart (SBO)
          // B = P:    MN-major, token groups of 8 are 128 B apart (LBO); the second group of 8 columns aliases
          //     the first (SBO 0): columns 8..15 of the result duplicate 0..7 and are never read
          umma_f16_w(d_o, v_lo + ks * 16, hi_2048, p_lo + ks * 16, hi_0, idesc_o, ks > 0 ? 1u : acc0);
        }
        umma_commit(smem_u32(&sm.pv_done[grp]));
        umma_commit(smem_u32(&sm.v_free[vb]));
      }
    }
  }

  else if (warp < 4 || warp >= W_ROPE2) {
    // ============================= RoPE warps =============================
    // Two threads per token: threads (w, lane) and (W_ROPE2 + w, lane) own token 32 w + lane of every tile, which is
    // tensor-memory lane 32 w + lane -- the lanes a warp in SM sub-partition w may access.  The first takes the
    // rotation pairs j = 0..31 (dims j and 64 + j), the second j = 32..63.  They turn the K row of product (1) into
    // K' for product (2) in place: each 32-dim quarter of the row is packed into the first 16 columns of the
    // quarter, columns its own thread has read before, so the two threads never touch each other's columns.
    // They know nothing about batch rows.
    const int w4 = warp & 3, half = warp >= W_ROPE2 ? 1 : 0;
    const int tok = 32 * w4 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * w4) << 16);
    int buf = 0;            // accumulator buffer c % 3 and its phase (c / 3) & 1
    uint32_t bpar = 0;
    for (int c = 0; c < n_stages; ++c) {
      if (!mbar_wait(smem_u32(&sm.t_ready[buf]), bpar, abort_flag)) break;
      tc_fence_after();
      const uint32_t k_addr = lane_addr + TM_K + 128 * buf;
      // ---------------- K row from tensor memory: [RMSNorm,] RoPE, K' back as packed 16-bit pairs ----------------
      float ss = 0.f;
#pragma unroll 1   // kept rolled: the warp roles of an SM sub-partition share a small instruction cache
      for (int ii = 0; ii < 4; ++ii) {
        // pairs j = 8i..8i+7: dims j (columns 8i..) and j+64 (columns 64+8i..); table cells 8i..: per two pairs
        // one word {cos_j, cos_j+1} and one word {sin_j, sin_j+1} in fp16
        const int i = 4 * half + ii;
        float lo[8], hi[8];
        uint32_t tg[8];
        tmem_ld_rope_chunk(lo, hi, tg, k_addr + 8 * i, k_addr + 64 + 8 * i, lane_addr + TM_TRIG + 8 * i);
        if (KNORM) {
          // RMSNorm of K (Qwen3): the weight is applied here, the per-token 1/rms scales the score later
          const float4 w0 = *reinterpret_cast<const float4*>(&sm.knorm_w[8 * i]);
          const float4 w1 = *reinterpret_cast<const float4*>(&sm.knorm_w[8 * i + 4]);
          const float4 w2 = *reinterpret_cast<const float4*>(&sm.knorm_w[64 + 8 * i]);
          const float4 w3 = *reinterpret_cast<const float4*>(&sm.knorm_w[64 + 8 * i + 4]);
          const float wl[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          const float wh[8] = {w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            ss = fmaf(lo[e], lo[e], fmaf(hi[e], hi[e], ss));
            lo[e] *= wl[e];
            hi[e] *= wh[e];
          }
        }
        uint32_t plo[4], phi[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float2 L = make_float2(lo[2 * m], lo[2 * m + 1]), H = make_float2(hi[2 * m], hi[2 * m + 1]);
          const float2 C = __half22float2(*reinterpret_cast<const __half2*>(&tg[2 * m]));
          const float2 S = __half22float2(*reinterpret_cast<const __half2*>(&tg[2 * m + 1]));
          const float2 u = __fmul2_rn(H, S);
          const float2 lo2 = __ffma2_rn(L, C, make_float2(-u.x, -u.y));
          const float2 hi2 = __ffma2_rn(L, S, __fmul2_rn(H, C));
          plo[m] = Pack<T>::two(lo2.x, lo2.y);
          phi[m] = Pack<T>::two(hi2.x, hi2.y);
        }
        // dims 8i..8i+7 -> packed columns 32 half + 4 ii.., dims 64+8i.. -> 64 + 32 half + 4 ii..: inside the
        // columns this thread read in this or an earlier round
        tmem_st4(k_addr + 32 * half + 4 * ii, plo[0], plo[1], plo[2], plo[3]);
        tmem_st4(k_addr + 64 + 32 * half + 4 * ii, phi[0], phi[1], phi[2], phi[3]);
      }
      if (KNORM) sm.rs_buf[c % RS_RING][half][tok] = ss;
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.kp_ready[buf]));
      if (++buf == NBUF_T) { buf = 0; bpar ^= 1u; }
    }
  }

  else if (warp < NCW) {
  // ============================= softmax warps =============================
  // Thread (wq, lane) owns token 32 wq + lane of every tile: it reads the token's scores from product (2),
  // forms the softmax weights against the reference maximum m_ref shared by the four warps, and stores P for
  // product (3).  These warps follow the batch rows and write each row's result.
  const int wq = warp & 3;
  const int tok = 32 * wq + lane;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * wq) << 16);
  const uint32_t o_addr = lane_addr + TM_O;

  int row = row0;
  while (row < p.batch && sm.prefix[row] < u_end) {
    const int c_lo = max(sm.prefix[row], u_begin) - u_begin;     // tiles of this row in this CTA: [c_lo, c_hi)
    const int c_hi = min(sm.prefix[row + 1], u_end) - u_begin;
    float m_ref[HP], l_part[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) { m_ref[h] = -INFINITY; l_part[h] = 0.f; }
    int c_last = -1;            // last tile of the row that was processed
    bool dead = false;

    for (int c = c_lo; c < c_hi; ++c) {
      if (dead || *abort_flag) { dead = true; continue; }
      const int buf = c & 1;
      const uint32_t par = (uint32_t)((c >> 1) & 1);
      const bool first = c == c_lo;     // O holds nothing of this row yet
      // ---------------- scores of this token for the group's heads ----------------
      if (!mbar_wait(smem_u32(&sm.s_ready[buf]), par, abort_flag)) { dead = true; continue; }
      tc_fence_after();
      float s[HP];
      tmem_ld4(s, lane_addr + TM_S + 16 * buf);
      if (KNORM) {
        const float rs = rsqrtf((sm.rs_buf[c % RS_RING][0][tok] + sm.rs_buf[c % RS_RING][1][tok]) * (1.0f / D) + p.k_norm_eps);
#pragma unroll
        for (int h = 0; h < HP; ++h) s[h] *= rs;
      }
      const bool valid = (sm.kvalid[c % KV_RING][wq] >> lane) & 1u;
      float mx[HP];
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        if (!valid) s[h] = -INFINITY;
        mx[h] = warp_max_redux(s[h]);
      }
      // tile maxima: the four warps meet on an mbarrier (bounded wait, unlike a named barrier)
      if (lane == 0) {
        *reinterpret_cast<float4*>(sm.tmax[buf][wq]) = make_float4(mx[0], mx[1], mx[2], mx[3]);
        mbar_arrive(smem_u32(&sm.grp_sync));
      }
      if (!mbar_wait(smem_u32(&sm.grp_sync), (uint32_t)(c & 1), abort_flag)) { dead = true; continue; }
      float factor[HP];
      bool grow = false;
      {
        const float4 t0 = *reinterpret_cast<const float4*>(sm.tmax[buf][0]);
        const float4 t1 = *reinterpret_cast<const float4*>(sm.tmax[buf][1]);
        const float4 t2 = *reinterpret_cast<const float4*>(sm.tmax[buf][2]);
        const float4 t3 = *reinterpret_cast<const float4*>(sm.tmax[buf][3]);
        const float tm[HP] = {fmaxf(fmaxf(t0.x, t1.x), fmaxf(t2.x, t3.x)), fmaxf(fmaxf(t0.y, t1.y), fmaxf(t2.y, t3.y)),
                              fmaxf(fmaxf(t0.z, t1.z), fmaxf(t2.z, t3.z)), fmaxf(fmaxf(t0.w, t1.w), fmaxf(t2.w, t3.w))};
#pragma unroll
        for (int h = 0; h < HP; ++h) {
          factor[h] = 1.f;
          if (tm[h] > m_ref[h] + M_SLACK) {   // also the first tile with a token: -inf + slack = -inf
            factor[h] = exp2f(m_ref[h] - tm[h]);   // 0 when there was no reference yet
            m_ref[h] = tm[h];
            grow = true;
          }
        }
      }
      // the P tile of this parity was read by product (3) of tile c-2
      if (c >= 2 && !mbar_wait(smem_u32(&sm.pv_done[buf]), (uint32_t)(((c >> 1) - 1) & 1), abort_flag)) { dead = true; continue; }
      if (grow) {   // uniform over the four warps: every thread sees the same maxima
#pragma unroll
        for (int h = 0; h < HP; ++h) l_part[h] *= factor[h];
        if (!first) {
          // O is rescaled in tensor memory: product (3) of tile c-1 must be complete as well
          if (!mbar_wait(smem_u32(&sm.pv_done[buf ^ 1]), (uint32_t)(((c - 1) >> 1) & 1), abort_flag)) { dead = true; continue; }
          tc_fence_after();
          float o[4];
          tmem_ld4(o, o_addr);
          tmem_st4(o_addr, __float_as_uint(o[0] * factor[0]), __float_as_uint(o[1] * factor[1]),
                   __float_as_uint(o[2] * factor[2]), __float_as_uint(o[3] * factor[3]));
          tmem_wait_st();
        }
      }
      float pr[HP];
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        pr[h] = exp2f(s[h] - (m_ref[h] == -INFINITY ? 0.f : m_ref[h]));
        l_part[h] += pr[h];
      }
      *reinterpret_cast<uint4*>(sm.p_tile[buf] + tok * 16) = make_uint4(Pack<T>::two(pr[0], pr[1]), Pack<T>::two(pr[2], pr[3]), 0u, 0u);
      proxy_fence_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.p_ready[buf]));
      c_last = c;
    }

    // ---------------- row flush ----------------
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    if (c_last >= 0 && !dead && mbar_wait(smem_u32(&sm.pv_done[c_last & 1]), (uint32_t)((c_last >> 1) & 1), abort_flag)) {
      tc_fence_after();
      tmem_ld4(o, o_addr);   // O^T[r = tok][head]
    }
#pragma unroll
    for (int h = 0; h < HP; ++h) {
      const float l = warp_sum(l_part[h]);
      if (lane == 0) sm.lsum[wq][h] = l;
    }
    consumer_bar();
    float L[HP];
#pragma unroll
    for (int h = 0; h < HP; ++h) L[h] = (sm.lsum[0][h] + sm.lsum[1][h]) + (sm.lsum[2][h] + sm.lsum[3][h]);
    if (!FUSED) {
      // partial record (row, cta) -> entry row + blockIdx.x of this KV head
      float* ws = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p.workspace) + ws_header_bytes());
      const size_t entries_per_group = (size_t)p.batch + n_cta;
      float* rec = ws + (((size_t)g * entries_per_group + (size_t)row + blockIdx.x) * HP) * PART_STRIDE;
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        rec[h * PART_STRIDE + 2 + tok] = o[h];
        if (tok == 0) { rec[h * PART_STRIDE] = m_ref[h]; rec[h * PART_STRIDE + 1] = L[h]; }
      }
      consumer_bar();   // lsum may be rewritten by the next row
    } else {
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        sm.lat[h][tok] = L[h] > 0.f ? o[h] / L[h] : 0.f;
        if (L[h] <= 0.f && tok == 0 && h < G) set_status(p.status, DKV_ST_EMPTY_ROW);
      }
      // the up-projection is done by the whole block after the pipeline has drained (a fused CTA has one row)
    }
    ++row;
  }
  }   // softmax warps

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
  if (warp == W_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
  if (*abort_flag && tid == 0) set_status(p.status, DKV_ST_TIMEOUT);
}

// Merge the split partials of one (batch row, KV head) for its query heads and project through Bv.
// 512 threads: thread (h, r) merges latent component r of head h over the row's partial records (online softmax
// merge, eight records per round with independent loads); the 32 KB of Bv are fetched into registers before
// anything else, so that their latency hides behind the merge, and are used for all heads of the group.
template <typename T>
__global__ void __launch_bounds__(512) split_combine_kernel(dkv_attn_args p) {
  __shared__ float lat_s[HP][128];
  __shared__ float red_s[16][HP][128];
  const WsHeader* wh = reinterpret_cast<const WsHeader*>(p.workspace);
  const float* ws = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(p.workspace) + ws_header_bytes());
  const int i = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = tid >> 7, r = tid & 127;
  if (row_routed_out(p, p.batch_index ? p.batch_index[i] : i)) return;   // the row belongs to the other kernel
  const int G = p.n_q_heads / p.n_basis_groups, R = p.rank;
  // Bv pieces of this thread: rows tid/16 + 32 j, columns 8 (tid % 16) .. +8
  const int c8 = tid & 15, row0 = tid >> 4;
  uint4 bv[4];
  {
    const T* vup = reinterpret_cast<const T*>(p.v_up) + (size_t)g * R * D;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = row0 + 32 * j;
      bv[j] = row < R ? __ldg(reinterpret_cast<const uint4*>(vup + (size_t)row * D) + c8) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
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
  const float* rec0 = ws + (((size_t)g * entries_per_group + (size_t)i) * HP + h) * PART_STRIDE;
  const size_t rec_step = (size_t)HP * PART_STRIDE;   // record k sits at rec0 + k * rec_step
  float M = -INFINITY, L = 0.f, v = 0.f;
  if (h < G) {
    for (int base = k_lo; base <= k_hi; base += 8) {
      float m[8], l[8], x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = base + j;
        m[j] = -INFINITY; l[j] = 0.f; x[j] = 0.f;
        if (k <= k_hi) {
          const int ub = unit_begin(k, n_cta, total_units), ue = unit_begin(k + 1, n_cta, total_units);
          if (ue > ub && ub < u_hi && ue > u_lo) {
            const float* rec = rec0 + (size_t)k * rec_step;
            m[j] = __ldcg(rec); l[j] = __ldcg(rec + 1); x[j] = __ldcg(rec + 2 + r);
          }
        }
      }
      float cm = m[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) cm = fmaxf(cm, m[j]);
      const float newM = fmaxf(M, cm);
      if (newM != -INFINITY) {
        const float keep = exp2f(M - newM);     // 0 while nothing was merged yet
        L *= keep; v *= keep;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float w = m[j] == -INFINITY ? 0.f : exp2f(m[j] - newM);
          L = fmaf(w, l[j], L);
          v = fmaf(w, x[j], v);
        }
        M = newM;
      }
    }
    if (L <= 0.f && r == 0) set_status(p.status, DKV_ST_EMPTY_ROW);
  }
  lat_s[h][r] = L > 0.f ? v / L : 0.f;
  __syncthreads();
  // projection: out[hh][8 c8 + e] += lat[hh][row] * Bv[row][8 c8 + e] over this thread's four rows
  float acc[HP][8];
#pragma unroll
  for (int hh = 0; hh < HP; ++hh)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[hh][e] = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int row = row0 + 32 * j;
    const T* bp = reinterpret_cast<const T*>(&bv[j]);
    float b[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) b[e] = to_f32(bp[e]);
#pragma unroll
    for (int hh = 0; hh < HP; ++hh) {
      const float lr = lat_s[hh][row];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[hh][e] = fmaf(lr, b[e], acc[hh][e]);
    }
  }
#pragma unroll
  for (int hh = 0; hh < HP; ++hh)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[hh][e] += __shfl_xor_sync(0xffffffffu, acc[hh][e], 16);
  if (lane < 16) {
#pragma unroll
    for (int hh = 0; hh < HP; ++hh) {
      *reinterpret_cast<float4*>(&red_s[warp][hh][8 * c8]) = make_float4(acc[hh][0], acc[hh][1], acc[hh][2], acc[hh][3]);
      *reinterpret_cast<float4*>(&red_s[warp][hh][8 * c8 + 4]) = make_float4(acc[hh][4], acc[hh][5], acc[hh][6], acc[hh][7]);
    }
  }
  __syncthreads();
  if (h < G) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < 16; ++w) o += red_s[w][h][r];
    const int b = p.batch_index ? p.batch_index[i] : i;
    T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)(g * G + h) * p.out_stride_h;
    op[r] = from_f32<T>(o);
  }
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
  dim3 grid(a->batch, a->n_basis_groups);
  // launched the ordinary way: measured, an early (programmatic) launch of the combine or of the next append
  // costs more than it hides -- their CTAs wait on the SMs the decode kernel is using
  if (a->dtype == DKV_BF16) split_combine_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(*a);
  else split_combine_kernel<__half><<<grid, 512, 0, st>>>(*a);
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
