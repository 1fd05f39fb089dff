// Tensor-core decode attention over per-KV-head ragged arenas (bf16 / fp16, D = 128, R <= 128,
// lengths multiples of 8, gap-free prefix-sum packed rows).  One kernel template serves
//   * the short-cache fused path: one CTA per (batch row, KV head), result projected in-kernel;
//   * the long-cache split path: a persistent grid that partitions each KV head's token space
//     evenly over CTAs and writes (m, l, latent accumulator) partials, merged by a combine kernel.
//
// Per CTA: one producer warp + 8 consumer warps.
//   producer : reads the token lengths of a 64-token stage, scans them into byte offsets, allocates
//              a byte range in a shared-memory ring and pulls the stage's contiguous K and V bytes
//              with two bulk async copies (cp.async.bulk, mbarrier completion).  It also rotates the
//              group's queries back by the stage's base position so consumers only apply a local
//              (0..63) rotation to K.
//   consumer : each warp owns a 16-token group of a stage:
//              K  = X[16 x r] . Bk[r x 128]      mma.sync m16n8k16, X read with ldmatrix straight from
//                                                the ragged bytes (zero chunk beyond a row's length)
//              K' = RoPE_local(K)                 fp32 in registers, pairs (j, j+64) sit in one thread
//              S^T= Q~[heads x 128] . K'^T        mma.sync, accumulator fragments reused as B operand
//              online softmax (exp2, quad shuffles), P^T reused as B operand
//              O^T[r x heads] += XV^T . P         mma.sync, XV read with ldmatrix.trans
//
// Reference math: src/dynakv/kernels/fused.py:28-142 (fused), two_stage.py:52-157,211-281 (two-stage;
// the latent-space V accumulation with one up-projection at the end is two_stage.py:261-277).
#include <math.h>

#include "dkv_common.cuh"

namespace dkv {

constexpr int D = 128;
constexpr int NCW = 11;                // consumer warps (12 warps = 3 per SM sub-partition)
constexpr int NTHREADS = (NCW + 1) * 32;
constexpr int ST_TOK = 64;             // tokens per stage
constexpr int GRP_PER_STAGE = ST_TOK / 16;  // 16-token groups, each handled by one consumer warp
constexpr int NSLOT = 8;               // stages in flight (metadata slots)
constexpr int PD = 6;                  // producer prefetch distance for lengths (stages)
constexpr int LSTG = PD + 1;
constexpr int BASIS_PITCH = 272;       // bytes per basis row in smem (256 + 16: conflict-free ldmatrix)
constexpr int Q_PITCH = 272;
constexpr int HP = 4;                  // query heads per KV head supported by this kernel
constexpr int RING_BYTES = 88 * 1024;
constexpr int MAX_BATCH = 1024;
constexpr int PART_STRIDE = 2 + 128;   // floats per (head) partial record: m, l, latent[128]
constexpr uint32_t SPIN_LIMIT = 1u << 22;

struct __align__(16) StageHdr {
  uint32_t kbase;  // shared-memory byte address of the stage's K bytes
  uint32_t vbase;
  int32_t n_tok;
  int32_t pad;
};

struct SmemLayout {
  alignas(128) unsigned char ring[RING_BYTES];
  alignas(16) unsigned char basis[128 * BASIS_PITCH];
  alignas(16) float4 trig[ST_TOK * 64 / 2];          // [t][nt ^ (t&7)][q] -> {c_j, s_j, c_j+1, s_j+1}
  alignas(16) unsigned char qrot[NSLOT][HP * Q_PITCH];
  alignas(16) unsigned long long meta[NSLOT][ST_TOK];
  alignas(16) StageHdr hdr[NSLOT];
  alignas(16) float merge[NCW][HP][PART_STRIDE];
  alignas(16) int lens_stage[LSTG][132];             // kA[32] kB[32] vA[32] vB[32] goffK goffV
  alignas(16) float knorm_w[D];
  alignas(16) unsigned char zero_chunk[16];
  alignas(8) unsigned long long full_bar[NSLOT];
  alignas(8) unsigned long long empty_bar[NSLOT];
  int prefix[MAX_BATCH + 1];
  int ring_start[NSLOT];
  int abort_flag;
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
// Bounded wait: returns false (and raises the CTA's abort flag) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
    if (mbar_test(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
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
__global__ void __launch_bounds__(NTHREADS, 1) mma_decode_kernel(dkv_attn_args p, float log_theta, int n_cta) {
  extern __shared__ unsigned char smem_raw[];
  SmemLayout& sm = *reinterpret_cast<SmemLayout*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.y;                        // KV head == basis group == arena within the batch row
  const int G = p.n_q_heads / p.n_basis_groups;    // query heads sharing this KV head (<= HP)
  const int R = p.rank;
  volatile int* abort_flag = &sm.abort_flag;

  // ---- prologue: partition table, barriers, basis, local-rotation table -------------------------
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
        mbar_init(smem_u32(&sm.full_bar[s]), 1);
        mbar_init(smem_u32(&sm.empty_bar[s]), GRP_PER_STAGE);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
  }
  if (tid < 4) reinterpret_cast<uint32_t*>(sm.zero_chunk)[tid] = 0u;
  {
    // basis rows [R][128] -> smem with padded pitch; rows >= R are zero
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.k_up) + (size_t)g * R * D);
    for (int e = tid; e < 128 * 16; e += NTHREADS) {
      const int r = e >> 4, c = e & 15;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < R) v = src[r * 16 + c];
      *reinterpret_cast<uint4*>(sm.basis + r * BASIS_PITCH + c * 16) = v;
    }
    // local rotation table for offsets t = 0..63: angle = t * exp(-(2j/D) ln theta)
    float* tr = reinterpret_cast<float*>(sm.trig);
    for (int e = tid; e < ST_TOK * 64; e += NTHREADS) {
      const int t = e >> 6, j = e & 63;
      const float f = expf(-((float)(2 * j) / (float)D) * log_theta);
      float sn, cs;
      sincosf((float)t * f, &sn, &cs);
      const int nt = j >> 3, q = (j & 7) >> 1;
      const int idx = ((t * 8 + (nt ^ (t & 7))) * 4 + q) * 4 + (j & 1) * 2;
      tr[idx] = cs;
      tr[idx + 1] = sn;
    }
    if (KNORM && tid < D) sm.knorm_w[tid] = p.k_norm_weight[tid];
  }
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

  if (warp == NCW) {
    // =========================== producer warp ===========================
    const float f_lo = expf(-((float)(2 * lane) / (float)D) * log_theta);
    const float f_hi = expf(-((float)(2 * (lane + 32)) / (float)D) * log_theta);
    float c64a, s64a, c64b, s64b;
    sincosf((float)ST_TOK * f_lo, &s64a, &c64a);
    sincosf((float)ST_TOK * f_hi, &s64b, &c64b);
    const float qscale = rsqrtf((float)D) * 1.4426950408889634f;  // softmax scale and log2(e) folded into q
    float qa0[HP], qa1[HP], qb0[HP], qb1[HP];                      // rotated q: dims lane, lane+64 | lane+32, lane+96

    // length prefetch for stage c into lens_stage[c % LSTG]
    auto prefetch = [&](int c, int row_hint) {
      if (c < n_stages) {
        const int u = u_begin + c;
        int i = row_hint;
        while (u >= sm.prefix[i + 1]) ++i;
        const int b = p.batch_index ? p.batch_index[i] : i;
        const int a = b * p.arenas_per_batch + g;
        const int s0 = (u - sm.prefix[i]) * ST_TOK;
        const int S_i = row_tokens(p, i);
        int* dst = sm.lens_stage[c % LSTG];
        const int32_t* lk = p.k.lens + (size_t)a * p.k.lens_stride_a + s0;
        const int32_t* lv = p.v.lens + (size_t)a * p.v.lens_stride_a + s0;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int t = lane + 32 * hh;
          if (s0 + t < S_i) {
            cp_async4(smem_u32(dst + t), lk + t);
            cp_async4(smem_u32(dst + 64 + t), lv + t);
          } else {
            dst[t] = 0;
            dst[64 + t] = 0;
          }
        }
        if (lane == 0) {
          cp_async4(smem_u32(dst + 128), p.k.offs + (size_t)a * p.k.offs_stride_a + s0);
          cp_async4(smem_u32(dst + 129), p.v.offs + (size_t)a * p.v.offs_stride_a + s0);
        }
      }
      cp_async_commit();
    };
    for (int c = 0; c < PD; ++c) prefetch(c, row0);

    int row = row0;
    int head = 0;         // ring allocation cursor (lane 0 owns the allocator; kept warp-uniform)
    int oldest = 0;       // oldest stage whose ring bytes are still owned by consumers
    bool wrapped = false;
    bool ok = true;
    for (int c = 0; c < n_stages && ok; ++c) {
      prefetch(c + PD, row);
      cp_async_wait<PD>();
      __syncwarp();
      const int u = u_begin + c;
      while (u >= sm.prefix[row + 1]) ++row;
      const bool row_start = (c == 0) || (u == sm.prefix[row]);
      const int b = p.batch_index ? p.batch_index[row] : row;
      const int a = b * p.arenas_per_batch + g;
      const int s0 = (u - sm.prefix[row]) * ST_TOK;
      const int n_tok = min(ST_TOK, row_tokens(p, row) - s0);
      const int* ls = sm.lens_stage[c % LSTG];
      int kA = ls[lane], kB = ls[32 + lane], vA = ls[64 + lane], vB = ls[96 + lane];
      const int goffK = ls[128], goffV = ls[129];
      {
        const int bad = (kA | kB | vA | vB);
        const bool is_bad = (bad & 7) != 0 || bad < 0 || kA > R || kB > R || vA > R || vB > R;
        if (__any_sync(0xffffffffu, is_bad)) {
          if (lane == 0) set_status(p.status, DKV_ST_BAD_LENGTH);
          kA = min(max(kA, 0), R) & ~7; kB = min(max(kB, 0), R) & ~7;
          vA = min(max(vA, 0), R) & ~7; vB = min(max(vB, 0), R) & ~7;
        }
        if (((goffK | goffV) & 7) != 0 || goffK < 0 || goffV < 0) {
          // a misaligned arena offset cannot be bulk-copied: drop the stage's payload, keep going
          if (lane == 0) set_status(p.status, DKV_ST_BAD_LENGTH);
          kA = kB = vA = vB = 0;
        }
      }
      // exclusive scans (tokens 0..31 on the A registers, 32..63 on the B registers)
      int ik = kA, iv = vA, jk = kB, jv = vB;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t0 = __shfl_up_sync(0xffffffffu, ik, o), t1 = __shfl_up_sync(0xffffffffu, iv, o);
        const int t2 = __shfl_up_sync(0xffffffffu, jk, o), t3 = __shfl_up_sync(0xffffffffu, jv, o);
        if (lane >= o) { ik += t0; iv += t1; jk += t2; jv += t3; }
      }
      const int totKA = __shfl_sync(0xffffffffu, ik, 31), totVA = __shfl_sync(0xffffffffu, iv, 31);
      const int totK = totKA + __shfl_sync(0xffffffffu, jk, 31), totV = totVA + __shfl_sync(0xffffffffu, jv, 31);
      const int offKA = ik - kA, offKB = totKA + jk - kB, offVA = iv - vA, offVB = totVA + jv - vB;  // elements
      if ((int64_t)goffK + totK > p.k.flat_stride || (int64_t)goffV + totV > p.v.flat_stride) {
        if (lane == 0) set_status(p.status, DKV_ST_OVERFLOW);   // metadata points past the arena row
        *abort_flag = 1;
        ok = false;
        break;
      }
      const int bytesK = totK * 2, bytesV = totV * 2, need = bytesK + bytesV;

      // ---- slot + ring space (allocator state is identical on all lanes) ----
      const int slot = c % NSLOT;
      auto release_oldest = [&]() -> bool {
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
      while (ok && oldest <= c - NSLOT) ok = release_oldest();
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
        ok = release_oldest();
      }
      if (!ok) break;
      head = start + need;
      __syncwarp();
      if (lane == 0) sm.ring_start[slot] = start;

      // ---- stage metadata ----
      {
        const unsigned long long mA = (unsigned long long)(offKA >> 3) | ((unsigned long long)(offVA >> 3) << 16) |
                                      ((unsigned long long)kA << 32) | ((unsigned long long)vA << 40);
        const unsigned long long mB = (unsigned long long)(offKB >> 3) | ((unsigned long long)(offVB >> 3) << 16) |
                                      ((unsigned long long)kB << 32) | ((unsigned long long)vB << 40);
        sm.meta[slot][lane] = mA;
        sm.meta[slot][32 + lane] = mB;
        if (lane == 0) {
          StageHdr h;
          h.kbase = smem_u32(sm.ring + start);
          h.vbase = smem_u32(sm.ring + start + bytesK);
          h.n_tok = n_tok;
          h.pad = 0;
          sm.hdr[slot] = h;
        }
      }
      // ---- queries rotated back by the stage base position ----
      if (row_start) {
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
          qa0[h] = x0 * c64a + x1 * s64a; qa1[h] = x1 * c64a - x0 * s64a;
          qb0[h] = y0 * c64b + y1 * s64b; qb1[h] = y1 * c64b - y0 * s64b;
        }
      }
#pragma unroll
      for (int h = 0; h < HP; ++h) {
        T* qd = reinterpret_cast<T*>(sm.qrot[slot] + h * Q_PITCH);
        qd[lane] = from_f32<T>(qa0[h]); qd[lane + 64] = from_f32<T>(qa1[h]);
        qd[lane + 32] = from_f32<T>(qb0[h]); qd[lane + 96] = from_f32<T>(qb1[h]);
      }
      __syncwarp();
      if (lane == 0) {
        const uint32_t bar = smem_u32(&sm.full_bar[slot]);
        mbar_arrive_expect_tx(bar, (uint32_t)need);
        const T* kf = reinterpret_cast<const T*>(p.k.flat) + (size_t)a * p.k.flat_stride + goffK;
        const T* vf = reinterpret_cast<const T*>(p.v.flat) + (size_t)a * p.v.flat_stride + goffV;
        if (bytesK > 0) bulk_g2s(smem_u32(sm.ring + start), kf, (uint32_t)bytesK, bar);
        if (bytesV > 0) bulk_g2s(smem_u32(sm.ring + start + bytesK), vf, (uint32_t)bytesV, bar);
      }
    }
    cp_async_wait<0>();
    if (!ok && lane == 0) set_status(p.status, DKV_ST_OVERFLOW);
    return;
  }

  // ============================= consumer warps =============================
  // 16-token groups are dealt round-robin to the consumer warps: this warp handles groups warp, warp+NCW, ...
  // of the CTA's stage sequence (group index = stage * 4 + position in stage)
  const int gq = lane >> 2, qq = lane & 3;
  const uint32_t zero_addr = smem_u32(sm.zero_chunk);
  const uint32_t basis_lane = smem_u32(sm.basis) + ((lane & 7) + 8 * ((lane >> 3) & 1)) * BASIS_PITCH + (lane >> 4) * 16;
  const float4* trig4 = sm.trig;

  int row = row0;
  int grp = warp;             // next group of this warp
  while (row < p.batch && sm.prefix[row] < u_end) {
    const int c_hi = min(sm.prefix[row + 1], u_end) - u_begin;   // stages of this row: [.., c_hi)
    float m_run = -INFINITY, l_part = 0.f;
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }

    for (; grp < c_hi * GRP_PER_STAGE; grp += NCW) {
      const int c = grp / GRP_PER_STAGE, gi = grp % GRP_PER_STAGE;
      const int slot = c % NSLOT;
      if (*abort_flag) continue;
      if (!mbar_wait(smem_u32(&sm.full_bar[slot]), (uint32_t)((c / NSLOT) & 1), abort_flag)) continue;
      const StageHdr hdr = sm.hdr[slot];
      const int tl = lane & 15;
      unsigned long long meta = 0ull;
      if (gi * 16 < hdr.n_tok) meta = sm.meta[slot][gi * 16 + tl];
      const int klen = (int)((meta >> 32) & 0xff), vlen = (int)((meta >> 40) & 0xff);
      const uint32_t koff = (uint32_t)(meta & 0xffff), voff = (uint32_t)((meta >> 16) & 0xffff);
      const uint32_t valid = __ballot_sync(0xffffffffu, klen > 0) & 0xffffu;
      if (valid != 0u) {
        const int kmax = __reduce_max_sync(0xffffffffu, klen);
        const int vmax = __reduce_max_sync(0xffffffffu, vlen);
        // ---------------- K = X . Bk ----------------
        float acc[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
        const uint32_t krow = hdr.kbase + koff * 16u;
        const int cpar16 = lane >> 4;
        uint32_t a[4];
        ldsm_x4(a, (cpar16 * 8 < klen) ? krow + cpar16 * 16 : zero_addr);
        for (int ks = 0; ks * 16 < kmax; ++ks) {
          // next k-step's coefficient fragment while the tensor pipe works on this one
          uint32_t an[4] = {0u, 0u, 0u, 0u};
          if ((ks + 1) * 16 < kmax) {
            const int chunk = 2 * (ks + 1) + cpar16;
            ldsm_x4(an, (chunk * 8 < klen) ? krow + chunk * 16 : zero_addr);
          }
          // basis fragments are fetched four ldmatrix at a time, ahead of the eight MMAs that use them
          const uint32_t brow = basis_lane + ks * 16 * BASIS_PITCH;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t bb[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) ldsm_x4_t_const(bb[j], brow + (half * 4 + j) * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int ntp = half * 4 + j;
              Mma<T>::run(acc[2 * ntp], a[0], a[1], a[2], a[3], bb[j][0], bb[j][1]);
              Mma<T>::run(acc[2 * ntp + 1], a[0], a[1], a[2], a[3], bb[j][2], bb[j][3]);
            }
          }
          a[0] = an[0]; a[1] = an[1]; a[2] = an[2]; a[3] = an[3];
        }
        // ---------------- optional RMSNorm of K (Qwen3) ----------------
        float rs0 = 1.f, rs1 = 1.f;
        if (KNORM) {
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            s0 = fmaf(acc[i][0], acc[i][0], fmaf(acc[i][1], acc[i][1], s0));
            s1 = fmaf(acc[i][2], acc[i][2], fmaf(acc[i][3], acc[i][3], s1));
          }
          s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
          s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
          rs0 = rsqrtf(s0 * (1.0f / D) + p.k_norm_eps);
          rs1 = rsqrtf(s1 * (1.0f / D) + p.k_norm_eps);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 w = *reinterpret_cast<const float2*>(&sm.knorm_w[8 * i + 2 * qq]);
            acc[i][0] *= w.x * rs0; acc[i][1] *= w.y * rs0;
            acc[i][2] *= w.x * rs1; acc[i][3] *= w.y * rs1;
          }
        }
        // ---------------- local RoPE, pack to 16-bit B fragments ----------------
        uint32_t kb[16][2];
        {
          const int tA = gi * 16 + gq, tB = tA + 8;
#pragma unroll
          for (int nt = 0; nt < 8; ++nt) {
            const float4 ta = trig4[(tA * 8 + (nt ^ (tA & 7))) * 4 + qq];
            const float4 tb = trig4[(tB * 8 + (nt ^ (tB & 7))) * 4 + qq];
            const float lo0 = acc[nt][0], lo1 = acc[nt][1], hi0 = acc[nt + 8][0], hi1 = acc[nt + 8][1];
            kb[nt][0] = Mma<T>::pack(lo0 * ta.x - hi0 * ta.y, lo1 * ta.z - hi1 * ta.w);
            kb[nt + 8][0] = Mma<T>::pack(hi0 * ta.x + lo0 * ta.y, hi1 * ta.z + lo1 * ta.w);
            const float lo2 = acc[nt][2], lo3 = acc[nt][3], hi2 = acc[nt + 8][2], hi3 = acc[nt + 8][3];
            kb[nt][1] = Mma<T>::pack(lo2 * tb.x - hi2 * tb.y, lo3 * tb.z - hi3 * tb.w);
            kb[nt + 8][1] = Mma<T>::pack(hi2 * tb.x + lo2 * tb.y, hi3 * tb.z + lo3 * tb.w);
          }
        }
        // ---------------- S^T[heads x tokens] = Q~ . K'^T ----------------
        float s_lo[4] = {0.f, 0.f, 0.f, 0.f}, s_hi[4] = {0.f, 0.f, 0.f, 0.f};  // tokens 0-7 / 8-15
        {
          // ldmatrix rows 0..3 = heads, rows 4..7 read the zero chunk
          const uint32_t qbase = smem_u32(sm.qrot[slot]);
          const int qr = lane & 7;
          const uint32_t qaddr = (qr < HP) ? qbase + qr * Q_PITCH + (lane >> 3) * 16 : zero_addr;
          uint32_t qa[4][4];
#pragma unroll
          for (int kp = 0; kp < 4; ++kp)   // {kd=2kp: d 0-7, d 8-15 ; kd=2kp+1: d 0-7, d 8-15}
            ldsm_x4(qa[kp], (qr < HP) ? qaddr + kp * 64 : zero_addr);
#pragma unroll
          for (int kp = 0; kp < 4; ++kp) {
            Mma<T>::run(s_lo, qa[kp][0], 0u, qa[kp][1], 0u, kb[4 * kp][0], kb[4 * kp + 1][0]);
            Mma<T>::run(s_hi, qa[kp][0], 0u, qa[kp][1], 0u, kb[4 * kp][1], kb[4 * kp + 1][1]);
            Mma<T>::run(s_lo, qa[kp][2], 0u, qa[kp][3], 0u, kb[4 * kp + 2][0], kb[4 * kp + 3][0]);
            Mma<T>::run(s_hi, qa[kp][2], 0u, qa[kp][3], 0u, kb[4 * kp + 2][1], kb[4 * kp + 3][1]);
          }
        }
        // ---------------- online softmax (base 2) ----------------
        float sc0 = s_lo[0], sc1 = s_lo[1], sc2 = s_hi[0], sc3 = s_hi[1];   // tokens 2q, 2q+1, 8+2q, 9+2q
        if (KNORM) {
          // scores scale with 1/rms of their token: fetch it from the lane that owns the token row
          // (already folded into acc above, nothing to do)
        }
        if (!((valid >> (2 * qq)) & 1u)) sc0 = -INFINITY;
        if (!((valid >> (2 * qq + 1)) & 1u)) sc1 = -INFINITY;
        if (!((valid >> (8 + 2 * qq)) & 1u)) sc2 = -INFINITY;
        if (!((valid >> (9 + 2 * qq)) & 1u)) sc3 = -INFINITY;
        float mx = fmaxf(fmaxf(sc0, sc1), fmaxf(sc2, sc3));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float alpha = exp2f(m_run - m_new);
        const float p0 = exp2f(sc0 - m_new), p1 = exp2f(sc1 - m_new), p2 = exp2f(sc2 - m_new), p3 = exp2f(sc3 - m_new);
        l_part = l_part * alpha + (p0 + p1) + (p2 + p3);
        m_run = m_new;
        const uint32_t pb0 = Mma<T>::pack(p0, p1), pb1 = Mma<T>::pack(p2, p3);
        const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * qq), al1 = __shfl_sync(0xffffffffu, alpha, 8 * qq + 4);
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { oacc[i][0] *= al0; oacc[i][1] *= al1; oacc[i][2] *= al0; oacc[i][3] *= al1; }
        }
        // ---------------- O^T[r x heads] += XV^T . P ----------------
        {
          const int tv = (lane & 7) + 8 * (lane >> 4);
          const uint32_t voff_t = __shfl_sync(0xffffffffu, voff, tv);
          const int vlen_t = __shfl_sync(0xffffffffu, vlen, tv);
          const uint32_t vrow = hdr.vbase + voff_t * 16u;
          const int cpar = (lane >> 3) & 1;
          uint32_t va[8][4];
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            if (mt * 16 < vmax) {
              const int chunk = 2 * mt + cpar;
              ldsm_x4_t(va[mt], (chunk * 8 < vlen_t) ? vrow + chunk * 16 : zero_addr);
            }
          }
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            if (mt * 16 < vmax) Mma<T>::run(oacc[mt], va[mt][0], va[mt][1], va[mt][2], va[mt][3], pb0, pb1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.empty_bar[slot]));
    }

    // ---------------- row flush: merge the consumer warps' partial states ----------------
    l_part += __shfl_xor_sync(0xffffffffu, l_part, 1);
    l_part += __shfl_xor_sync(0xffffffffu, l_part, 2);
    if (gq < HP && qq == 0) { sm.merge[warp][gq][0] = m_run; sm.merge[warp][gq][1] = l_part; }
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
  if (*abort_flag && tid == 0) set_status(p.status, DKV_ST_OVERFLOW);
}

// Merge the split partials of one (batch row, query head) and project through Bv.
template <typename T>
__global__ void __launch_bounds__(128) split_combine_kernel(dkv_attn_args p) {
  __shared__ float lat_s[128];
  const WsHeader* wh = reinterpret_cast<const WsHeader*>(p.workspace);
  const float* ws = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(p.workspace) + ws_header_bytes());
  const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int G = p.n_q_heads / p.n_basis_groups, g = h / G, hl = h - g * G, R = p.rank;
  const int n_cta = wh->n_cta, total_units = wh->total_units;
  const int u_lo = wh->prefix[i], u_hi = wh->prefix[i + 1];
  const size_t entries_per_group = (size_t)p.batch + n_cta;
  // CTA k of this KV head covered units [unit_begin(k), unit_begin(k+1)); those that overlap this row's
  // units [u_lo, u_hi) each left one partial record at entry (row + k).
  auto overlaps = [&](int k) {
    const int ub = unit_begin(k, n_cta, total_units), ue = unit_begin(k + 1, n_cta, total_units);
    return ue > ub && ub < u_hi && ue > u_lo;
  };
  int k_lo = 0, k_hi = -1;
  if (u_hi > u_lo && total_units > 0) {
    // first CTA whose range ends after u_lo, last CTA whose range starts before u_hi
    k_lo = (int)(((long long)u_lo * n_cta) / total_units);
    while (k_lo > 0 && unit_begin(k_lo, n_cta, total_units) > u_lo) --k_lo;
    k_hi = min(n_cta - 1, (int)(((long long)u_hi * n_cta + total_units - 1) / total_units));
  }
  float M = -INFINITY;
  for (int k = k_lo; k <= k_hi; ++k) {
    if (!overlaps(k)) continue;
    const float* rec = ws + (((size_t)g * entries_per_group + (size_t)i + k) * HP + hl) * PART_STRIDE;
    M = fmaxf(M, rec[0]);
  }
  float v = 0.f, L = 0.f;
  for (int k = k_lo; k <= k_hi; ++k) {
    if (!overlaps(k)) continue;
    const float* rec = ws + (((size_t)g * entries_per_group + (size_t)i + k) * HP + hl) * PART_STRIDE;
    const float mw = rec[0];
    const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
    v = fmaf(rec[2 + tid], wgt, v);
    L = fmaf(rec[1], wgt, L);
  }
  lat_s[tid] = L > 0.f ? v / L : 0.f;
  if (L <= 0.f && tid == 0) set_status(p.status, DKV_ST_EMPTY_ROW);
  __syncthreads();
  const T* vup = reinterpret_cast<const T*>(p.v_up) + (size_t)g * R * D;
  float o = 0.f;
  for (int r = 0; r < R; ++r) o = fmaf(lat_s[r], to_f32(vup[(size_t)r * D + tid]), o);
  const int b = p.batch_index ? p.batch_index[i] : i;
  T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)h * p.out_stride_h;
  op[tid] = from_f32<T>(o);
}

// ------------------------------------------------------------------ host side
static size_t smem_bytes() { return sizeof(SmemLayout) + 128; }

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
    if (e == cudaSuccess) kern<<<grid, NTHREADS, smem, st>>>(*a, log_theta, n_cta);
  } else {
    auto kern = mma_decode_kernel<T, FUSED, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, NTHREADS, smem, st>>>(*a, log_theta, n_cta);
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

}  // namespace dkv
