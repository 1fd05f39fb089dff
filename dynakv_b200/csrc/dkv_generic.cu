// Generic (CUDA-core, fp32-accumulate) decode attention over the ragged compressed cache.
//
// Handles every layout the reference API can express: any element type, rank R up to 1024,
// any integer lengths, lens/offs as strided views, joint latent rows shared by all heads or
// per-KV-head arenas.  It is the path for fp32 inputs and for caches that do not meet the
// alignment contract of the tensor-core path, and it implements the reference's stage-1 /
// stage-2 operators (scores, softmax.V) with their exact conventions.
//
// Math (reference: src/dynakv/kernels/fused.py:28-142, two_stage.py:52-157, 211-281):
//   k_s = x^k_s . Bk[g]            (first len_s coefficients only)
//   k'_s = RoPE_s(k_s)              (pairs (j, j+D/2), angle = s * exp(-(2j/D) ln theta), fp32)
//   score_s = D^-1/2 (q . k'_s)
//   softmax over s, accumulate sum_s p_s x^v_s in latent space, project once through Bv[g].
#include <math.h>

#include <type_traits>

#include "dkv_common.cuh"

namespace dkv {

enum { MODE_ATTN = 0, MODE_SCORES = 1, MODE_SOFTMAX_V = 2, MODE_ATTN_SPLIT = 3 };
// MODE_ATTN_SPLIT: blockIdx.z takes a slice of the tokens and leaves a partial record (m, l, latent accumulator) in
// the workspace; generic_combine_kernel merges the records of a (row, head) and projects through Bv.

constexpr int GD = 128;       // head_dim
constexpr int GTT = 32;       // tokens per tile
constexpr int GRC = 64;       // latent coefficients staged per step
constexpr int GTHREADS = 256;
constexpr int GZ_TOKENS = 256;  // tokens per blockIdx.z slice in MODE_SCORES

template <typename T, int MODE>
__global__ void __launch_bounds__(GTHREADS)
generic_decode_kernel(dkv_attn_args p, const T* __restrict__ scores_in, int64_t sc_sb, int64_t sc_sh, float log_theta,
                      int split_tokens) {
  __shared__ float q_s[GD];
  __shared__ float k_s[GTT][GD + 1];
  // staging: fp32 path = x tile [GTT][GRC] floats; 16-bit path = x tile [GTT][GRC + 8] and basis chunk
  // [GRC][GD + 8] in the storage type (row pitches of 144 and 272 bytes keep ldmatrix free of bank conflicts)
  __shared__ __align__(16) unsigned char stage_raw[GTT * (GRC + 8) * 2 + GRC * (GD + 8) * 2];
  float (*x_s)[GRC] = reinterpret_cast<float (*)[GRC]>(stage_raw);
  __shared__ float sc_s[GTT], p_s[GTT];
  __shared__ int lenk_s[GTT], offk_s[GTT], lenv_s[GTT], offv_s[GTT];
  __shared__ float alpha_s, l_s;
  __shared__ int rmax_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = p.batch_index ? p.batch_index[blockIdx.x] : blockIdx.x;
  const int h = blockIdx.y;
  const int A = p.arenas_per_batch, Hq = p.n_q_heads, R = p.rank;
  const int g = h / (Hq / p.n_basis_groups);
  const int a = b * A + (h * A) / Hq;
  if ((MODE == MODE_ATTN || MODE == MODE_ATTN_SPLIT) && row_routed_out(p, b)) return;   // the row belongs to the other kernel
  int S = p.seq_len;
  if (p.seq_lens) S = min(S, max(p.seq_lens[b], 0));
  int t_begin = 0, t_end = S;
  if (MODE == MODE_SCORES) {
    t_begin = blockIdx.z * GZ_TOKENS;
    t_end = min(p.seq_len, t_begin + GZ_TOKENS);  // scores are written for every column
  }
  if (MODE == MODE_ATTN_SPLIT) {
    t_begin = min(S, (int)blockIdx.z * split_tokens);
    t_end = min(S, t_begin + split_tokens);
  }

  const T* kflat = reinterpret_cast<const T*>(p.k.flat) + (size_t)a * p.k.flat_stride;
  const T* vflat = reinterpret_cast<const T*>(p.v.flat) + (size_t)a * p.v.flat_stride;
  const T* kup = reinterpret_cast<const T*>(p.k_up) + (size_t)g * R * GD;
  const T* vup = reinterpret_cast<const T*>(p.v_up) + (size_t)g * R * GD;
  const float scale = rsqrtf((float)GD);

  if (MODE != MODE_SOFTMAX_V && tid < GD) {
    const T* qp = reinterpret_cast<const T*>(p.q) + (size_t)b * p.q_stride_b + (size_t)h * p.q_stride_h;
    q_s[tid] = to_f32(qp[tid]);
  }
  // rotation frequencies of this lane's two pairs (dims lane, lane + 64 and lane + 32, lane + 96) and the rotation by
  // 8 positions (the token stride of a warp)
  const float fa = expf(-((float)(2 * lane) / (float)GD) * log_theta);
  const float fb = expf(-((float)(2 * (lane + 32)) / (float)GD) * log_theta);
  float s8a, c8a, s8b, c8b;
  sincosf(8.f * fa, &s8a, &c8a);
  sincosf(8.f * fb, &s8b, &c8b);
  float m_run = -INFINITY;
  float acc_lat[4] = {0.f, 0.f, 0.f, 0.f};
  if (tid == 0) l_s = 0.f;
  const int d = tid & (GD - 1), th = tid >> 7;
  __syncthreads();

  for (int t0 = t_begin; t0 < t_end; t0 += GTT) {
    // ---- token metadata ----
    if (tid < GTT) {
      const int s = t0 + tid;
      const bool in = s < t_end;
      int lk = 0, ok = 0, lv = 0, ov = 0;
      if (in) {
        if (MODE != MODE_SOFTMAX_V) {
          lk = p.k.lens[(size_t)a * p.k.lens_stride_a + (size_t)s * p.k.lens_stride_s];
          ok = p.k.offs[(size_t)a * p.k.offs_stride_a + (size_t)s * p.k.offs_stride_s];
          lk = min(max(lk, 0), R);
          if (ok < 0 || (int64_t)ok + lk > p.k.flat_stride) {   // would read outside the arena row: dropped, flagged
            set_status(p.status, DKV_ST_BAD_LENGTH);
            lk = 0; ok = 0;
          }
        }
        if (MODE != MODE_SCORES) {
          lv = p.v.lens[(size_t)a * p.v.lens_stride_a + (size_t)s * p.v.lens_stride_s];
          ov = p.v.offs[(size_t)a * p.v.offs_stride_a + (size_t)s * p.v.offs_stride_s];
          lv = min(max(lv, 0), R);
          if (ov < 0 || (int64_t)ov + lv > p.v.flat_stride) {
            set_status(p.status, DKV_ST_BAD_LENGTH);
            lv = 0; ov = 0;
          }
        }
      }
      lenk_s[tid] = lk; offk_s[tid] = ok; lenv_s[tid] = lv; offv_s[tid] = ov;
      int mx = lk;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (tid == 0) rmax_s = mx;
    }
    __syncthreads();

    if (MODE != MODE_SOFTMAX_V) {
      // ---- K reconstruction: k[t][d] = sum_r x[t][r] * Bk[r][d] ----
      const int rmax = rmax_s;
      if constexpr (sizeof(T) == 2) {
        // 16-bit storage: mma.sync m16n8k16 with fp32 accumulation (what the reference's tl.dot does); warp w owns
        // output dims 16w..16w+15 of all 32 tokens
        T (*xs)[GRC + 8] = reinterpret_cast<T (*)[GRC + 8]>(stage_raw);
        T (*bs)[GD + 8] = reinterpret_cast<T (*)[GD + 8]>(stage_raw + GTT * (GRC + 8) * 2);
        const bool vec = (reinterpret_cast<uintptr_t>(p.k_up) & 15) == 0;
        float acc[2][2][4];
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
        // The chunk after the one being multiplied is already on its way from global memory into registers (8
        // coefficients and 4 basis pieces per thread), so a step costs max(load, products), not their sum.
        constexpr int XPT = GTT * GRC / GTHREADS;            // x elements per thread per chunk (8)
        constexpr int BPT = GRC * (GD / 8) / GTHREADS;       // 16-byte basis pieces per thread per chunk (4)
        T xr[XPT];
        uint4 br[BPT];
        auto fetch = [&](int r0) {
#pragma unroll
          for (int u = 0; u < XPT; ++u) {
            const int e = tid + u * GTHREADS, t = e / GRC, r = r0 + (e - t * GRC);
            xr[u] = (r < lenk_s[t]) ? kflat[(size_t)offk_s[t] + r] : from_f32<T>(0.f);
          }
#pragma unroll
          for (int u = 0; u < BPT; ++u) {
            const int e = tid + u * GTHREADS, rr = e >> 4, c = e & 15, r = r0 + rr;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < R) {
              if (vec) {
                v = __ldg(reinterpret_cast<const uint4*>(kup + (size_t)r * GD) + c);
              } else {
                T tmp[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) tmp[i] = kup[(size_t)r * GD + 8 * c + i];
                v = *reinterpret_cast<const uint4*>(tmp);
              }
            }
            br[u] = v;
          }
        };
        if (rmax > 0) fetch(0);
        for (int r0 = 0; r0 < rmax; r0 += GRC) {
#pragma unroll
          for (int u = 0; u < XPT; ++u) {
            const int e = tid + u * GTHREADS, t = e / GRC;
            xs[t][e - t * GRC] = xr[u];
          }
#pragma unroll
          for (int u = 0; u < BPT; ++u) {
            const int e = tid + u * GTHREADS;
            *reinterpret_cast<uint4*>(&bs[e >> 4][8 * (e & 15)]) = br[u];
          }
          __syncthreads();
          if (r0 + GRC < rmax) fetch(r0 + GRC);
          const int ksteps = (min(GRC, rmax - r0) + 15) >> 4;
          for (int ks = 0; ks < ksteps; ++ks) {
            uint32_t af[2][4], bf[4];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
              const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&xs[16 * m + (lane & 15)][16 * ks + 8 * (lane >> 4)]);
              asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                           : "=r"(af[m][0]), "=r"(af[m][1]), "=r"(af[m][2]), "=r"(af[m][3]) : "r"(addr));
            }
            {
              const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&bs[16 * ks + (lane & 15)][16 * warp + 8 * (lane >> 4)]);
              asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                           : "=r"(bf[0]), "=r"(bf[1]), "=r"(bf[2]), "=r"(bf[3]) : "r"(addr));
            }
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
              for (int n = 0; n < 2; ++n) {
                if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                               : "+f"(acc[m][n][0]), "+f"(acc[m][n][1]), "+f"(acc[m][n][2]), "+f"(acc[m][n][3])
                               : "r"(af[m][0]), "r"(af[m][1]), "r"(af[m][2]), "r"(af[m][3]), "r"(bf[2 * n]), "r"(bf[2 * n + 1]));
                } else {
                  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                               : "+f"(acc[m][n][0]), "+f"(acc[m][n][1]), "+f"(acc[m][n][2]), "+f"(acc[m][n][3])
                               : "r"(af[m][0]), "r"(af[m][1]), "r"(af[m][2]), "r"(af[m][3]), "r"(bf[2 * n]), "r"(bf[2 * n + 1]));
                }
              }
          }
          __syncthreads();
        }
        const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            const int row = 16 * m + gq, col = 16 * warp + 8 * n + 2 * tq;
            k_s[row][col] = acc[m][n][0]; k_s[row][col + 1] = acc[m][n][1];
            k_s[row + 8][col] = acc[m][n][2]; k_s[row + 8][col + 1] = acc[m][n][3];
          }
      } else {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        for (int r0 = 0; r0 < rmax; r0 += GRC) {
          for (int e = tid; e < GTT * GRC; e += GTHREADS) {
            const int t = e / GRC, rr = e - t * GRC, r = r0 + rr;
            x_s[t][rr] = (r < lenk_s[t]) ? to_f32(kflat[(size_t)offk_s[t] + r]) : 0.f;
          }
          __syncthreads();
          const int nr = min(GRC, rmax - r0);
          for (int rr = 0; rr < nr; ++rr) {
            const float bv = to_f32(kup[(size_t)(r0 + rr) * GD + d]);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = fmaf(x_s[th * 16 + i][rr], bv, acc[i]);
          }
          __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) k_s[th * 16 + i][d] = acc[i];
      }
      __syncthreads();

      // ---- optional RMSNorm, RoPE, q.k : one warp per token (tokens warp, warp + 8, ...) ----
      // 16-bit types: exact sincos for the warp's first token of the tile, then a rotation by 8 positions per step
      // (three steps; the 16-bit tolerance is 2e-2).  fp32 keeps one exact sincos per token, the reference's arithmetic.
      float sa = 0.f, ca = 1.f, sb = 0.f, cb = 1.f;
      for (int t = warp; t < GTT; t += GTHREADS / 32) {
        const int s = t0 + t;
        float k0a = k_s[t][lane], k0b = k_s[t][lane + 32];            // dims j = lane, lane+32
        float k1a = k_s[t][lane + 64], k1b = k_s[t][lane + 96];       // dims j + 64
        if (p.k_norm_weight) {
          float ss = warp_sum(k0a * k0a + k0b * k0b + k1a * k1a + k1b * k1b);
          const float rs = rsqrtf(ss * (1.0f / GD) + p.k_norm_eps);
          k0a = p.k_norm_weight[lane] * (k0a * rs);
          k0b = p.k_norm_weight[lane + 32] * (k0b * rs);
          k1a = p.k_norm_weight[lane + 64] * (k1a * rs);
          k1b = p.k_norm_weight[lane + 96] * (k1b * rs);
        }
        if (sizeof(T) != 2 || t == warp) {
          sincosf((float)s * fa, &sa, &ca);
          sincosf((float)s * fb, &sb, &cb);
        } else {
          const float ca2 = ca * c8a - sa * s8a, sa2 = sa * c8a + ca * s8a;
          const float cb2 = cb * c8b - sb * s8b, sb2 = sb * c8b + cb * s8b;
          ca = ca2; sa = sa2; cb = cb2; sb = sb2;
        }
        float part = q_s[lane] * (k0a * ca - k1a * sa) + q_s[lane + 64] * (k1a * ca + k0a * sa) +
                     q_s[lane + 32] * (k0b * cb - k1b * sb) + q_s[lane + 96] * (k1b * cb + k0b * sb);
        part = warp_sum(part);
        if (lane == 0) {
          const bool in = s < t_end;
          if (MODE == MODE_SCORES) {
            if (in) {
              const float v = (lenk_s[t] > 0 ? part : -1.0e4f) * scale;
              T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)h * p.out_stride_h;
              op[s] = from_f32<T>(v);
            }
          } else {
            sc_s[t] = (in && lenk_s[t] > 0) ? part * scale : -INFINITY;
          }
        }
      }
      __syncthreads();
    } else {
      if (tid < GTT) {
        const int s = t0 + tid;
        sc_s[tid] = (s < t_end) ? to_f32(scores_in[(size_t)b * sc_sb + (size_t)h * sc_sh + s]) : -INFINITY;
      }
      __syncthreads();
    }

    if (MODE != MODE_SCORES) {
      // ---- online softmax over the tile (warp 0) ----
      if (warp == 0) {
        const float sc = sc_s[lane];
        const float m_new = fmaxf(m_run, warp_max(sc));
        const float alpha = (m_new == -INFINITY) ? 1.f : __expf(m_run - m_new);
        const float pv = (sc == -INFINITY) ? 0.f : __expf(sc - m_new);
        const float lsum = warp_sum(pv);
        p_s[lane] = pv;
        if (lane == 0) { alpha_s = alpha; l_s = l_s * alpha + lsum; }
        m_run = m_new;
      }
      __syncthreads();
      // every thread tracks the running max through alpha only; warp 0 owns m_run
      const float alpha = alpha_s;
      // ---- latent-space V accumulation: thread owns latent indices tid + 256 i; eight tokens' loads in flight ----
#pragma unroll
      for (int i = 0; i < 4; ++i) acc_lat[i] *= alpha;
      for (int tb = 0; tb < GTT; tb += 8) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int t = tb + u;
          const int lv = p_s[t] != 0.f ? lenv_s[t] : 0;
          const T* row = vflat + (size_t)offv_s[t];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = tid + i * GTHREADS;
            v[i][u] = r < lv ? to_f32(row[r]) : 0.f;     // lv <= R
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float pv = p_s[tb + u];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc_lat[i] = fmaf(pv, v[i][u], acc_lat[i]);
        }
      }
      __syncthreads();
    }
  }

  if (MODE == MODE_SCORES) return;
  if (MODE == MODE_ATTN_SPLIT) {
    // partial record of this slice: [m, l, acc[R]] at ((row, head), slice)
    float* rec = reinterpret_cast<float*>(p.workspace) +
                 (((size_t)blockIdx.x * Hq + h) * gridDim.z + blockIdx.z) * (size_t)(2 + R);
    if (tid == 0) { rec[0] = m_run; rec[1] = l_s; }      // warp 0 owns the running maximum
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = tid + i * GTHREADS;
      if (r < R) rec[2 + r] = acc_lat[i];
    }
    return;
  }

  // ---- normalise and project the latent accumulator through Bv ----
  float* lat_s = &k_s[0][0];  // >= 1024 floats
  const float l = l_s;
  float inv;
  if (MODE == MODE_SOFTMAX_V) inv = 1.f / fmaxf(l, 1e-6f);
  else inv = l > 0.f ? 1.f / l : 0.f;
  if (MODE == MODE_ATTN && l <= 0.f && tid == 0) set_status(p.status, DKV_ST_EMPTY_ROW);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = tid + i * GTHREADS;
    if (r < R) lat_s[r] = acc_lat[i] * inv;
  }
  __syncthreads();
  const int r_half = (R + 1) / 2;
  const int r_lo = th * r_half, r_hi = min(R, r_lo + r_half);
  float o = 0.f;
  for (int r = r_lo; r < r_hi; ++r) o = fmaf(lat_s[r], to_f32(vup[(size_t)r * GD + d]), o);
  __syncthreads();
  float* half_s = &x_s[0][0];  // first 128 floats of the staging tile
  if (th == 1) half_s[d] = o;
  __syncthreads();
  if (th == 0) {
    const float o1 = half_s[d];
    T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)h * p.out_stride_h;
    op[d] = from_f32<T>(o + o1);
  }
}

// Merge the slices' partial records of one (row, head) and project through Bv (MODE_ATTN_SPLIT's second half).
template <typename T>
__global__ void __launch_bounds__(GTHREADS) generic_combine_kernel(dkv_attn_args p, int n_split) {
  __shared__ float lat_s[1024];
  __shared__ float w_s[64];
  __shared__ float red_s[16][GD];
  __shared__ float L_s;
  const int tid = threadIdx.x, h = blockIdx.y, Hq = p.n_q_heads, R = p.rank;
  const int b = p.batch_index ? p.batch_index[blockIdx.x] : blockIdx.x;
  if (row_routed_out(p, b)) return;
  const int g = h / (Hq / p.n_basis_groups);
  const float* rec0 = reinterpret_cast<const float*>(p.workspace) + (((size_t)blockIdx.x * Hq + h) * n_split) * (size_t)(2 + R);
  if (tid < 32) {
    float M = -INFINITY;
    for (int k = tid; k < n_split; k += 32) M = fmaxf(M, rec0[(size_t)k * (2 + R)]);
    M = warp_max(M);
    float L = 0.f;
    for (int k = tid; k < n_split; k += 32) {
      const float m = rec0[(size_t)k * (2 + R)];
      const float w = (m == -INFINITY) ? 0.f : __expf(m - M);
      w_s[k] = w;
      L = fmaf(w, rec0[(size_t)k * (2 + R) + 1], L);
    }
    L = warp_sum(L);
    if (tid == 0) L_s = L;
  }
  __syncthreads();
  const float L = L_s;
  if (L <= 0.f && tid == 0) set_status(p.status, DKV_ST_EMPTY_ROW);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int r = tid; r < R; r += GTHREADS) {
    float v = 0.f;
    for (int k = 0; k < n_split; ++k)
      if (w_s[k] != 0.f) v = fmaf(w_s[k], rec0[(size_t)k * (2 + R) + 2 + r], v);
    lat_s[r] = v * inv;
  }
  __syncthreads();
  // projection through Bv: thread (rg, dg) takes latent rows rg, rg + 16, ... and the 8 output dims 8 dg..8 dg + 7
  // (one 16-byte load per row, eight rows in flight); the 16 row groups are added up through shared memory
  const T* vup = reinterpret_cast<const T*>(p.v_up) + (size_t)g * R * GD;
  const int dg = tid & 15, rg = tid >> 4;
  const bool vec = (reinterpret_cast<uintptr_t>(p.v_up) & 15) == 0 && sizeof(T) == 2;
  float acc8[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc8[e] = 0.f;
  if (vec) {
#pragma unroll 8
    for (int r = rg; r < R; r += 16) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(vup + (size_t)r * GD) + dg);
      const T* vp = reinterpret_cast<const T*>(&v);
      const float lr = lat_s[r];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc8[e] = fmaf(lr, to_f32(vp[e]), acc8[e]);
    }
  } else {
#pragma unroll 4
    for (int r = rg; r < R; r += 16) {
      const float lr = lat_s[r];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc8[e] = fmaf(lr, to_f32(vup[(size_t)r * GD + 8 * dg + e]), acc8[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red_s[rg][8 * dg + e] = acc8[e];
  __syncthreads();
  if (tid < GD) {
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) o += red_s[k][tid];
    T* op = reinterpret_cast<T*>(p.out) + (size_t)b * p.out_stride_b + (size_t)h * p.out_stride_h;
    op[tid] = from_f32<T>(o);
  }
}

// Slices of the token axis for the two-stage entry on caches that take this path: at least 128 tokens each, at most 64.
static int generic_split_tokens(const dkv_attn_args* a) {
  int t = (a->seq_len + 63) / 64;
  t = (t + GTT - 1) / GTT * GTT;
  return t < 128 ? 128 : t;
}
static int generic_n_split(const dkv_attn_args* a) {
  const int t = generic_split_tokens(a);
  const int n = (a->seq_len + t - 1) / t;
  return n < 1 ? 1 : n;
}
size_t generic_split_workspace_bytes(const dkv_attn_args* a) {
  const int n = generic_n_split(a);
  if (n <= 1) return 0;
  return (size_t)a->batch * a->n_q_heads * n * (size_t)(2 + a->rank) * sizeof(float);
}

int check_attn_args(const dkv_attn_args* a, const char* who, bool need_q, bool need_k, bool need_v) {
  DKV_REQUIRE(a != nullptr, DKV_E_ARG, "%s: null args", who);
  DKV_REQUIRE(a->dtype >= DKV_F32 && a->dtype <= DKV_BF16, DKV_E_ARG, "%s: bad dtype %d", who, a->dtype);
  DKV_REQUIRE(a->head_dim == 128, DKV_E_ARG, "%s: head_dim must be 128 (got %d)", who, a->head_dim);
  DKV_REQUIRE(a->rank >= 1 && a->rank <= 1024, DKV_E_ARG, "%s: rank must be in 1..1024 (got %d)", who, a->rank);
  DKV_REQUIRE(a->batch >= 0 && a->seq_len >= 0, DKV_E_ARG, "%s: negative batch or seq_len", who);
  DKV_REQUIRE(a->n_q_heads >= 1 && a->n_basis_groups >= 1 && a->n_q_heads % a->n_basis_groups == 0, DKV_E_ARG,
              "%s: n_q_heads (%d) must be a positive multiple of n_basis_groups (%d)", who, a->n_q_heads,
              a->n_basis_groups);
  DKV_REQUIRE(a->arenas_per_batch >= 1 && a->n_q_heads % a->arenas_per_batch == 0, DKV_E_ARG,
              "%s: n_q_heads (%d) must be a multiple of arenas_per_batch (%d)", who, a->n_q_heads, a->arenas_per_batch);
  DKV_REQUIRE(a->n_q_heads <= 65535, DKV_E_LIMIT, "%s: too many heads", who);
  DKV_REQUIRE(a->out != nullptr, DKV_E_ARG, "%s: null out", who);
  if (need_q) DKV_REQUIRE(a->q != nullptr, DKV_E_ARG, "%s: null q", who);
  if (need_k) DKV_REQUIRE(a->k_up && a->k.flat && a->k.lens && a->k.offs, DKV_E_ARG, "%s: null K-side input", who);
  if (need_v) DKV_REQUIRE(a->v_up && a->v.flat && a->v.lens && a->v.offs, DKV_E_ARG, "%s: null V-side input", who);
  return DKV_OK;
}

template <int MODE>
static int launch_generic(const dkv_attn_args* a, const void* scores, int64_t sb, int64_t sh) {
  if (a->batch == 0) return DKV_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  dim3 grid(a->batch, a->n_q_heads, 1);
  if (MODE == MODE_SCORES) {
    if (a->seq_len == 0) return DKV_OK;
    grid.z = (a->seq_len + GZ_TOKENS - 1) / GZ_TOKENS;
    DKV_REQUIRE(grid.z <= 65535, DKV_E_LIMIT, "dkv_scores: seq_len too large");
  }
  const float log_theta = (float)log((double)a->theta);
  int split_tokens = 0, n_split = 1;
  if (MODE == MODE_ATTN_SPLIT) {
    split_tokens = generic_split_tokens(a);
    n_split = generic_n_split(a);
    grid.z = n_split;
  }
  if (a->dtype == DKV_F32)
    generic_decode_kernel<float, MODE><<<grid, GTHREADS, 0, st>>>(*a, (const float*)scores, sb, sh, log_theta, split_tokens);
  else if (a->dtype == DKV_F16)
    generic_decode_kernel<__half, MODE><<<grid, GTHREADS, 0, st>>>(*a, (const __half*)scores, sb, sh, log_theta, split_tokens);
  else
    generic_decode_kernel<__nv_bfloat16, MODE><<<grid, GTHREADS, 0, st>>>(*a, (const __nv_bfloat16*)scores, sb, sh,
                                                                        log_theta, split_tokens);
  DKV_CHECK_LAUNCH();
  if (MODE == MODE_ATTN_SPLIT) {
    const dim3 cgrid(a->batch, a->n_q_heads);
    if (a->dtype == DKV_F32) generic_combine_kernel<float><<<cgrid, GTHREADS, 0, st>>>(*a, n_split);
    else if (a->dtype == DKV_F16) generic_combine_kernel<__half><<<cgrid, GTHREADS, 0, st>>>(*a, n_split);
    else generic_combine_kernel<__nv_bfloat16><<<cgrid, GTHREADS, 0, st>>>(*a, n_split);
    DKV_CHECK_LAUNCH();
  }
  return DKV_OK;
}

int generic_attention(const dkv_attn_args* a) { return launch_generic<MODE_ATTN>(a, nullptr, 0, 0); }

// Two-stage entry on this path: slices of the token axis + merge when the caller's workspace holds the records,
// one CTA per (row, head) otherwise.
int generic_two_stage(const dkv_attn_args* a) {
  const size_t need = generic_split_workspace_bytes(a);
  if (need == 0 || a->workspace == nullptr || a->workspace_bytes < need) return generic_attention(a);
  return launch_generic<MODE_ATTN_SPLIT>(a, nullptr, 0, 0);
}

}  // namespace dkv

using namespace dkv;

extern "C" int dkv_scores(const dkv_attn_args* a) {
  if (int rc = check_attn_args(a, "dkv_scores", true, true, false)) return rc;
  return launch_generic<MODE_SCORES>(a, nullptr, 0, 0);
}

extern "C" int dkv_softmax_v(const dkv_attn_args* a, const void* scores, int64_t sc_stride_b, int64_t sc_stride_h) {
  if (int rc = check_attn_args(a, "dkv_softmax_v", false, false, true)) return rc;
  DKV_REQUIRE(scores != nullptr, DKV_E_ARG, "dkv_softmax_v: null scores");
  return launch_generic<MODE_SOFTMAX_V>(a, scores, sc_stride_b, sc_stride_h);
}
