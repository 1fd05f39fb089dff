// Cache-update kernels: decode append, bulk (prefill) pack, ragged -> dense decompress.
//
// Layout contract (reference: src/dynakv/kernels/compressed_cache.py:7-34, 184-209):
//   lens[a,s] = r_s,  offs[a,s] = sum_{t<s} lens[a,t],  flat[a, offs .. offs+r_s) = first r_s
//   coefficients of token s,  ptr[a] = sum_s lens[a,s].  Payload is copied verbatim (bit-exact).
#include "dkv_common.cuh"

namespace dkv {

template <typename T>
__device__ __forceinline__ void copy_row(T* dst, const T* src, int n, int lane) {
  for (int i = lane; i < n; i += 32) dst[i] = src[i];
}

// Validate a length against [0, max_dim] and the declared step; returns the sanitised value.  A length that is not
// a multiple of the step is rounded UP (capped at max_dim): the stored row is then a superset of what the caller
// asked to keep, never a truncation of it.  Either way the call is flagged.
__device__ __forceinline__ int checked_len(int len, int max_dim, int step, int32_t* status, int lane) {
  bool bad = (len < 0) || (len > max_dim) || (step > 1 && (len % step) != 0);
  if (bad) {
    if (lane == 0) set_status(status, DKV_ST_BAD_LENGTH);
    len = min(max(len, 0), max_dim);
    if (step > 1 && (len % step) != 0) len = min(len + step - len % step, max_dim - max_dim % step);
  }
  return len;
}

// One block per batch row; each warp owns one (arena, side) row at a time.
template <typename T>
__global__ void __launch_bounds__(512) append_decode_kernel(dkv_append_args p) {
  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int A = p.arenas_per_batch;
  const int pos = p.seq_lens ? p.seq_lens[b] : p.seq_pos;
  const bool pos_ok = pos >= 0 && pos < p.seq_capacity;
  if (!pos_ok && threadIdx.x == 0) set_status(p.status, DKV_ST_OVERFLOW);

  for (int item = warp; pos_ok && item < 2 * A; item += n_warps) {
    const int side_idx = item / A, j = item - side_idx * A;
    const dkv_side& sd = side_idx ? p.v : p.k;
    const int a = b * A + j;
    const T* src = reinterpret_cast<const T*>(side_idx ? p.new_v : p.new_k) + (size_t)a * p.max_dim;
    int len = (side_idx ? p.len_v : p.len_k)[a];
    len = checked_len(len, p.max_dim, p.len_multiple, p.status, lane);
    const int off = sd.ptr[a];
    if ((int64_t)off + len > sd.flat_stride) {
      if (lane == 0) {   // the token is recorded as empty, so that attention never reads stale metadata for it
        set_status(p.status, DKV_ST_OVERFLOW);
        sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s] = 0;
        sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s] = off;
      }
      continue;
    }
    T* dst = reinterpret_cast<T*>(sd.flat) + (size_t)a * sd.flat_stride + off;
    copy_row(dst, src, len, lane);
    __syncwarp();
    if (lane == 0) {
      sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s] = len;
      sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s] = off;
      sd.ptr[a] = off + len;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && p.seq_lens && pos_ok) p.seq_lens[b] = pos + 1;
}

// Decode append with in-kernel projection (per-head layout, max_dim == head_dim == 128):
// coefficient r = sum_d x[d] * basis[j, r, d].  One block per batch row; each (arena, side) row is
// shared by `wpi` warps.  A warp takes 8 basis rows per iteration: lane l holds x[4l..4l+3], loads its
// 8-byte slice of each row (coalesced 256 B per row), and the 8 dot products are reduced with
// interleaved shuffles, so eight independent L2 loads are in flight per lane.
template <typename T>
__global__ void __launch_bounds__(1024) append_project_kernel(dkv_append_args p, int wpi) {
  pdl_launch_dependents();   // the attention kernel after this one may start its set-up (which reads no cache state) now
  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int A = p.arenas_per_batch;
  const int pos = p.seq_lens ? p.seq_lens[b] : p.seq_pos;
  const bool pos_ok = pos >= 0 && pos < p.seq_capacity;
  if (!pos_ok && threadIdx.x == 0) set_status(p.status, DKV_ST_OVERFLOW);
  const int n_items = 2 * A;
  const int warps_total = blockDim.x >> 5;
  for (int item = warp / wpi; pos_ok && item < n_items; item += warps_total / wpi) {
    const int sub = warp % wpi;
    const int side_idx = item / A, j = item - side_idx * A;
    const dkv_side& sd = side_idx ? p.v : p.k;
    const int a = b * A + j;
    const T* src = reinterpret_cast<const T*>(side_idx ? p.new_v : p.new_k) + (size_t)a * 128;
    int len = (side_idx ? p.len_v : p.len_k)[a];
    len = checked_len(len, 128, p.len_multiple, p.status, lane + sub);
    const int off = sd.ptr[a];
    if ((int64_t)off + len > sd.flat_stride) {
      if (lane == 0 && sub == 0) {   // recorded as an empty token (the pointer pass below then adds nothing)
        set_status(p.status, DKV_ST_OVERFLOW);
        sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s] = 0;
        sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s] = off;
      }
      continue;
    }
    T* dst = reinterpret_cast<T*>(sd.flat) + (size_t)a * sd.flat_stride + off;
    const T* basis = reinterpret_cast<const T*>(side_idx ? p.v_basis : p.k_basis) + (size_t)j * 128 * 128;
    float x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = to_f32(src[lane * 4 + e]);
    for (int r0 = sub * 8; r0 < len; r0 += 8 * wpi) {
      float acc[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const T* row = basis + (size_t)(r0 + u) * 128 + lane * 4;   // r0 + u < 128 always (len <= 128, step 8)
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) s = fmaf(x[e], to_f32(row[e]), s);
        acc[u] = s;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
      }
      if (lane < 8 && r0 + lane < len) {
        float v = acc[0];
#pragma unroll
        for (int u = 1; u < 8; ++u) v = (lane == u) ? acc[u] : v;
        dst[r0 + lane] = from_f32<T>(v);
      }
    }
    if (lane == 0 && sub == 0) {
      sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s] = len;
      sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s] = off;
    }
  }
  __syncthreads();   // every warp has read ptr[] and seq_lens[] before they move
  for (int item = threadIdx.x; pos_ok && item < n_items; item += blockDim.x) {
    const int side_idx = item / A, j = item - side_idx * A;
    const dkv_side& sd = side_idx ? p.v : p.k;
    const int a = b * A + j;
    const int len = sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s];
    const int off = sd.ptr[a];
    if ((int64_t)off + len <= sd.flat_stride) sd.ptr[a] = off + len;
  }
  if (threadIdx.x == 0 && p.seq_lens && pos_ok) p.seq_lens[b] = pos + 1;
}

// The same append with one CTA per (arena row, side): grid (2 * arenas_per_batch, batch), 8 warps that take 8 basis
// rows each per iteration (at most two iterations).  Each CTA advances its own write pointer; the per-row token
// counter is read by all CTAs of a batch row, so the last of them to finish (a ticket per batch row, left at zero
// again) advances it.
template <typename T>
__global__ void __launch_bounds__(256) append_project_grid_kernel(dkv_append_args p) {
  pdl_launch_dependents();
  const int b = blockIdx.y, item = blockIdx.x, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int A = p.arenas_per_batch;
  const int pos = p.seq_lens ? p.seq_lens[b] : p.seq_pos;
  const bool pos_ok = pos >= 0 && pos < p.seq_capacity;
  if (!pos_ok && tid == 0 && item == 0) set_status(p.status, DKV_ST_OVERFLOW);
  if (pos_ok) {
    const int side_idx = item / A, j = item - side_idx * A;
    const dkv_side& sd = side_idx ? p.v : p.k;
    const int a = b * A + j;
    const T* src = reinterpret_cast<const T*>(side_idx ? p.new_v : p.new_k) + (size_t)a * 128;
    const int len = checked_len((side_idx ? p.len_v : p.len_k)[a], 128, p.len_multiple, p.status, tid);
    const int off = sd.ptr[a];
    const bool fits = (int64_t)off + len <= sd.flat_stride;
    if (fits) {
      T* dst = reinterpret_cast<T*>(sd.flat) + (size_t)a * sd.flat_stride + off;
      const T* basis = reinterpret_cast<const T*>(side_idx ? p.v_basis : p.k_basis) + (size_t)j * 128 * 128;
      float x[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = to_f32(src[lane * 4 + e]);
      for (int r0 = warp * 8; r0 < len; r0 += 64) {
        float acc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const T* row = basis + (size_t)(r0 + u) * 128 + lane * 4;   // r0 + u < 128 always (len <= 128, step 8)
          float s = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) s = fmaf(x[e], to_f32(row[e]), s);
          acc[u] = s;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
          for (int u = 0; u < 8; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
        }
        if (lane < 8 && r0 + lane < len) {
          float v = acc[0];
#pragma unroll
          for (int u = 1; u < 8; ++u) v = (lane == u) ? acc[u] : v;
          dst[r0 + lane] = from_f32<T>(v);
        }
      }
    }
    __syncthreads();   // every thread has read ptr[a]
    if (tid == 0) {
      if (!fits) set_status(p.status, DKV_ST_OVERFLOW);   // recorded as an empty token
      sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s] = fits ? len : 0;
      sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s] = off;
      if (fits) sd.ptr[a] = off + len;
    }
  } else {
    __syncthreads();
  }
  if (tid == 0 && p.seq_lens) {     // tid 0 read seq_lens[b] above; the barrier orders the other threads' reads
    __threadfence();
    if (atomicAdd(&p.tickets[b], 1) == 2 * A - 1) {
      p.tickets[b] = 0;
      if (pos_ok) p.seq_lens[b] = pos + 1;
    }
  }
}

// Bulk (prefill) pack, two kernels on the caller's stream.
//  1. pack_scan_kernel, one CTA per (block of 1024 new tokens, arena row): validates the row's new lengths, adds
//     them up (the whole for the fits test, the part before its block for its first offset) and writes lens / offs
//     of its tokens.  A block whose payload does not fit is flagged and its tokens are recorded as empty (lens 0,
//     offs = the write pointer: the rule of the decode append), so that attention never reads stale metadata for
//     them; a block whose positions do not fit the metadata row is flagged and nothing is written.  The write
//     pointer is read by every CTA of the row, so it is not advanced here.
//  2. pack_copy_kernel, one CTA per (block of 256 new tokens, arena row): reads the metadata just written, copies
//     the payload, and the CTA that holds the row's last new token advances the write pointer to that token's end.  A warp's 32 rows land back to back in the arena, so its payload is one run; with 16-bit elements,
//     lengths multiples of 8 and aligned bases and strides the run moves as 16-byte pieces, one per lane whatever
//     the rows' lengths (the source of a piece is found by a binary search over the rows' piece prefixes, held
//     one per lane), four pieces per lane in flight; element by element otherwise.
constexpr int SCAN_THREADS = 1024, COPY_THREADS = 256;

struct pack_row {
  int base, n_new, pos0;
};
__device__ __forceinline__ pack_row pack_row_of(const dkv_pack_args& p, int a, int b) {
  pack_row r;
  r.base = p.side.ptr[a];
  r.n_new = p.row_counts ? min(max(p.row_counts[b], 0), p.n_new) : p.n_new;
  r.pos0 = p.seq_lens ? p.seq_lens[b] : p.seq_pos;
  return r;
}
__device__ __forceinline__ bool positions_fit(const dkv_pack_args& p, const pack_row& r) {
  return r.pos0 >= 0 && r.pos0 + r.n_new <= p.seq_capacity;
}

__global__ void __launch_bounds__(SCAN_THREADS) pack_scan_kernel(dkv_pack_args p) {
  __shared__ int red[2 * SCAN_THREADS / 32];
  __shared__ int warp_tot[SCAN_THREADS / 32];
  const int a = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const dkv_side& sd = p.side;
  const pack_row r = pack_row_of(p, a, a / p.arenas_per_batch);
  const int s0 = blockIdx.x * SCAN_THREADS;
  const int32_t* nl = p.new_lens + (size_t)a * p.n_new;
  if (s0 >= r.n_new && s0 > 0) return;
  int32_t* flag = blockIdx.x == 0 ? p.status : nullptr;      // each fault is flagged by the row's first CTA
  if (!positions_fit(p, r)) {
    if (tid == 0) set_status(flag, DKV_ST_OVERFLOW);
    return;
  }
  // ---- the row's total (fits test) and the part before this CTA's tokens (its first offset): every CTA of the row
  // repeats the sum, four lengths per load, the repair path of checked_len only behind a cheap validity test
  const int step = p.len_multiple, mask = (step & (step - 1)) == 0 ? step - 1 : -1;
  auto valid_len = [&](int len) {
    const bool bad = (unsigned)len > (unsigned)p.max_dim || (mask >= 0 ? (len & mask) : (len % step)) != 0;
    return bad ? checked_len(len, p.max_dim, step, flag, 0) : len;
  };
  int before = 0, rest = 0;
  auto add = [&](int s, int len) {
    len = valid_len(len);
    if (s < s0) before += len; else rest += len;
  };
  if ((reinterpret_cast<uintptr_t>(nl) & 15) == 0) {
    const int n4 = r.n_new >> 2;
    for (int q = tid; q < n4; q += SCAN_THREADS) {
      const int4 v = __ldg(reinterpret_cast<const int4*>(nl) + q);
      add(4 * q, v.x); add(4 * q + 1, v.y); add(4 * q + 2, v.z); add(4 * q + 3, v.w);
    }
    for (int s = 4 * n4 + tid; s < r.n_new; s += SCAN_THREADS) add(s, nl[s]);
  } else {
    for (int s = tid; s < r.n_new; s += SCAN_THREADS) add(s, nl[s]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, o);
    rest += __shfl_xor_sync(0xffffffffu, rest, o);
  }
  if (lane == 0) { red[2 * warp] = before; red[2 * warp + 1] = rest; }
  __syncthreads();
  before = red[2 * lane];
  rest = red[2 * lane + 1];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, o);
    rest += __shfl_xor_sync(0xffffffffu, rest, o);
  }
  const bool fits = (int64_t)r.base + before + rest <= sd.flat_stride;
  if (!fits && tid == 0) set_status(flag, DKV_ST_OVERFLOW);

  // ---- metadata of this CTA's 1024 tokens
  const int s = s0 + tid;
  const int len = (fits && s < r.n_new) ? valid_len(nl[s]) : 0;
  int incl = len;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int w_incl = warp_tot[lane];       // inclusive scan of the 32 warp totals, repeated by every warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, w_incl, o);
    if (lane >= o) w_incl += t;
  }
  const int wbase = warp ? __shfl_sync(0xffffffffu, w_incl, warp - 1) : 0;
  if (s < r.n_new) {
    const int pos = r.pos0 + s;
    sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s] = len;
    sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s] =
        r.base + (fits ? before : 0) + wbase + incl - len;
  }
}

template <typename T>
__global__ void __launch_bounds__(COPY_THREADS) pack_copy_kernel(dkv_pack_args p, int vec16) {
  const int a = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = a / p.arenas_per_batch, j = a - b * p.arenas_per_batch;
  const dkv_side& sd = p.side;
  const int n_new = p.row_counts ? min(max(p.row_counts[b], 0), p.n_new) : p.n_new;
  const int pos0 = p.seq_lens ? p.seq_lens[b] : p.seq_pos;
  const int s0 = blockIdx.x * COPY_THREADS + 32 * warp;      // this warp's first token
  if (s0 >= n_new || pos0 < 0 || pos0 + n_new > p.seq_capacity) return;
  const int s = s0 + lane;
  int len = 0, off = 0;
  if (s < n_new) {
    const int pos = pos0 + s;
    len = sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s];
    off = sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s];
    if (s == n_new - 1) sd.ptr[a] = off + len;
  }
  const int first_off = __shfl_sync(0xffffffffu, off, 0);
  int run = off + len - first_off;                           // elements of the warp's run up to and with this row
  run = __shfl_sync(0xffffffffu, run, min(31, n_new - 1 - s0));
  if (run <= 0) return;
  const T* rows = reinterpret_cast<const T*>(p.states) + (size_t)b * p.stride_b + (size_t)j * p.stride_j +
                  (size_t)s0 * p.stride_s;
  T* flat = reinterpret_cast<T*>(sd.flat) + (size_t)a * sd.flat_stride + first_off;
  const int pre = s < n_new ? off - first_off : run;         // elements of the run before this row
  if (vec16 && (first_off & 7) == 0) {
    const int n_pieces = run >> 3, pre8 = pre >> 3;
    uint4* dst = reinterpret_cast<uint4*>(flat);
    for (int g0 = 0; g0 < n_pieces; g0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int g = g0 + 32 * u + lane;
        int i = 0;
#pragma unroll
        for (int bit = 16; bit > 0; bit >>= 1) {
          const int cand = i + bit;                                        // <= 31 by construction
          if (__shfl_sync(0xffffffffu, pre8, cand) <= g) i = cand;
        }
        const int first = __shfl_sync(0xffffffffu, pre8, i);
        if (g < n_pieces) v[u] = __ldcs(reinterpret_cast<const uint4*>(rows + (size_t)i * p.stride_s) + (g - first));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int g = g0 + 32 * u + lane;
        if (g < n_pieces) dst[g] = v[u];
      }
    }
  } else {
    for (int g0 = 0; g0 < run; g0 += 32) {
      const int g = g0 + lane;
      int i = 0;
#pragma unroll
      for (int bit = 16; bit > 0; bit >>= 1) {
        const int cand = i + bit;
        if (__shfl_sync(0xffffffffu, pre, cand) <= g) i = cand;
      }
      const int first = __shfl_sync(0xffffffffu, pre, i);
      if (g < run) flat[g] = rows[(size_t)i * p.stride_s + (g - first)];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) decompress_kernel(dkv_side sd, T* dense, int n_tok, int max_dim) {
  const int a = blockIdx.y, lane = threadIdx.x & 31;
  const int s = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (s >= n_tok) return;
  int len = min(max(sd.lens[(size_t)a * sd.lens_stride_a + (size_t)s * sd.lens_stride_s], 0), max_dim);
  int off = sd.offs[(size_t)a * sd.offs_stride_a + (size_t)s * sd.offs_stride_s];
  if (off < 0 || (int64_t)off + len > sd.flat_stride) { len = 0; off = 0; }   // never read outside the arena row
  const T* src = reinterpret_cast<const T*>(sd.flat) + (size_t)a * sd.flat_stride + off;
  T* dst = dense + ((size_t)a * n_tok + s) * max_dim;
  for (int i = lane; i < max_dim; i += 32) dst[i] = i < len ? src[i] : from_f32<T>(0.f);
}

static int check_side(const dkv_side& s, const char* what) {
  DKV_REQUIRE(s.flat && s.lens && s.offs, DKV_E_ARG, "%s: flat/lens/offs must be non-null", what);
  DKV_REQUIRE(s.flat_stride >= 0, DKV_E_ARG, "%s: negative flat_stride", what);
  return DKV_OK;
}

}  // namespace dkv

using namespace dkv;

extern "C" int dkv_append_decode(const dkv_append_args* a) {
  DKV_REQUIRE(a != nullptr, DKV_E_ARG, "dkv_append_decode: null args");
  DKV_REQUIRE(a->batch >= 0 && a->arenas_per_batch >= 1 && a->max_dim >= 1 && a->max_dim <= 1024, DKV_E_ARG,
              "dkv_append_decode: bad sizes (batch=%d arenas_per_batch=%d max_dim=%d)", a->batch,
              a->arenas_per_batch, a->max_dim);
  DKV_REQUIRE(a->dtype >= DKV_F32 && a->dtype <= DKV_BF16, DKV_E_ARG, "dkv_append_decode: bad dtype %d", a->dtype);
  DKV_REQUIRE(a->new_k && a->new_v && a->len_k && a->len_v, DKV_E_ARG, "dkv_append_decode: null input");
  DKV_REQUIRE((a->k_basis == nullptr) == (a->v_basis == nullptr), DKV_E_ARG,
              "dkv_append_decode: give both bases or neither");
  DKV_REQUIRE(a->len_multiple >= 1, DKV_E_ARG, "dkv_append_decode: len_multiple must be >= 1");
  if (int rc = check_side(a->k, "dkv_append_decode k")) return rc;
  if (int rc = check_side(a->v, "dkv_append_decode v")) return rc;
  DKV_REQUIRE(a->k.ptr && a->v.ptr, DKV_E_ARG, "dkv_append_decode: write pointers must be non-null");
  if (a->batch == 0) return DKV_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  const int items = 2 * a->arenas_per_batch;
  const int threads = 32 * (items < 16 ? items : 16);
  const bool proj = a->k_basis != nullptr;
  int wpi = 1;   // warps per (arena, side) row in the projecting kernel: fill a 1024-thread block
  while (wpi * 2 * items <= 32 && wpi < 4) wpi *= 2;
  if (proj)
    DKV_REQUIRE(a->max_dim == 128 && a->dtype != DKV_F32 && items <= 32, DKV_E_ARG,
                "dkv_append_decode: in-kernel projection needs 128-wide 16-bit rows and at most 16 arenas per batch row");
  const bool per_item = proj && (a->seq_lens == nullptr || a->tickets != nullptr) && a->batch <= 65535;
#define LAUNCH(T)                                                             \
  do {                                                                        \
    if (per_item) append_project_grid_kernel<T><<<dim3(items, a->batch), 256, 0, st>>>(*a); \
    else if (proj) append_project_kernel<T><<<a->batch, 32 * wpi * items, 0, st>>>(*a, wpi); \
    else append_decode_kernel<T><<<a->batch, threads, 0, st>>>(*a);    \
  } while (0)
  if (a->dtype == DKV_F32) LAUNCH(float);
  else if (a->dtype == DKV_F16) LAUNCH(__half);
  else LAUNCH(__nv_bfloat16);
#undef LAUNCH
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}

extern "C" int dkv_pack_bulk(const dkv_pack_args* a) {
  DKV_REQUIRE(a != nullptr, DKV_E_ARG, "dkv_pack_bulk: null args");
  DKV_REQUIRE(a->batch >= 0 && a->arenas_per_batch >= 1 && a->n_new >= 0 && a->max_dim >= 1 && a->max_dim <= 1024,
              DKV_E_ARG, "dkv_pack_bulk: bad sizes");
  DKV_REQUIRE(a->dtype >= DKV_F32 && a->dtype <= DKV_BF16, DKV_E_ARG, "dkv_pack_bulk: bad dtype %d", a->dtype);
  DKV_REQUIRE(a->states && a->new_lens && a->side.ptr, DKV_E_ARG, "dkv_pack_bulk: null input");
  DKV_REQUIRE(a->len_multiple >= 1, DKV_E_ARG, "dkv_pack_bulk: len_multiple must be >= 1");
  if (int rc = check_side(a->side, "dkv_pack_bulk side")) return rc;
  const int n_arena = a->batch * a->arenas_per_batch;
  if (n_arena == 0 || a->n_new == 0) return DKV_OK;
  DKV_REQUIRE(n_arena <= 65535, DKV_E_LIMIT, "dkv_pack_bulk: at most 65535 arena rows per call");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  // 16-byte copies when every row start is 16-byte aligned on both sides: 16-bit elements, lengths declared as
  // multiples of 8 (offsets are then multiples of 8 too), aligned bases and strides
  const bool two_byte = a->dtype != DKV_F32;
  const int vec16 = two_byte && a->len_multiple % 8 == 0 && (((uintptr_t)a->states | (uintptr_t)a->side.flat) & 15) == 0 &&
                    a->stride_b % 8 == 0 && a->stride_j % 8 == 0 && a->stride_s % 8 == 0 && a->side.flat_stride % 8 == 0;
  const dim3 scan_grid((unsigned)((a->n_new + SCAN_THREADS - 1) / SCAN_THREADS), (unsigned)n_arena);
  pack_scan_kernel<<<scan_grid, SCAN_THREADS, 0, st>>>(*a);
  const dim3 grid((unsigned)((a->n_new + COPY_THREADS - 1) / COPY_THREADS), (unsigned)n_arena);
  if (a->dtype == DKV_F32) pack_copy_kernel<float><<<grid, COPY_THREADS, 0, st>>>(*a, 0);
  else pack_copy_kernel<uint16_t><<<grid, COPY_THREADS, 0, st>>>(*a, vec16);
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}

extern "C" int dkv_decompress(int32_t dtype, int32_t n_arena, int32_t n_tok, int32_t max_dim, const dkv_side* side,
                              void* dense, void* stream) {
  DKV_REQUIRE(side && dense, DKV_E_ARG, "dkv_decompress: null argument");
  DKV_REQUIRE(n_arena >= 0 && n_tok >= 0 && max_dim >= 1, DKV_E_ARG, "dkv_decompress: bad sizes");
  DKV_REQUIRE(n_arena <= 65535, DKV_E_LIMIT, "dkv_decompress: at most 65535 arena rows per call");
  if (int rc = check_side(*side, "dkv_decompress side")) return rc;
  if (n_arena == 0 || n_tok == 0) return DKV_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((n_tok + 7) / 8, n_arena);
  if (dtype == DKV_F32) decompress_kernel<float><<<grid, 256, 0, st>>>(*side, (float*)dense, n_tok, max_dim);
  else if (dtype == DKV_F16) decompress_kernel<__half><<<grid, 256, 0, st>>>(*side, (__half*)dense, n_tok, max_dim);
  else if (dtype == DKV_BF16)
    decompress_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*side, (__nv_bfloat16*)dense, n_tok, max_dim);
  else DKV_REQUIRE(false, DKV_E_ARG, "dkv_decompress: bad dtype %d", dtype);
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}
