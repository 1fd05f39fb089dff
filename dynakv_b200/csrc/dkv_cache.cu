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

// Bulk (prefill) pack.  One CTA per (block of 512 new tokens, arena row): every CTA sums the row's new lengths itself
// (the part before its block gives its first offset, the whole gives the fits test -- a few KB from L2 against tens
// of KB of payload), writes its tokens' metadata, and copies its payload with 16-byte copies when the layout allows
// (16-bit elements, lengths multiples of 8, aligned bases and strides), element by element otherwise.  A row whose
// block does not fit is flagged and left untouched by all of its CTAs.  The write pointers are read by every CTA, so
// they are advanced by a second, one-thread-per-row kernel behind the copy.
constexpr int PACK_THREADS = 512;

template <int THREADS>
__device__ __forceinline__ int2 block_sum2(int x, int y, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    x += __shfl_xor_sync(0xffffffffu, x, o);
    y += __shfl_xor_sync(0xffffffffu, y, o);
  }
  __syncthreads();
  if (lane == 0) { scratch[2 * warp] = x; scratch[2 * warp + 1] = y; }
  __syncthreads();
  int sx = 0, sy = 0;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) { sx += scratch[2 * w]; sy += scratch[2 * w + 1]; }
  return make_int2(sx, sy);
}

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
__device__ __forceinline__ bool pack_fits(const dkv_pack_args& p, const pack_row& r, int total) {
  return (int64_t)r.base + total <= p.side.flat_stride && r.pos0 >= 0 && r.pos0 + r.n_new <= p.seq_capacity;
}

template <typename T>
__global__ void __launch_bounds__(PACK_THREADS) pack_bulk_kernel(dkv_pack_args p, int vec16) {
  __shared__ int scratch[2 * PACK_THREADS / 32];
  __shared__ int warp_tot[PACK_THREADS / 32];
  const int a = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = a / p.arenas_per_batch, j = a - b * p.arenas_per_batch;
  const dkv_side& sd = p.side;
  const pack_row r = pack_row_of(p, a, b);
  const int s0 = blockIdx.x * PACK_THREADS;
  if (s0 >= r.n_new && s0 > 0) return;
  const int32_t* nl = p.new_lens + (size_t)a * p.n_new;

  // ---- the row's total (fits test) and the part before this block (first offset); bad lengths flagged once
  int before = 0, rest = 0;
  for (int s = tid; s < r.n_new; s += PACK_THREADS) {
    const int len = checked_len(nl[s], p.max_dim, p.len_multiple, blockIdx.x == 0 ? p.status : nullptr, 0);
    if (s < s0) before += len; else rest += len;
  }
  const int2 sums = block_sum2<PACK_THREADS>(before, rest, scratch);
  if (!pack_fits(p, r, sums.x + sums.y)) {
    if (tid == 0 && blockIdx.x == 0) set_status(p.status, DKV_ST_OVERFLOW);
    return;  // metadata, payload and write pointer are left untouched
  }

  // ---- offsets of this block's tokens
  const int s = s0 + tid;
  const int len = s < r.n_new ? checked_len(nl[s], p.max_dim, p.len_multiple, nullptr, 1) : 0;
  int incl = len;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int wbase = 0;
  for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
  const int off = r.base + sums.x + wbase + incl - len;
  if (s < r.n_new) {
    const int pos = r.pos0 + s;
    sd.lens[(size_t)a * sd.lens_stride_a + (size_t)pos * sd.lens_stride_s] = len;
    sd.offs[(size_t)a * sd.offs_stride_a + (size_t)pos * sd.offs_stride_s] = off;
  }

  // ---- payload of this warp's 32 tokens
  const T* st = reinterpret_cast<const T*>(p.states) + (size_t)b * p.stride_b + (size_t)j * p.stride_j;
  T* flat = reinterpret_cast<T*>(sd.flat) + (size_t)a * sd.flat_stride;
  const int half = lane >> 4, hl = lane & 15;
  vec16 = vec16 && (r.base & 7) == 0;    // an arena written earlier with odd lengths falls back to element copies
  if (vec16 && p.max_dim <= 128) {
    // a row is at most 16 pieces of 16 bytes: one piece per lane of a half-warp, four pairs of rows in flight
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 v[4];
      int roff[4];
      bool on[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int li = i + 2 * u + half;
        const int rlen = __shfl_sync(0xffffffffu, len, li);
        roff[u] = __shfl_sync(0xffffffffu, off, li);
        const int rs = s0 + 32 * warp + li;
        on[u] = hl * 8 < rlen;      // rlen is 0 past the end of the block
        if (on[u]) v[u] = __ldcs(reinterpret_cast<const uint4*>(st + (size_t)rs * p.stride_s) + hl);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (on[u]) reinterpret_cast<uint4*>(flat + roff[u])[hl] = v[u];
    }
  } else {
    for (int i = 0; i < 32; i += 2) {
      const int li = i + half;
      const int rlen = __shfl_sync(0xffffffffu, len, li);
      const int roff = __shfl_sync(0xffffffffu, off, li);
      const int rs = s0 + 32 * warp + li;
      if (rlen > 0) {
        const T* src = st + (size_t)rs * p.stride_s;
        T* dst = flat + roff;
        if (vec16) {
          for (int c = hl; c * 8 < rlen; c += 16)
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
        } else {
          for (int e = hl; e < rlen; e += 16) dst[e] = src[e];
        }
      }
    }
  }
}

// Advances the write pointers behind pack_bulk_kernel: one CTA per arena row repeats the sum and the fits test.
__global__ void __launch_bounds__(256) pack_advance_kernel(dkv_pack_args p) {
  __shared__ int scratch[2 * 256 / 32];
  const int a = blockIdx.x;
  const pack_row r = pack_row_of(p, a, a / p.arenas_per_batch);
  const int32_t* nl = p.new_lens + (size_t)a * p.n_new;
  int total = 0;
  for (int s = threadIdx.x; s < r.n_new; s += 256) total += checked_len(nl[s], p.max_dim, p.len_multiple, nullptr, 1);
  const int2 sums = block_sum2<256>(total, 0, scratch);
  if (threadIdx.x == 0 && pack_fits(p, r, sums.x)) p.side.ptr[a] = r.base + sums.x;
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
#define LAUNCH(T)                                                             \
  do {                                                                        \
    if (proj) append_project_kernel<T><<<a->batch, 32 * wpi * items, 0, st>>>(*a, wpi); \
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
  const dim3 grid((unsigned)((a->n_new + PACK_THREADS - 1) / PACK_THREADS), (unsigned)n_arena);
  if (a->dtype == DKV_F32) pack_bulk_kernel<float><<<grid, PACK_THREADS, 0, st>>>(*a, 0);
  else pack_bulk_kernel<uint16_t><<<grid, PACK_THREADS, 0, st>>>(*a, vec16);
  pack_advance_kernel<<<n_arena, 256, 0, st>>>(*a);
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
