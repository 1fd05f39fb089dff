// Cutoff gate: how many leading spectral coefficients of a token row are kept.
//   logits = b + x . W ; p = softmax(logits) ; c_j = p_0 + .. + p_j ;
//   length = #{ i < low_rank : c_{d-1-i} >= threshold }          (the kept set is a prefix: c is non-decreasing)
// Reference: kv_process_fused, src/dynakv/kernels/compressed_attention.py:84-119 (one side per call; the
// reference runs K and V rows through one concatenated softmax/cumsum call, which is row-wise anyway).
// Sums are fp32 whatever the storage type; with native_rounding the intermediate tensors are rounded to the storage
// type where the reference's torch ops materialise them.  Two kernels: the logits (8 rows per CTA, so that W is read
// once per 8 rows; the reduction is cut in chunks when there are few rows), then one warp per row for the rest.
#include <math.h>

#include "dkv_common.cuh"

namespace dkv {

constexpr int GATE_ROWS = 8;       // rows per CTA of the logits kernel
constexpr int GATE_MAX_DIM = 1024;
constexpr int GATE_TILE = 128;     // columns per CTA (one per thread) and reduction indices per chunk

// logits, split over column blocks (x), reduction chunks (y) and row tiles (z): part[y][row][col] =
// sum_{i in chunk y} x[row][i] * W[i][col].  fp32, i ascending.  With few rows (decode) the reduction is cut in
// d/128 chunks so that the d x d weight is read by many CTAs at once; the chunks are added in a fixed order by
// the second kernel, so the result does not depend on scheduling.
template <typename T>
__global__ void __launch_bounds__(GATE_TILE) gate_logits_kernel(dkv_gate_args p, int chunk_len, int stage_w) {
  __shared__ float xs[GATE_ROWS][GATE_MAX_DIM];
  extern __shared__ __align__(16) unsigned char gate_wtile[];   // [GATE_TILE][GATE_TILE] of T when stage_w
  const int d = p.dim, tid = threadIdx.x;
  const int col0 = blockIdx.x * GATE_TILE, col = col0 + tid;
  const int i0 = blockIdx.y * chunk_len, i1 = min(i0 + chunk_len, d);
  const int row0 = blockIdx.z * GATE_ROWS;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* w = reinterpret_cast<const T*>(p.w);
  if (stage_w) {
    // the whole 128 x 128 weight tile in one round of 16-byte async copies (one memory round trip instead of
    // one per group of rows); only used when the tile is complete and 16-byte aligned
    constexpr int PER_ROW = GATE_TILE * (int)sizeof(T) / 16;
    for (int e = tid; e < GATE_TILE * PER_ROW; e += GATE_TILE) {
      const int i = e / PER_ROW, c = e - i * PER_ROW;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(gate_wtile + ((size_t)i * GATE_TILE) * sizeof(T) + c * 16);
      const unsigned char* src = reinterpret_cast<const unsigned char*>(w + (size_t)(i0 + i) * d + col0) + c * 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int e = tid; e < GATE_ROWS * (i1 - i0); e += GATE_TILE) {
    const int r = e / (i1 - i0), i = e - r * (i1 - i0);
    xs[r][i] = (row0 + r < p.n_rows) ? to_f32(x[(size_t)(row0 + r) * p.x_stride + i0 + i]) : 0.f;
  }
  if (stage_w) asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  float acc[GATE_ROWS];
#pragma unroll
  for (int r = 0; r < GATE_ROWS; ++r) acc[r] = 0.f;
  if (col < d) {
    if (stage_w) {
      const T* wt = reinterpret_cast<const T*>(gate_wtile);
#pragma unroll 8
      for (int i = 0; i < GATE_TILE; ++i) {
        const float wv = to_f32(wt[i * GATE_TILE + tid]);
#pragma unroll
        for (int r = 0; r < GATE_ROWS; ++r) acc[r] = fmaf(xs[r][i], wv, acc[r]);
      }
    } else {
      int i = i0;
      for (; i + 8 <= i1; i += 8) {
        float wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) wv[u] = to_f32(w[(size_t)(i + u) * d + col]);   // 8 independent loads in flight
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
          for (int r = 0; r < GATE_ROWS; ++r) acc[r] = fmaf(xs[r][i - i0 + u], wv[u], acc[r]);
      }
      for (; i < i1; ++i) {
        const float wv = to_f32(w[(size_t)i * d + col]);
#pragma unroll
        for (int r = 0; r < GATE_ROWS; ++r) acc[r] = fmaf(xs[r][i - i0], wv, acc[r]);
      }
    }
    float* part = reinterpret_cast<float*>(p.workspace) + (size_t)blockIdx.y * p.n_rows * d;
#pragma unroll
    for (int r = 0; r < GATE_ROWS; ++r)
      if (row0 + r < p.n_rows) part[(size_t)(row0 + r) * d + col] = acc[r];
  }
}

// The rest of a row, one warp per row, from its logits (in lg, shared memory) and this lane's partial maximum:
// softmax, running sum, count, optional masked copy.  Shared by the two-kernel path and the single-kernel path for
// narrow rows, so that both do the same arithmetic in the same order.
template <typename T>
__device__ __forceinline__ void gate_finish_row(const dkv_gate_args& p, int row, float* lg, float mx, int lane, bool native,
                                                float thr) {
  const int d = p.dim;
  mx = warp_max(mx);
  float z = 0.f;
  for (int j = lane; j < d; j += 32) {
    const float e = expf(lg[j] - mx);
    lg[j] = e;
    z += e;
  }
  z = warp_sum(z);
  __syncwarp();
  // lane l owns the contiguous columns [l*per, (l+1)*per): local sums, exclusive scan over lanes, then the walk
  const int per = (d + 31) / 32;
  const int j0 = min(lane * per, d), j1 = min(j0 + per, d);
  if (native) {   // softmax writes the probabilities in the storage type
    for (int j = lane; j < d; j += 32) lg[j] = to_f32(from_f32<T>(lg[j] / z));
    z = 1.f;
    __syncwarp();
  }
  float local = 0.f;
  for (int j = j0; j < j1; ++j) local += lg[j] / z;
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  float run = incl - local;
  const int lo = d - min(max(p.low_rank, 0), d);   // only columns >= lo can count
  int cnt = 0;
  for (int j = j0; j < j1; ++j) {
    run += lg[j] / z;
    const float c = native ? to_f32(from_f32<T>(run)) : run;   // cumsum writes every running sum in the storage type
    if (j >= lo && c >= thr) ++cnt;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (p.len_multiple > 1) cnt = min((cnt + p.len_multiple - 1) / p.len_multiple * p.len_multiple, d - d % p.len_multiple);
  if (lane == 0) p.lengths[row] = cnt;
  if (p.masked) {
    const T* x = reinterpret_cast<const T*>(p.x);
    T* out = reinterpret_cast<T*>(p.masked) + (size_t)row * p.masked_stride;
    const T* xr = x + (size_t)row * p.x_stride;
    for (int i = lane; i < d; i += 32) out[i] = i < cnt ? xr[i] : from_f32<T>(0.f);
  }
}

// one warp per row: logits = b + sum of the chunk partials, softmax, running sum, count
template <typename T>
__global__ void __launch_bounds__(256) gate_count_kernel(dkv_gate_args p, int n_chunks) {
  __shared__ float lg_s[8][GATE_MAX_DIM];
  const int d = p.dim, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * 8 + warp;
  if (row >= p.n_rows) return;
  const T* b = reinterpret_cast<const T*>(p.b);
  const bool native = p.native_rounding != 0 && sizeof(T) == 2;
  const float thr = native ? to_f32(from_f32<T>(p.threshold)) : p.threshold;   // the comparison converts the scalar
  const float* part = reinterpret_cast<const float*>(p.workspace);
  float* lg = lg_s[warp];
  float mx = -INFINITY;
  const size_t cstride = (size_t)p.n_rows * d;   // between the partials of consecutive chunks
  for (int jb = lane; jb < d; jb += 32 * 4) {
    // four columns at a time, all their partials loaded before the (fixed-order) additions
    float pv[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = jb + 32 * u;
#pragma unroll
      for (int c = 0; c < 8; ++c) pv[u][c] = (j < d && c < n_chunks) ? part[c * cstride + (size_t)row * d + j] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = jb + 32 * u;
      if (j < d) {
        float v = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) v += pv[u][c];
        v += to_f32(b[j]);
        if (native) v = to_f32(from_f32<T>(v));   // addmm writes the logits in the storage type
        lg[j] = v;
        mx = fmaxf(mx, v);
      }
    }
  }
  gate_finish_row<T>(p, row, lg, mx, lane, native, thr);
}

// Narrow rows (dim <= 128, the per-head decode shape), K and V sides in one launch: blockIdx.y picks the side, a
// CTA takes 8 rows; the logits go straight to shared memory (same fp32 sum, i ascending, as the two-kernel path
// with one reduction chunk), then one warp per row finishes as above.
template <typename T>
__global__ void __launch_bounds__(256) gate_small_kernel(dkv_gate_args pk, dkv_gate_args pv) {
  __shared__ float xs[8][GATE_TILE];
  __shared__ float lg_s[8][GATE_TILE];
  const dkv_gate_args& p = blockIdx.y ? pv : pk;
  const int d = p.dim, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row0 = blockIdx.x * 8;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* w = reinterpret_cast<const T*>(p.w);
  const T* b = reinterpret_cast<const T*>(p.b);
  const bool native = p.native_rounding != 0 && sizeof(T) == 2;
  const float thr = native ? to_f32(from_f32<T>(p.threshold)) : p.threshold;
  for (int e = tid; e < 8 * d; e += 256) {
    const int r = e / d, i = e - r * d;
    xs[r][i] = (row0 + r < p.n_rows) ? to_f32(x[(size_t)(row0 + r) * p.x_stride + i]) : 0.f;
  }
  __syncthreads();
  {
    const int col = tid & (GATE_TILE - 1), rq = (tid >> 7) * 4;   // four rows per thread
    if (col < d) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      int i = 0;
      for (; i + 8 <= d; i += 8) {
        float wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) wv[u] = to_f32(w[(size_t)(i + u) * d + col]);
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[r] = fmaf(xs[rq + r][i + u], wv[u], acc[r]);
      }
      for (; i < d; ++i) {
        const float wv = to_f32(w[(size_t)i * d + col]);
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[r] = fmaf(xs[rq + r][i], wv, acc[r]);
      }
      const float bias = to_f32(b[col]);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float v = acc[r] + bias;
        if (native) v = to_f32(from_f32<T>(v));   // addmm writes the logits in the storage type
        lg_s[rq + r][col] = v;
      }
    }
  }
  __syncthreads();
  const int row = row0 + warp;
  if (row >= p.n_rows) return;
  float* lg = lg_s[warp];
  float mx = -INFINITY;
  for (int j = lane; j < d; j += 32) mx = fmaxf(mx, lg[j]);
  gate_finish_row<T>(p, row, lg, mx, lane, native, thr);
}

static int gate_chunks(const dkv_gate_args* a) {
  // few rows: cut the reduction so that d/128 x d/128 CTAs share the weight read; many rows: the row tiles
  // already fill the GPU
  return a->n_rows <= 64 ? (a->dim + GATE_TILE - 1) / GATE_TILE : 1;   // at most 8 (dim <= 1024)
}

}  // namespace dkv

extern "C" size_t dkv_gate_workspace_bytes(const dkv_gate_args* a) {
  if (a == nullptr || a->n_rows <= 0 || a->dim <= 0) return 0;
  return (size_t)dkv::gate_chunks(a) * (size_t)a->n_rows * (size_t)a->dim * sizeof(float);
}

extern "C" int dkv_gate_lengths(const dkv_gate_args* a) {
  using namespace dkv;
  DKV_REQUIRE(a != nullptr, DKV_E_ARG, "dkv_gate_lengths: null args");
  DKV_REQUIRE(a->dtype >= DKV_F32 && a->dtype <= DKV_BF16, DKV_E_ARG, "dkv_gate_lengths: bad dtype %d", a->dtype);
  DKV_REQUIRE(a->n_rows >= 0 && a->dim >= 1 && a->dim <= GATE_MAX_DIM, DKV_E_LIMIT,
              "dkv_gate_lengths: dim must be in 1..%d, got %d", GATE_MAX_DIM, a->dim);
  DKV_REQUIRE(a->x && a->w && a->b && a->lengths, DKV_E_ARG, "dkv_gate_lengths: null input");
  DKV_REQUIRE(a->x_stride >= a->dim && (!a->masked || a->masked_stride >= a->dim), DKV_E_ARG,
              "dkv_gate_lengths: row strides must be at least dim");
  if (a->n_rows == 0) return DKV_OK;
  DKV_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= dkv_gate_workspace_bytes(a), DKV_E_WORKSPACE,
              "dkv_gate_lengths: workspace too small: need %zu bytes, got %zu", dkv_gate_workspace_bytes(a), a->workspace_bytes);
  DKV_REQUIRE((a->n_rows + GATE_ROWS - 1) / GATE_ROWS <= 65535, DKV_E_LIMIT, "dkv_gate_lengths: at most %d rows per call", 65535 * GATE_ROWS);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  const int n_chunks = gate_chunks(a);
  const int chunk_len = n_chunks == 1 ? a->dim : GATE_TILE;
  dim3 grid((a->dim + GATE_TILE - 1) / GATE_TILE, n_chunks, (a->n_rows + GATE_ROWS - 1) / GATE_ROWS);
  const int cgrid = (a->n_rows + 7) / 8;
  // weight tiles are staged through shared memory when the reduction is chunked and every tile is whole and aligned
  const size_t esz = dtype_size(a->dtype);
  const int stage_w = (n_chunks > 1 && a->dim % GATE_TILE == 0 && ((uintptr_t)a->w & 15) == 0) ? 1 : 0;
  const size_t wsmem = stage_w ? (size_t)GATE_TILE * GATE_TILE * esz : 0;
#define LAUNCH(T)                                                                        \
  do {                                                                                   \
    if (wsmem > 0) /* static 32 KB + the tile exceed the default 48 KB */                \
      cudaFuncSetAttribute(gate_logits_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wsmem); \
    gate_logits_kernel<T><<<grid, GATE_TILE, wsmem, st>>>(*a, chunk_len, stage_w);       \
    gate_count_kernel<T><<<cgrid, 256, 0, st>>>(*a, n_chunks);                           \
  } while (0)
  if (a->dtype == DKV_F32) LAUNCH(float);
  else if (a->dtype == DKV_F16) LAUNCH(__half);
  else LAUNCH(__nv_bfloat16);
#undef LAUNCH
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}

extern "C" int dkv_gate_lengths_pair(const dkv_gate_args* k, const dkv_gate_args* v) {
  using namespace dkv;
  DKV_REQUIRE(k != nullptr && v != nullptr, DKV_E_ARG, "dkv_gate_lengths_pair: null args");
  DKV_REQUIRE(k->dtype == v->dtype && k->dim == v->dim && k->n_rows == v->n_rows && k->stream == v->stream, DKV_E_ARG,
              "dkv_gate_lengths_pair: the two sides must agree in dtype, dim, rows and stream");
  DKV_REQUIRE(k->dtype >= DKV_F32 && k->dtype <= DKV_BF16, DKV_E_ARG, "dkv_gate_lengths_pair: bad dtype %d", k->dtype);
  DKV_REQUIRE(k->n_rows >= 0 && k->dim >= 1 && k->dim <= GATE_TILE, DKV_E_LIMIT,
              "dkv_gate_lengths_pair: dim must be in 1..%d (wider rows: dkv_gate_lengths per side)", GATE_TILE);
  for (const dkv_gate_args* a : {k, v}) {
    DKV_REQUIRE(a->x && a->w && a->b && a->lengths, DKV_E_ARG, "dkv_gate_lengths_pair: null input");
    DKV_REQUIRE(a->x_stride >= a->dim && (!a->masked || a->masked_stride >= a->dim), DKV_E_ARG,
                "dkv_gate_lengths_pair: row strides must be at least dim");
  }
  if (k->n_rows == 0) return DKV_OK;
  DKV_REQUIRE((k->n_rows + 7) / 8 <= 2147483647 / 8, DKV_E_LIMIT, "dkv_gate_lengths_pair: too many rows");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(k->stream);
  const dim3 grid((k->n_rows + 7) / 8, 2);
  if (k->dtype == DKV_F32) gate_small_kernel<float><<<grid, 256, 0, st>>>(*k, *v);
  else if (k->dtype == DKV_F16) gate_small_kernel<__half><<<grid, 256, 0, st>>>(*k, *v);
  else gate_small_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*k, *v);
  DKV_CHECK_LAUNCH();
  return DKV_OK;
}
