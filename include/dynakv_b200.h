/*
 * dynakv_b200 -- C ABI of the B200 (sm_100a) compressed-KV-cache decode path.
 *
 * Every entry point takes plain device pointers, element strides, sizes and a
 * CUDA stream handle; nothing here depends on torch or on C++ types.  All
 * launches are asynchronous on `stream`; no entry point allocates or frees
 * device memory and none synchronises, so a sequence of calls can be captured
 * in a CUDA graph.  Return value: 0 on success, a negative DKV_E_* code when an
 * argument was rejected on the host before any launch (dkv_last_error() then
 * holds a message for the calling thread).  Conditions only the device can see
 * (arena overflow, a length that breaks the declared alignment contract) are
 * recorded in a caller-provided 32-bit status word and never trap.
 *
 * Each declaration names the interface of the reference project that it
 * replaces (file:line inside the reference's source tree).
 */
#ifndef DYNAKV_B200_H_
#define DYNAKV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DKV_VERSION 2

/* element types of cache payload, bases, queries and outputs */
enum { DKV_F32 = 0, DKV_F16 = 1, DKV_BF16 = 2 };

/* host-side error codes */
enum {
  DKV_OK = 0,
  DKV_E_ARG = -1,       /* null pointer / bad size / unsupported shape */
  DKV_E_ALIGN = -2,     /* pointer or stride breaks a documented alignment rule */
  DKV_E_WORKSPACE = -3, /* workspace too small */
  DKV_E_CUDA = -4,      /* the CUDA runtime refused the launch */
  DKV_E_LIMIT = -5      /* size beyond a fixed built-in maximum */
};

/* bits of the device status word */
enum {
  DKV_ST_OVERFLOW = 1,   /* an append/pack would have written past flat capacity or seq capacity; skipped */
  DKV_ST_BAD_LENGTH = 2, /* a length was negative, above max_dim, or not a multiple of the declared step */
  DKV_ST_EMPTY_ROW = 4,  /* attention over a row with no valid token; output written as zeros */
  DKV_ST_TIMEOUT = 8     /* a bounded wait inside a kernel ran out; that call's output is not valid */
};

/* One side (K or V) of one layer's ragged cache.
 * Layout contract (compressed_cache.py:7-34,184-209): for arena row a and token s
 *   lens[a,s] = kept coefficients r_s, offs[a,s] = sum_{t<s} lens[a,t] (elements),
 *   flat[a, offs[a,s] .. +lens[a,s]) = the first r_s coefficients of the token.
 * An "arena row" is a batch row in the reference's joint layout (arenas_per_batch = 1)
 * or a (batch row, KV head) pair in the per-head layout (arenas_per_batch = Hkv);
 * arena index = b * arenas_per_batch + kv_head. */
typedef struct dkv_side {
  void* flat;            /* [n_arena, flat_stride] elements */
  int64_t flat_stride;   /* elements between arena rows (= capacity of a row) */
  int32_t* lens;         /* [n_arena, seq_capacity] view */
  int64_t lens_stride_a; /* elements between arena rows */
  int64_t lens_stride_s; /* elements between tokens */
  int32_t* offs;
  int64_t offs_stride_a;
  int64_t offs_stride_s;
  int32_t* ptr;          /* [n_arena] write pointer = sum of lens (flat_ptr_gpu, compressed_cache.py:126) */
} dkv_side;

/* ---- decode attention -------------------------------------------------- */

typedef struct dkv_attn_args {
  int32_t dtype;            /* DKV_F32 / DKV_F16 / DKV_BF16: q, flat, bases, out */
  int32_t batch;            /* rows processed by this call */
  int32_t n_q_heads;        /* Hq */
  int32_t n_basis_groups;   /* leading dim of k_up/v_up: Hkv or Hq; heads per group = Hq / groups */
  int32_t arenas_per_batch; /* 1 (joint latent row shared by all heads) or Hkv (per-head arenas) */
  int32_t head_dim;         /* D, must be 128 */
  int32_t rank;             /* R = k_up.shape[1], 1..1024 */
  int32_t seq_len;          /* S: tokens (columns of lens/offs) to attend over */
  const void* q;            /* [*, Hq, D], already rotated; D contiguous */
  int64_t q_stride_b, q_stride_h;
  const void* k_up;         /* [groups, R, D] contiguous */
  const void* v_up;
  dkv_side k, v;
  const int32_t* seq_lens;    /* optional [batch rows]: tokens valid per batch row (<= S); NULL = S for all */
  const int32_t* batch_index; /* optional [batch]: which batch rows to process; NULL = 0..batch-1 */
  const float* k_norm_weight; /* optional [D] fp32: RMSNorm of reconstructed K before RoPE (Qwen3) */
  float k_norm_eps;
  float theta;              /* RoPE base */
  int32_t len_multiple;     /* caller's promise: every length is a multiple of this (1 or 8) and rows are
                               gap-free prefix-sum packed; 8 enables the 16-byte-aligned tensor-core path */
  void* out;                /* [*, Hq, D]; D contiguous */
  int64_t out_stride_b, out_stride_h;
  void* workspace;          /* scratch for the split path (see dkv_split_workspace_bytes) */
  size_t workspace_bytes;
  int32_t* status;          /* optional device status word (OR-ed into) */
  int32_t n_sm;             /* SM count of the device, for grid sizing; 0 = query */
  void* stream;             /* cudaStream_t */
  /* Device-side routing (KernelPolicy.select per row, src/dynakv/kernels/router.py:8-17, evaluated on the GPU so
   * that a captured graph keeps routing correctly while sequences grow): a batch row takes part in this call only
   * if  route_min_tokens <= tokens(row)  and ( route_max_tokens == 0 or tokens(row) < route_max_tokens ), with
   * tokens(row) = min(seq_len, seq_lens[row]).  Rows outside are skipped: nothing is written for them and they
   * raise no status bit.  Both 0 = every row (the default). */
  int32_t route_min_tokens;
  int32_t route_max_tokens;
} dkv_attn_args;

/* Short-cache path: one launch that reconstructs K, applies RoPE, runs QK, online softmax and V.
 * Replaces fused_attention_dispatch (src/dynakv/kernels/fused.py:144-170). */
int dkv_fused_decode(const dkv_attn_args* a);

/* Long-cache path: split-KV partial attention into `workspace`, then a combine + V up-projection.
 * Replaces the abx_sparse -> avx pair as the router uses it (src/dynakv/kernels/router.py:50-59,
 * two_stage.py:159-189,283-324). dkv_two_stage_decode = dkv_split_decode then dkv_split_combine. */
size_t dkv_split_workspace_bytes(const dkv_attn_args* a);
int dkv_split_decode(const dkv_attn_args* a);
int dkv_split_combine(const dkv_attn_args* a);
int dkv_two_stage_decode(const dkv_attn_args* a);

/* Long-cache path for callers that cannot allocate device memory.  (No counterpart in the reference.)
 * Same inputs, outputs and results as dkv_two_stage_decode on a cache that qualifies for the split
 * tensor-core path, but `workspace` / `workspace_bytes` are ignored: the per-split partial results go to a
 * 2 MiB array built into the library (each GPU that loads the library holds it until the process ends).
 * Meant for hosts that gave all device memory to their own pool at start-up, or that call from a context
 * where cudaMalloc is forbidden; it calls no allocating routine of CUDA or any library.
 *  - DKV_E_LIMIT when the call needs more scratch than the array holds (the message gives both sizes):
 *    roughly groups * (batch + SMs/groups) * 2080 bytes, i.e. about 100 batch rows with 8 KV heads on a 148-SM GPU;
 *    DKV_E_ARG when the cache does not qualify for the split path (nothing is computed).
 *  - The first call on a device looks the array's address up (cudaGetSymbolAddress); make that first call
 *    outside any stream capture.  Every call sets the kernels' shared-memory attribute (cudaFuncSetAttribute,
 *    a host-side setting that allocates nothing), as dkv_two_stage_decode does.
 *  - All calls on a device share the array.  Nothing in it has to be cleared between calls (every record
 *    that is read was written by the same call), but two calls that overlap on the GPU -- different
 *    streams, or graph branches -- race on it: keep calls on one device ordered. */
int dkv_two_stage_decode_noalloc(const dkv_attn_args* a);

/* Stage 1 of the reference's two-stage path as a standalone op: scaled scores [batch, Hq, S] in the
 * query dtype, tokens of length 0 get -1e4*scale. Replaces abx_sparse (two_stage.py:159-189).
 * `out` is the score tensor; out_stride_b/out_stride_h are its strides, S contiguous. */
int dkv_scores(const dkv_attn_args* a);

/* Stage 2 as a standalone op: softmax over given scores, latent-space V accumulation, up-projection.
 * Replaces avx (two_stage.py:283-324). scores: [batch, Hq, S] in dtype a->dtype, S contiguous. */
int dkv_softmax_v(const dkv_attn_args* a, const void* scores, int64_t sc_stride_b, int64_t sc_stride_h);

/* ---- cache update ------------------------------------------------------ */

typedef struct dkv_append_args {
  int32_t dtype;
  int32_t batch;
  int32_t arenas_per_batch;
  int32_t max_dim;          /* row width of new_k/new_v per arena (R) */
  const void* new_k;        /* [batch, arenas_per_batch, max_dim] contiguous: coefficient rows, or, when
                               k_basis != NULL, pre-RoPE head vectors [batch, arenas_per_batch, D=max_dim] */
  const void* new_v;
  const int32_t* len_k;     /* [batch, arenas_per_batch] kept length r_t per new row */
  const int32_t* len_v;
  const void* k_basis;      /* optional [arenas_per_batch, R, D]: project the row onto the basis first */
  const void* v_basis;
  dkv_side k, v;
  int32_t seq_pos;          /* token index to write when seq_lens == NULL (seq_ptr, compressed_cache.py:131) */
  int32_t* seq_lens;        /* optional [batch]: per-row token count; written at seq_lens[b], then incremented */
  int32_t seq_capacity;     /* columns available in lens/offs */
  int32_t len_multiple;     /* lengths must be multiples of this, else DKV_ST_BAD_LENGTH */
  int32_t* status;
  void* stream;
  int32_t* tickets;         /* optional [batch], zero before the first call and left zero by every call: with it (or
                               with seq_lens == NULL) the projecting append runs one CTA per (arena row, side)
                               instead of one per batch row; the last CTA of a batch row advances seq_lens[b].
                               Calls that share a tickets array must not overlap. */
} dkv_append_args;

/* Decode-step append of one token per arena row, K and V together, all rows in one launch.
 * Replaces update_cache_decode_kernel and its two launches per layer
 * (src/dynakv/kernels/compressed_cache.py:7-34,170-181,222-223). */
int dkv_append_decode(const dkv_append_args* a);

typedef struct dkv_pack_args {
  int32_t dtype;
  int32_t batch;
  int32_t arenas_per_batch;
  int32_t n_new;            /* tokens in the block */
  int32_t max_dim;
  const void* states;       /* element (b, j, s, i) at states[b*stride_b + j*stride_j + s*stride_s + i] */
  int64_t stride_b, stride_j, stride_s;
  const int32_t* new_lens;  /* [batch*arenas_per_batch, n_new] contiguous */
  const int32_t* row_counts; /* optional [batch]: only the first row_counts[b] tokens of row b are stored */
  const int32_t* seq_lens;  /* optional [batch]: first token index of row b (read only); NULL = seq_pos */
  dkv_side side;
  int32_t seq_pos;          /* first token index to write when seq_lens == NULL */
  int32_t seq_capacity;
  int32_t len_multiple;
  int32_t* status;
  void* stream;
} dkv_pack_args;

/* Bulk (prefill) pack of a block of tokens into one side: exclusive scan of the lengths, lens/offs
 * written, kept coefficients copied back to back, write pointer advanced (two kernels on `stream`).
 * An arena row whose new payload would pass flat_stride sets DKV_ST_OVERFLOW, keeps its write pointer and records
 * the block's tokens as empty (lens 0, offs = the write pointer: the rule of dkv_append_decode); a row whose
 * positions would pass seq_capacity sets DKV_ST_OVERFLOW and is not touched at all.
 * Replaces the per-row python loop of _update_layer_cache (compressed_cache.py:184-209). */
int dkv_pack_bulk(const dkv_pack_args* a);

/* Diagnostic, no counterpart in the reference: clock cycles per 128-token tile that the tensor pipe of one SM is
 * held by the decode kernel's tcgen05.mma chains, issued back to back by one thread over zero operands with nothing
 * else running on the SM.  `products` is a mask: 1 = K reconstruction (8 x M128 N128 K16), 2 = scores (8 x M128 N16
 * K16, A in tensor memory), 4 = latent accumulation (8 x M128 N16 K16); 11 = products 1 and 2 from one thread with
 * product 4's chain issued concurrently by a thread of another warp, as the decode kernel does; 23 = all three from
 * one thread with a tcgen05.commit behind every chain (the kernel's four commits per tile); 39 and 43 = 7 and 11
 * over non-zero operands.  Launches n_cta
 * CTAs (one per SM when n_cta <= the SM count) of `tiles` tiles each and writes cycles[c] = elapsed clock64 of CTA c
 * for all its tiles (and, for 11, cycles[n_cta + c] for the second thread: `cycles` holds 2 * n_cta values).
 * The wait for the products is bounded; DKV_ST_TIMEOUT is set in *status when it runs out. */
int dkv_probe_tensor_pipe(int32_t products, int32_t tiles, int32_t n_cta, int64_t* cycles, int32_t* status, void* stream);

/* Bulk (prefill) projection of pre-RoPE rows onto per-head spectral bases on the tensor core:
 *   out[t, h*128 + r] = sum_d x[t, h*128 + d] * basis[h, r, d]        (16-bit in and out, fp32 accumulation).
 * Replaces the one-time fold of the projection into k_proj / v_proj
 * (src/dynakv/kernels/compressed_attention.py:267-275): with per-head 128 x 128 bases the projection is applied to
 * the projection layers' output instead, as a batched 128-wide GEMM over the tokens.  The result is what
 * dkv_pack_bulk takes as `states`. */
typedef struct dkv_project_args {
  int32_t dtype;        /* DKV_F16 / DKV_BF16 */
  int32_t n_tokens;     /* rows of x and out */
  int32_t n_heads;      /* bases; a row holds n_heads * 128 elements */
  const void* x;        /* [n_tokens, n_heads * 128], 16-byte aligned */
  int64_t x_stride;     /* elements between rows, multiple of 8 */
  const void* basis;    /* [n_heads, 128 (r), 128 (d)] contiguous */
  void* out;            /* [n_tokens, n_heads * 128] */
  int64_t out_stride;
  int32_t* status;      /* optional device status word */
  void* stream;
} dkv_project_args;
int dkv_project_bulk(const dkv_project_args* a);

/* Ragged -> dense zero-padded [n_arena, n_tok, max_dim] (contiguous), gathered by offs.
 * Replaces simple_decompress (compressed_cache.py:36-56). */
int dkv_decompress(int32_t dtype, int32_t n_arena, int32_t n_tok, int32_t max_dim, const dkv_side* side,
                   void* dense, void* stream);

/* ---- cutoff gate ------------------------------------------------------- */
/* Kept-coefficient count of token rows: logits = b + x.W, p = softmax(logits), c = cumsum(p),
 * length = #{ i < low_rank : c[dim-1-i] >= threshold } (threshold 0.1 in the reference); optionally the
 * rows with everything past their length zeroed.
 * Replaces kv_process_fused -- src/dynakv/kernels/compressed_attention.py:84-119 (one side, K or V, per call).
 * Arithmetic: sums in fp32.  With native_rounding != 0 and a 16-bit dtype the intermediate tensors are rounded to
 * that dtype where the reference's torch ops materialise them (logits after addmm, probabilities after softmax,
 * every running sum after cumsum, and the threshold itself), so that lengths agree with the reference run in the
 * same dtype; with 0 nothing is rounded (the fp32 result on the stored values).
 * len_multiple > 1 rounds every length UP to that multiple (capped at dim rounded down to it): the kept set is a
 * superset of the gate's, in the form the tensor-core decode kernels take (multiples of 8). */
typedef struct dkv_gate_args {
  int32_t dtype;          /* DKV_F32 / DKV_F16 / DKV_BF16: type of x, w, b, masked */
  int32_t n_rows;         /* token rows */
  int32_t dim;            /* width of a row = rows and columns of w (<= 1024) */
  int32_t low_rank;       /* positions >= low_rank never count */
  float threshold;
  const void* x;          /* [n_rows, dim] */
  int64_t x_stride;       /* elements between rows */
  const void* w;          /* [dim, dim] row-major */
  const void* b;          /* [dim] */
  int32_t* lengths;       /* out [n_rows] */
  void* masked;           /* out [n_rows, dim] or NULL */
  int64_t masked_stride;
  void* workspace;        /* fp32 scratch of dkv_gate_workspace_bytes(args) bytes */
  size_t workspace_bytes;
  void* stream;
  int32_t len_multiple;   /* 0 or 1: exact counts */
  int32_t native_rounding;
} dkv_gate_args;
size_t dkv_gate_workspace_bytes(const dkv_gate_args* args);
int dkv_gate_lengths(const dkv_gate_args* args);

/* The gate for narrow rows (dim <= 128: one row per (sequence, KV head), the decode shape of the per-head layout),
 * K and V sides in ONE launch and without a workspace: same arithmetic, in the same order, as dkv_gate_lengths on
 * each side (kv_process_fused computes both sides in one call too, compressed_attention.py:92-114).  The two
 * argument blocks must agree in dtype, dim, n_rows and stream; workspace fields are ignored. */
int dkv_gate_lengths_pair(const dkv_gate_args* k, const dkv_gate_args* v);

/* ---- misc -------------------------------------------------------------- */
int dkv_version(void);
const char* dkv_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* DYNAKV_B200_H_ */
