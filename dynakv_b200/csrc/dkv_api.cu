// C-ABI entry points of the decode-attention paths and library-wide helpers.
#include <stdarg.h>
#include <string.h>

#include "dkv_common.cuh"

namespace dkv {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// implemented in dkv_generic.cu / dkv_mma_decode.cu
int check_attn_args(const dkv_attn_args* a, const char* who, bool need_q, bool need_k, bool need_v);
int generic_attention(const dkv_attn_args* a);
int generic_two_stage(const dkv_attn_args* a);
size_t generic_split_workspace_bytes(const dkv_attn_args* a);
bool mma_path_ok(const dkv_attn_args* a);
size_t mma_split_workspace_bytes(const dkv_attn_args* a);
int mma_fused(const dkv_attn_args* a);
int mma_split(const dkv_attn_args* a);
int mma_combine(const dkv_attn_args* a);
int mma_two_stage_noalloc(const dkv_attn_args* a);

}  // namespace dkv

using namespace dkv;

extern "C" int dkv_version(void) { return DKV_VERSION; }

extern "C" const char* dkv_last_error(void) { return g_err; }

extern "C" int dkv_fused_decode(const dkv_attn_args* a) {
  if (int rc = check_attn_args(a, "dkv_fused_decode", true, true, true)) return rc;
  if (mma_path_ok(a)) return mma_fused(a);
  return generic_attention(a);
}

extern "C" size_t dkv_split_workspace_bytes(const dkv_attn_args* a) {
  if (a == nullptr) return 0;
  if (!mma_path_ok(a)) return generic_split_workspace_bytes(a);
  return mma_split_workspace_bytes(a);
}

extern "C" int dkv_split_decode(const dkv_attn_args* a) {
  if (int rc = check_attn_args(a, "dkv_split_decode", true, true, true)) return rc;
  DKV_REQUIRE(mma_path_ok(a), DKV_E_ARG,
              "dkv_split_decode: needs 16-bit elements, per-KV-head arenas, rank <= 128, lengths declared as "
              "multiples of 8 and 16-byte aligned arena rows; use dkv_two_stage_decode for other caches");
  return mma_split(a);
}

extern "C" int dkv_split_combine(const dkv_attn_args* a) {
  if (int rc = check_attn_args(a, "dkv_split_combine", false, false, false)) return rc;
  DKV_REQUIRE(a->v_up != nullptr, DKV_E_ARG, "dkv_split_combine: null v_up");
  DKV_REQUIRE(mma_path_ok(a), DKV_E_ARG, "dkv_split_combine: arguments do not describe a split-path call");
  return mma_combine(a);
}

extern "C" int dkv_two_stage_decode(const dkv_attn_args* a) {
  if (int rc = check_attn_args(a, "dkv_two_stage_decode", true, true, true)) return rc;
  if (!mma_path_ok(a)) return generic_two_stage(a);
  if (int rc = mma_split(a)) return rc;
  return mma_combine(a);
}

extern "C" int dkv_two_stage_decode_noalloc(const dkv_attn_args* a) {
  if (int rc = check_attn_args(a, "dkv_two_stage_decode_noalloc", true, true, true)) return rc;
  return mma_two_stage_noalloc(a);
}
