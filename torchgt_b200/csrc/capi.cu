// Error reporting, version and layout validation shared by every entry point of the C ABI.
#include <cstdarg>
#include <cstdio>

#include "attn_common.cuh"

namespace tgt {

namespace {
thread_local char g_error[512] = "";
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_layout(const tgt_layout* L, const char* name) {
  if (L == nullptr) return set_error(TGT_ERR_INVALID, "%s is null", name);
  if (L->n_rows < 0 || L->n_edges < 0 || L->n_rows >= (int64_t(1) << 31) - 1 ||
      L->n_edges >= (int64_t(1) << 31) - 1)
    return set_error(TGT_ERR_INVALID, "%s: n_rows/n_edges out of range", name);
  if (L->chunk_edges < 1) return set_error(TGT_ERR_INVALID, "%s: chunk_edges must be >= 1", name);
  if (L->n_chunks < 0 || L->n_hubs < 0 || L->n_hubs > L->n_chunks)
    return set_error(TGT_ERR_INVALID, "%s: inconsistent hub counts", name);
  if (L->n_rows > 0 && L->ptr == nullptr) return set_error(TGT_ERR_INVALID, "%s: ptr is null", name);
  if (L->n_edges > 0 && (L->other == nullptr || L->perm == nullptr))
    return set_error(TGT_ERR_INVALID, "%s: other/perm is null", name);
  if (L->n_chunks > 0 && (L->chunk_row == nullptr || L->chunk_begin == nullptr ||
                          L->hub_row == nullptr || L->hub_chunk_ptr == nullptr))
    return set_error(TGT_ERR_INVALID, "%s: hub arrays are null", name);
  return TGT_OK;
}

}  // namespace tgt

extern "C" int tgt_version(void) { return 100; }

extern "C" const char* tgt_last_error(void) { return tgt::g_error; }
