// Error reporting, version and layout validation shared by every entry point of the C ABI.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "attn_common.cuh"

namespace tgt {

namespace {
thread_local char g_error[512] = "";
std::atomic<int> g_forced_ge{0};
std::atomic<int> g_lane_mode{0};
// measured on B200: chaining the walk kernels gains 2-5 us per backward call; chaining the kernel that finishes
// cross-tile rows to its walk kernel loses up to 10 us with lane groups of 4, so that link stays ordinary
std::atomic<int> g_dependent_launch{kLinkWalk | kLinkAfterStitch};
}  // namespace

int lane_mode() { return g_lane_mode.load(std::memory_order_relaxed); }
int dependent_launch_mask() { return g_dependent_launch.load(std::memory_order_relaxed); }

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int forced_ge() { return g_forced_ge.load(std::memory_order_relaxed); }

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    set_error(TGT_ERR_UNSUPPORTED, "no current CUDA device with an ordinal below %d", kMaxDevices);
    return -1;
  }
  return dev;
}

int sm_count() {
  static std::atomic<int> cache[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0) return 148;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;
    }
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

int check_layout(const tgt_layout* L, const char* name) {
  if (L == nullptr) return set_error(TGT_ERR_INVALID, "%s is null", name);
  if (L->n_rows < 0 || L->n_edges < 0 || L->n_rows >= (int64_t(1) << 31) - 1 ||
      L->n_edges >= (int64_t(1) << 31) - 1)
    return set_error(TGT_ERR_INVALID, "%s: n_rows/n_edges out of range", name);
  if (L->n_edges > 0 && L->n_rows == 0)
    return set_error(TGT_ERR_INVALID, "%s: edges without rows", name);
  if (L->n_rows > 0 && L->ptr == nullptr) return set_error(TGT_ERR_INVALID, "%s: ptr is null", name);
  if (L->n_edges > 0 && (L->other == nullptr || L->perm == nullptr || L->seg == nullptr))
    return set_error(TGT_ERR_INVALID, "%s: other/perm/seg is null", name);
  return TGT_OK;
}

}  // namespace tgt

extern "C" int tgt_version(void) { return 101; }

extern "C" const char* tgt_last_error(void) { return tgt::g_error; }

extern "C" int tgt_debug_set_tile_edges(int edges_per_lane_group) {
  TGT_CHECK_ARG(edges_per_lane_group >= 0, "edges_per_lane_group must be >= 0");
  tgt::g_forced_ge.store(edges_per_lane_group, std::memory_order_relaxed);
  return TGT_OK;
}

extern "C" int tgt_debug_set_lane_mode(int mode) {
  TGT_CHECK_ARG(mode >= 0 && mode <= 2, "mode must be 0 (library's choice), 1 (16-byte lanes) or 2 (32-byte lanes)");
  tgt::g_lane_mode.store(mode, std::memory_order_relaxed);
  return TGT_OK;
}

extern "C" int tgt_debug_set_dependent_launch(int links) {
  TGT_CHECK_ARG(links >= 0 && links <= 7, "links is a bit mask of 1, 2 and 4");
  tgt::g_dependent_launch.store(links, std::memory_order_relaxed);
  return TGT_OK;
}
