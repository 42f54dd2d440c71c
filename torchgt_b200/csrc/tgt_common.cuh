// Shared device/host helpers for the torchgt_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/torchgt_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "torchgt_b200 kernels are written for sm_100a (B200) only"
#endif

namespace tgt {

// ---- error reporting (host) -------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);

#define TGT_CHECK_ARG(cond, ...)                               \
  do {                                                         \
    if (!(cond)) return tgt::set_error(TGT_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define TGT_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return tgt::set_error(TGT_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

constexpr int kMaxDevices = 64;  // device ordinals the per-device caches cover

// Ordinal of the current device, or -1 (error set) when it cannot be asked or lies outside the caches.
int current_device();
// Streaming multiprocessors of the current device (asked from the runtime once per device; 148 on a
// B200).  Grids and tile plans are sized from it.
int sm_count();

inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- programmatic dependent launch ----------------------------------------------------------------
// Consecutive kernels of one entry point are chained so that the next kernel's CTAs are placed on an SM as
// soon as the previous kernel's CTAs leave it, and do the part of their prologue that reads nothing the
// previous kernel writes (staging edge indices) while the previous kernel drains.  Every kernel launched
// this way executes dependent_wait() in all its CTAs before it touches such data and before it exits (so
// completion stays transitive along the chain); in a kernel launched the ordinary way both calls do nothing.
int dependent_launch_mask();   // tgt_debug_set_dependent_launch(): bits of the kinds of link that are chained
enum {
  kLinkWalk = 1,         // a walk kernel after the statistics kernel or after another walk kernel
  kLinkStitch = 2,       // the kernel that finishes cross-tile rows after its walk kernel
  kLinkAfterStitch = 4,  // a walk kernel after such a kernel
};

#ifdef __CUDACC__
__device__ __forceinline__ void dependent_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launches kernel<<<grid, block, 0, stream>>>(params); a non-zero `link` (one of the kinds above) marks it as
// the dependent of the kernel enqueued just before it on the stream, which must be one of this library's own.
template <class P>
inline cudaError_t launch_chained(void (*kernel)(const P), dim3 grid, unsigned block, cudaStream_t stream,
                                  int link, const P& params) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (link & dependent_launch_mask()) {
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, params);
}
#endif

// ---- sums of per-CTA partial results -----------------------------------------------------------------
// out[i] = sum over b < n_parts of partial[b * pitch + i] for the 32 consecutive values a block of
// kPartialSumThreads threads owns (i = blockIdx.x * 32 + lane).  Warp w adds the parts w, w + 16, ... with
// eight loads in flight and eight running sums, the sixteen warps' results are added in warp order: the
// association is fixed, so the result does not depend on timing.  Returns the sum in warp 0's lanes.
constexpr int kPartialSumThreads = 512;
#ifdef __CUDACC__
__device__ __forceinline__ float sum_partials(const float* __restrict__ partial, int n_parts, int64_t pitch, int i,
                                              bool live, float (&s_part)[16][32]) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
  if (live) {
    for (int b = warp; b < n_parts; b += 16 * 8) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int bb = b + 16 * j;
        if (bb < n_parts) s[j] += __ldg(partial + int64_t(bb) * pitch + i);
      }
    }
  }
  s_part[warp][lane] = ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]));
  __syncthreads();
  float total = 0.f;
  if (warp == 0) {
#pragma unroll
    for (int w = 0; w < 16; ++w) total += s_part[w][lane];
  }
  return total;
}
#endif

// ---- lane-wide vector access --------------------------------------------------------------------
// One lane moves W bytes of a row, W = 16 (4 fp32 or 8 bf16 values) or 32 (8 fp32 / 16 bf16 values,
// fetched with the 256-bit global loads and stores of sm_100), widened to fp32 registers.
template <typename T, int W>
struct Lane;

template <typename T>
using Vec16 = Lane<T, 16>;

template <>
struct Lane<float, 16> {
  static constexpr int kElems = 4;
  __device__ __forceinline__ static void load(const float* p, float (&r)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    r[0] = t.x; r[1] = t.y; r[2] = t.z; r[3] = t.w;
  }
  __device__ __forceinline__ static void store(float* p, const float (&r)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
  }
  // Packed form of one piece: operands wait in registers in this form until they are used.
  using Raw = float4;
  // The position is a 32-bit index in units of W bytes (cheaper addressing than 64-bit offsets).
  __device__ __forceinline__ static Raw raw_at(const float* base, unsigned v) {
    return __ldg(reinterpret_cast<const float4*>(base) + v);
  }
  __device__ __forceinline__ static Raw raw_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ static void unpack(const Raw& t, float (&r)[4]) {
    r[0] = t.x; r[1] = t.y; r[2] = t.z; r[3] = t.w;
  }
  __device__ __forceinline__ static void store_at(float* base, unsigned v, const float (&r)[4]) {
    store(reinterpret_cast<float*>(reinterpret_cast<float4*>(base) + v), r);
  }
};

// bf16 -> fp32 is a 16-bit left shift of the payload
__device__ __forceinline__ void bf16x2_to_f32(uint32_t w, float& lo, float& hi) {
  lo = __uint_as_float(w << 16);
  hi = __uint_as_float(w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t f32_to_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <>
struct Lane<__nv_bfloat16, 16> {
  static constexpr int kElems = 8;
  __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&r)[8]) {
    unpack(__ldg(reinterpret_cast<const uint4*>(p)), r);
  }
  __device__ __forceinline__ static void store(__nv_bfloat16* p, const float (&r)[8]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(f32_to_bf16x2(r[0], r[1]), f32_to_bf16x2(r[2], r[3]),
                                              f32_to_bf16x2(r[4], r[5]), f32_to_bf16x2(r[6], r[7]));
  }
  using Raw = uint4;
  __device__ __forceinline__ static Raw raw_at(const __nv_bfloat16* base, unsigned v) {
    return __ldg(reinterpret_cast<const uint4*>(base) + v);
  }
  __device__ __forceinline__ static Raw raw_zero() { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ static void unpack(const Raw& t, float (&r)[8]) {
    bf16x2_to_f32(t.x, r[0], r[1]); bf16x2_to_f32(t.y, r[2], r[3]);
    bf16x2_to_f32(t.z, r[4], r[5]); bf16x2_to_f32(t.w, r[6], r[7]);
  }
  __device__ __forceinline__ static void store_at(__nv_bfloat16* base, unsigned v, const float (&r)[8]) {
    store(reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint4*>(base) + v), r);
  }
};

// 32-byte lanes: one 256-bit load per piece (ld.global.nc.v8, sm_100), so a row of 32 bytes — one head
// of 8 fp32 values, the head slice of one rank of an 8-rank run — is one lane, one load, and its dot
// product needs no shuffle.  Addresses must be 32-byte aligned.
struct Raw32 {
  uint32_t w[8];
};
__device__ __forceinline__ Raw32 ld_nc_256(const void* p) {
  Raw32 r;
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]),
                 "=r"(r.w[6]), "=r"(r.w[7])
               : "l"(p));
  return r;
}
__device__ __forceinline__ void st_256(void* p, const Raw32& r) {
  asm volatile("st.global.v8.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};" ::"r"(r.w[0]), "r"(r.w[1]), "r"(r.w[2]),
               "r"(r.w[3]), "r"(r.w[4]), "r"(r.w[5]), "r"(r.w[6]), "r"(r.w[7]), "l"(p)
               : "memory");
}

template <>
struct Lane<float, 32> {
  static constexpr int kElems = 8;
  using Raw = Raw32;
  __device__ __forceinline__ static Raw raw_at(const float* base, unsigned v) {
    return ld_nc_256(reinterpret_cast<const char*>(base) + size_t(v) * 32);
  }
  __device__ __forceinline__ static Raw raw_zero() {
    Raw r;
#pragma unroll
    for (int i = 0; i < 8; ++i) r.w[i] = 0u;
    return r;
  }
  __device__ __forceinline__ static void unpack(const Raw& t, float (&r)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = __uint_as_float(t.w[i]);
  }
  __device__ __forceinline__ static void store_at(float* base, unsigned v, const float (&r)[8]) {
    Raw t;
#pragma unroll
    for (int i = 0; i < 8; ++i) t.w[i] = __float_as_uint(r[i]);
    st_256(reinterpret_cast<char*>(base) + size_t(v) * 32, t);
  }
};

template <>
struct Lane<__nv_bfloat16, 32> {
  static constexpr int kElems = 16;
  using Raw = Raw32;
  __device__ __forceinline__ static Raw raw_at(const __nv_bfloat16* base, unsigned v) {
    return ld_nc_256(reinterpret_cast<const char*>(base) + size_t(v) * 32);
  }
  __device__ __forceinline__ static Raw raw_zero() { return Lane<float, 32>::raw_zero(); }
  __device__ __forceinline__ static void unpack(const Raw& t, float (&r)[16]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) bf16x2_to_f32(t.w[i], r[2 * i], r[2 * i + 1]);
  }
  __device__ __forceinline__ static void store_at(__nv_bfloat16* base, unsigned v, const float (&r)[16]) {
    Raw t;
#pragma unroll
    for (int i = 0; i < 8; ++i) t.w[i] = f32_to_bf16x2(r[2 * i], r[2 * i + 1]);
    st_256(reinterpret_cast<char*>(base) + size_t(v) * 32, t);
  }
};

// Sum over a group of LANES adjacent lanes (LANES a power of two); every lane gets the total.
template <int LANES>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
  for (int off = 1; off < LANES; off <<= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

constexpr float kClampLo = -5.0f;
constexpr float kClampHi = 5.0f;
constexpr float kZEps = 1e-6f;

}  // namespace tgt
