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

constexpr int kMaxDevices = 64;  // device ordinals the per-device caches cover

// Ordinal of the current device, or -1 (error set) when it cannot be asked or lies outside the caches.
int current_device();
// Streaming multiprocessors of the current device (asked from the runtime once per device; 148 on a
// B200).  Grids and tile plans are sized from it.
int sm_count();

inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- 16-byte vector access --------------------------------------------------------------------
// One lane always moves 16 bytes of a row: 4 fp32 or 8 bf16 values, widened to fp32 registers.
template <typename T>
struct Vec16;

template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  __device__ __forceinline__ static void load(const float* p, float (&r)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    r[0] = t.x; r[1] = t.y; r[2] = t.z; r[3] = t.w;
  }
  __device__ __forceinline__ static void store(float* p, const float (&r)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
  }
  // Packed form of one 16-byte piece: operands wait in registers in this form until they are used.
  using Raw = float4;
  __device__ __forceinline__ static Raw raw_at(const float* base, unsigned v) {
    return __ldg(reinterpret_cast<const float4*>(base) + v);
  }
  __device__ __forceinline__ static Raw raw_zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ static void unpack(const Raw& t, float (&r)[4]) {
    r[0] = t.x; r[1] = t.y; r[2] = t.z; r[3] = t.w;
  }
  // The same with the position given as a 32-bit index in units of 16 bytes (cheaper addressing).
  __device__ __forceinline__ static void load_at(const float* base, unsigned v, float (&r)[4]) {
    load(reinterpret_cast<const float*>(reinterpret_cast<const float4*>(base) + v), r);
  }
  __device__ __forceinline__ static void store_at(float* base, unsigned v, const float (&r)[4]) {
    store(reinterpret_cast<float*>(reinterpret_cast<float4*>(base) + v), r);
  }
};

template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&r)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // bf16 -> fp32 is a 16-bit left shift of the payload
      r[2 * i] = __uint_as_float(w[i] << 16);
      r[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static void store(__nv_bfloat16* p, const float (&r)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * i], r[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  using Raw = uint4;
  __device__ __forceinline__ static Raw raw_at(const __nv_bfloat16* base, unsigned v) {
    return __ldg(reinterpret_cast<const uint4*>(base) + v);
  }
  __device__ __forceinline__ static Raw raw_zero() { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ static void unpack(const Raw& t, float (&r)[8]) {
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[2 * i] = __uint_as_float(w[i] << 16);
      r[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static void load_at(const __nv_bfloat16* base, unsigned v,
                                                 float (&r)[8]) {
    load(reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const uint4*>(base) + v), r);
  }
  __device__ __forceinline__ static void store_at(__nv_bfloat16* base, unsigned v,
                                                  const float (&r)[8]) {
    store(reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint4*>(base) + v), r);
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
