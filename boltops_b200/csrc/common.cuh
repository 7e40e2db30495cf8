// Shared helpers for the boltops_b200 CUDA sources (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/boltops_b200.h"

namespace bolt {

// Records the message returned by bolt_last_error() for this thread.
void set_error(const char* fmt, ...);

#define BOLT_REQUIRE(cond, ...)                 \
  do {                                          \
    if (!(cond)) {                              \
      ::bolt::set_error(__VA_ARGS__);           \
      return BOLT_ERR_INVALID;                  \
    }                                           \
  } while (0)

#define BOLT_CUDA(expr)                                                        \
  do {                                                                         \
    cudaError_t err__ = (expr);                                                \
    if (err__ != cudaSuccess) {                                                \
      ::bolt::set_error("%s failed: %s", #expr, cudaGetErrorString(err__));    \
      return BOLT_ERR_CUDA;                                                    \
    }                                                                          \
  } while (0)

#define BOLT_LAUNCH_CHECK()                                                    \
  do {                                                                         \
    cudaError_t err__ = cudaGetLastError();                                    \
    if (err__ != cudaSuccess) {                                                \
      ::bolt::set_error("kernel launch failed: %s", cudaGetErrorString(err__)); \
      return BOLT_ERR_CUDA;                                                    \
    }                                                                          \
  } while (0)

inline int sm_count_of_current_device() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

__host__ __device__ inline int dtype_bytes(int dt) {
  switch (dt) {
    case BOLT_BF16:
    case BOLT_F16: return 2;
    case BOLT_F32: return 4;
    default: return 1;
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Round a float through the storage type T (used to reproduce per-stage casts).
template <typename T>
__device__ __forceinline__ float round_through(float v) { return to_f32<T>(from_f32<T>(v)); }

// fp32 -> e4m3 (round-to-nearest-even, saturating to +-448) as one byte.
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
// fp32 -> int8: round to nearest even, then saturate (nearbyint + cast).
__device__ __forceinline__ int8_t f32_to_i8(float v) {
  float r = rintf(v);
  r = fminf(fmaxf(r, -128.f), 127.f);
  return (int8_t)(int)r;
}

// 16-byte vector of N elements of T.
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};

// silu(x) = x * (1 / (1 + exp(-x))), the reference kernels' form.
__device__ __forceinline__ float silu_f32(float x) { return x * __frcp_rn(1.0f + expf(-x)); }

}  // namespace bolt
