// Shared declarations for the sm_100a kernels: status codes, activations, bf16 helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lc0b200.h"

namespace lc0b200 {

using bf16 = __nv_bfloat16;

// Device address of four status words.  Word 0: first device-side failure code (0 = none);
// word 1: detail (role / barrier index); word 2: CTA; word 3: parity waited for.  Written by
// kernels whose bounded waits ran out; read and cleared by lc0b200_device_status().
unsigned int* device_status_words();

constexpr unsigned int kDeviceWaitTimeout = 1;
constexpr unsigned int kDeviceSmemMisaligned = 2;  // a kernel found its shared-memory window not 1024-byte aligned

__host__ __device__ inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

// Lc0's activation formulas in fp32.  Mish is the rational form
// e = exp(x); n = e^2 + 2e; q = x / (n + 2); x <= -0.6 ? n*q : x - 2q
// (reference: bt4/kernels/layer_norm.py:61-69), swish is x / (1 + exp(-x)) (:70-71).
__device__ __forceinline__ float act_mish(float x) {
  float e = __expf(x);
  float n = e * e + 2.0f * e;
  float q = __fdividef(x, n + 2.0f);
  return x <= -0.6f ? n * q : x - 2.0f * q;
}

__device__ __forceinline__ float act_swish(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int ACT>
__device__ __forceinline__ float activate(float x) {
  if (ACT == LC0B200_ACT_MISH) return act_mish(x);
  if (ACT == LC0B200_ACT_RELU) return fmaxf(x, 0.0f);
  if (ACT == LC0B200_ACT_SWISH) return act_swish(x);
  return x;
}

__device__ __forceinline__ float activate_rt(float x, int act) {
  switch (act) {
    case LC0B200_ACT_MISH: return act_mish(x);
    case LC0B200_ACT_RELU: return fmaxf(x, 0.0f);
    case LC0B200_ACT_SWISH: return act_swish(x);
    default: return x;
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(b);
}

// Four values times `inv`, rounded half-to-even and packed as int8 (low byte first).  The saturating
// conversion clamps to [-128, 127]; callers pass inv = 127 / max|x|, so that |x * inv| <= 127 and the
// result lies in [-127, 127] as the symmetric quantiser defines it.
__device__ __forceinline__ uint32_t quantize4_s8(float a, float b, float c, float d, float inv) {
  int q0, q1, q2, q3;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(a * inv));
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(b * inv));
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q2) : "f"(c * inv));
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q3) : "f"(d * inv));
  const uint32_t lo = __byte_perm(static_cast<uint32_t>(q0), static_cast<uint32_t>(q1), 0x0040);
  const uint32_t hi = __byte_perm(static_cast<uint32_t>(q2), static_cast<uint32_t>(q3), 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached = n;
  }
  return cached;
}

inline int launch_status() { return cudaPeekAtLastError() == cudaSuccess ? LC0B200_OK : LC0B200_ERR_CUDA; }

}  // namespace lc0b200
