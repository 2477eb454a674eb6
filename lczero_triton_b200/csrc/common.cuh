// Shared declarations for the sm_100a kernels: status codes, activations, bf16 helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/lc0b200.h"

namespace lc0b200 {

using bf16 = __nv_bfloat16;

// What the host side keeps per device.  Everything here is looked up once per device, with that
// device current, under a mutex (api.cu), so one process may drive several GPUs from several threads.
//   status: device address of four status words on THAT device.  Word 0: first device-side failure
//   code (0 = none); word 1: detail (role / barrier index); word 2: CTA; word 3: parity waited for.
//   Written by kernels whose bounded waits ran out; read and cleared by lc0b200_device_status().
constexpr int kMaxDevices = 64;
struct DeviceInfo {
  int index;
  int sm_count;
  unsigned int* status;
};
// nullptr when the runtime cannot name the current device or its index is out of range.
const DeviceInfo* device_info();
inline unsigned int* device_status_words() {
  const DeviceInfo* d = device_info();
  return d != nullptr ? d->status : nullptr;
}

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

// SM count of the current device.
inline int sm_count() {
  const DeviceInfo* d = device_info();
  return d != nullptr ? d->sm_count : 148;
}

// A kernel's opt-in to more than 48 KB of dynamic shared memory is a per-device attribute: one flag per
// device for each kernel (a static PerDeviceOnce beside the launch).  Racing first calls both set the
// attribute, which is harmless.
struct PerDeviceOnce {
  std::atomic<bool> done[kMaxDevices];
};
template <typename Kernel>
inline int allow_dynamic_smem(PerDeviceOnce& once, Kernel kernel, int bytes) {
  const DeviceInfo* d = device_info();
  if (d == nullptr) return LC0B200_ERR_CUDA;
  if (once.done[d->index].load(std::memory_order_acquire)) return LC0B200_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return LC0B200_ERR_CUDA;
  }
  once.done[d->index].store(true, std::memory_order_release);
  return LC0B200_OK;
}

// Programmatic dependent launch.  A kernel launched through launch_dependent() may be scheduled while the
// kernel before it on the stream is still running: its blocks become resident as soon as every block of the
// predecessor has executed grid_dependency_release() (or exited) and resources are free, and they run up to
// grid_dependency_wait(), which returns once the predecessor grid has COMPLETED and its writes are visible.
// What comes before the wait (launch latency, barrier and tensor-memory set-up, descriptor prefetch) thereby
// overlaps the predecessor's tail.  The rule every kernel here follows: release first, wait before the first
// access to global memory (reads of what the predecessor wrote, and writes the predecessor may still read).
// Waiting chains: kernel N+1 completes only after kernel N has, so data of kernel N-1 is visible too.
// Launched the ordinary way (or after a copy) both instructions return at once.  Stream capture records the
// edge as a programmatic one.  Every kernel of the library follows the rule; launch_dependent() asks for the
// overlap only for grids of at most kMaxDependentBlocks blocks.  A streaming kernel with one small block per
// row has 65536 and more blocks at the large batches, and there the programmatic launch costs more than its
// overlap gives (int8 forward at batch 4096: 5 % slower), while at small batches it is where most of the
// launches are.  LC0B200_PDL=0 compiles the ordinary launches back in (A/B measurements).
#ifndef LC0B200_PDL
#define LC0B200_PDL 1
#endif
__device__ __forceinline__ void grid_dependency_release() {
#if LC0B200_PDL
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void grid_dependency_wait() {
#if LC0B200_PDL
  asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}
constexpr unsigned long long kMaxDependentBlocks = 16384;
inline cudaLaunchAttribute dependent_launch_attribute(bool allowed = true) {
  cudaLaunchAttribute a = {};
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = (LC0B200_PDL && allowed) ? 1 : 0;
  return a;
}
template <typename... Params, typename... Args>
inline void launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t stream,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  const unsigned long long blocks = 1ull * grid.x * grid.y * grid.z;
  cudaLaunchAttribute attribute = dependent_launch_attribute(blocks <= kMaxDependentBlocks);
  cfg.attrs = &attribute;
  cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);  // the error stays in the thread's slot
}

// Status of the `<<<>>>` launch just made by this thread.  cudaGetLastError also CLEARS the thread's
// error slot, so one failed launch is reported once, by the call that made it, and neither by later
// calls of this library nor by the host framework's own launch checks.
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? LC0B200_OK : LC0B200_ERR_CUDA; }

}  // namespace lc0b200
