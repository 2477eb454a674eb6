// Policy-head tail kernels.
//   promotion_logits: bt4/kernels/promotion_logits.py:67-145
//   policy_tail: promotion logits + gather (bt4/kernels/policy_map.py:28-49) + f32 widening
//                (bt4/kernels/copy_type_converted.py:26-34) in one pass over the record.
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lc0b200 {

namespace {

constexpr int kRecord = 4288;
constexpr int kPromoStart = 4096;

// offsets[t][c] = keys[b, 56+t, :] . (W[:, c] + W[:, 3]) for t in 0..7, c in 0..2; one warp per t.
__device__ __forceinline__ void promotion_offsets(float (&dst)[3], const bf16* key_row, const bf16* w, int width,
                                                  int lane) {
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = lane; k < width; k += 32) {
    const float x = __bfloat162float(key_row[k]);
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[c] = fmaf(x, __bfloat162float(w[k * 4 + c]), acc[c]);
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[c] += __shfl_xor_sync(0xFFFFFFFFu, acc[c], o);
  }
  dst[0] = acc[0] + acc[3];
  dst[1] = acc[1] + acc[3];
  dst[2] = acc[2] + acc[3];
}

// One CTA (8 warps) per position.
__device__ __forceinline__ void promotion_logits_body(bf16* records, const bf16* __restrict__ keys,
                                                      const bf16* __restrict__ w, int width) {
  __shared__ float offs[8][3];
  const long long b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float o[3];
  promotion_offsets(o, keys + (b * 64 + 56 + warp) * width, w, width, lane);
  if (lane == 0) { offs[warp][0] = o[0]; offs[warp][1] = o[1]; offs[warp][2] = o[2]; }
  __syncthreads();
  bf16* rec = records + b * kRecord;
  if (threadIdx.x < 192) {
    const int s = threadIdx.x / 24, t = (threadIdx.x % 24) / 3, c = threadIdx.x % 3;
    const float qk = __bfloat162float(rec[(48 + s) * 64 + 56 + t]);
    rec[kPromoStart + threadIdx.x] = __float2bfloat16_rn(qk + offs[t][c]);
  }
}
__global__ void __launch_bounds__(256) promotion_logits_kernel(bf16* records, const bf16* __restrict__ keys,
                                                               const bf16* __restrict__ w, int width) {
  grid_dependency_release();
  grid_dependency_wait();
  promotion_logits_body(records, keys, w, width);
}

__global__ void __launch_bounds__(256) policy_tail_kernel(float* __restrict__ out, const bf16* __restrict__ records,
                                                          const bf16* __restrict__ keys, const bf16* __restrict__ w,
                                                          const int32_t* __restrict__ table, int width) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ float offs[8][3];
  const long long b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float o[3];
  promotion_offsets(o, keys + (b * 64 + 56 + warp) * width, w, width, lane);
  if (lane == 0) { offs[warp][0] = o[0]; offs[warp][1] = o[1]; offs[warp][2] = o[2]; }
  __syncthreads();
  const bf16* rec = records + b * kRecord;
  for (int i = threadIdx.x; i < 1858; i += 256) {
    const int src = table[i];
    float v = 0.0f;
    if (src >= 0 && src < kPromoStart) {
      v = __bfloat162float(rec[src]);
    } else if (src >= kPromoStart && src < kRecord) {
      const int j = src - kPromoStart;
      const int s = j / 24, t = (j % 24) / 3, c = j % 3;
      // Same rounding point as the unfused path: the promotion logit is a 16-bit record entry.
      v = __bfloat162float(__float2bfloat16_rn(__bfloat162float(rec[(48 + s) * 64 + 56 + t]) + offs[t][c]));
    }
    out[b * 1858 + i] = v;
  }
}

// Output probabilities: WDL softmax, (Q, D) = (W - L, D), and policy softmax over the legal moves, one CTA
// per position.
__global__ void __launch_bounds__(256) output_probabilities_kernel(float* __restrict__ policy_probs,
                                                                   float* __restrict__ wdl_probs,
                                                                   float* __restrict__ q_d,
                                                                   const float* __restrict__ policy_logits,
                                                                   const float* __restrict__ wdl_logits,
                                                                   const uint8_t* __restrict__ legal, int policy_size) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ float red[8];
  __shared__ float bcast;
  const long long b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if ((wdl_probs != nullptr || q_d != nullptr) && threadIdx.x == 0) {
    const float w = wdl_logits[b * 3], d = wdl_logits[b * 3 + 1], l = wdl_logits[b * 3 + 2];
    const float m = fmaxf(w, fmaxf(d, l));
    const float ew = expf(w - m), ed = expf(d - m), el = expf(l - m);
    const float inv = 1.0f / (ew + ed + el);
    if (wdl_probs != nullptr) {
      wdl_probs[b * 3] = ew * inv;
      wdl_probs[b * 3 + 1] = ed * inv;
      wdl_probs[b * 3 + 2] = el * inv;
    }
    if (q_d != nullptr) {
      q_d[b * 2] = ew * inv - el * inv;
      q_d[b * 2 + 1] = ed * inv;
    }
  }
  if (policy_probs == nullptr) return;
  const float* logits = policy_logits + b * policy_size;
  const uint8_t* mask = legal != nullptr ? legal + b * policy_size : nullptr;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < policy_size; i += 256) {
    if (mask == nullptr || mask[i] != 0) mx = fmaxf(mx, logits[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    bcast = m;
  }
  __syncthreads();
  mx = bcast;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < policy_size; i += 256) {
    if (mask == nullptr || mask[i] != 0) sum += expf(logits[i] - mx);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    for (int w = 0; w < 8; ++w) t += red[w];
    bcast = t > 0.0f ? 1.0f / t : 0.0f;
  }
  __syncthreads();
  const float inv = bcast;
  for (int i = threadIdx.x; i < policy_size; i += 256) {
    const bool on = mask == nullptr || mask[i] != 0;
    policy_probs[b * policy_size + i] = (on && inv > 0.0f) ? expf(logits[i] - mx) * inv : 0.0f;
  }
}

}  // namespace

int output_probabilities(float* policy_probs, float* wdl_probs, float* q_d, const float* policy_logits,
                         const float* wdl_logits, const uint8_t* legal, int batch, int policy_size, cudaStream_t st) {
  launch_dependent(output_probabilities_kernel, dim3(batch), dim3(256), 0, st, policy_probs, wdl_probs, q_d, policy_logits, wdl_logits, legal,
                                                     policy_size);
  return launch_status();
}

int promotion_logits(void* records, const void* keys, const void* w, int batch, int width, cudaStream_t st) {
  launch_dependent(promotion_logits_kernel, dim3(batch), dim3(256), 0, st, reinterpret_cast<bf16*>(records), reinterpret_cast<const bf16*>(keys),
                                                 reinterpret_cast<const bf16*>(w), width);
  return launch_status();
}

int policy_tail(float* out, const void* records, const void* keys, const void* w, const int32_t* table, int batch,
                int width, cudaStream_t st) {
  launch_dependent(policy_tail_kernel, dim3(batch), dim3(256), 0, st, out, reinterpret_cast<const bf16*>(records),
                                            reinterpret_cast<const bf16*>(keys), reinterpret_cast<const bf16*>(w),
                                            table, width);
  return launch_status();
}

}  // namespace lc0b200
