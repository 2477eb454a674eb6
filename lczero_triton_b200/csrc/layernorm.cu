// LayerNorm with the reference's fused prologue (bt4/kernels/layer_norm.py:37-161):
//   v = act(x + bias); if has_skip: v = alpha * v + skip
//   y = (v - mean) / sqrt(var + eps) * gamma + beta     (population variance, centred, fp32)
// HBM-bound: each row is read once and kept on chip.  Rows up to 2048 wide are held in the
// registers of ONE warp (warp-shuffle reductions, no shared memory, no block barrier); wider
// rows (smolgen's 8192-wide LN) use one CTA per row with the row cached in shared memory.
// The narrow kernel can also emit the per-row int8 quantisation of its result for the
// int8 GEMM that consumes it.
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lc0b200 {

namespace {

constexpr int kWarpsPerBlock = 2;  // measured: 2 beats 4 and 8 by 2-7 % on every row kernel here (more CTAs in flight, shorter tail)
constexpr int kMaxGroups = 8;  // 16-byte groups of 8 channels per lane: 32 lanes x 8 x 8 = 2048 channels

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  float2 t;
  t = unpack_bf16x2(raw.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16x2(raw.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16x2(raw.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16x2(raw.w); f[6] = t.x; f[7] = t.y;
}

struct LnParams {
  bf16* out;
  const bf16* in;
  const bf16* bias;
  const bf16* skip;
  const bf16* gamma;
  const bf16* beta;
  const bf16* alpha;
  int8_t* q_out;
  float* q_scale;
  long long rows;
  int width;
  int activation;
  int has_skip;
  float epsilon;
};

// One warp per row; GROUPS = ceil(width / 256) register groups per lane.  ACT / SKIP / QUANT fix the
// activation, the presence of the skip operand and of the int8 output at compile time (-1 = decided at run
// time from the parameters): the kernel is a stream of 16-byte loads and a few dozen instructions per
// element, and with everything decided per element at run time it issued instructions for 54 % of its
// cycles and reached two thirds of the memory bandwidth.  The combinations the forward pass uses are
// instantiated; anything else takes the run-time form.  All loads of a row are issued before any
// arithmetic.  The body is a device function so that a pointer-only entry point with baked shapes can
// wrap it too (lc0ex_bridge.py).
template <int GROUPS, int ACT, int SKIP, int QUANT>
__device__ __forceinline__ void layer_norm_warp_body(const LnParams& p) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * static_cast<long long>(kWarpsPerBlock) + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const bool has_skip = SKIP < 0 ? p.has_skip != 0 : SKIP != 0;
  const bool quant = QUANT < 0 ? p.q_out != nullptr : QUANT != 0;
  const int groups = p.width >> 3;
  const uint4* in = reinterpret_cast<const uint4*>(p.in + row * p.width);
  const uint4* skip = reinterpret_cast<const uint4*>(p.skip + row * p.width);
  const uint4* bias = reinterpret_cast<const uint4*>(p.bias);

  uint4 raw_in[GROUPS], raw_skip[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = lane + 32 * g;
    raw_in[g] = make_uint4(0u, 0u, 0u, 0u);
    raw_skip[g] = make_uint4(0u, 0u, 0u, 0u);
    if (idx < groups) {
      raw_in[g] = in[idx];
      if (has_skip) raw_skip[g] = skip[idx];
    }
  }
  const float alpha = has_skip ? __bfloat162float(*p.alpha) : 1.0f;

  float v[GROUPS][8];
  float sum = 0.0f;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = lane + 32 * g;
    if (idx < groups) {
      float x[8], b[8], s[8];
      unpack8(raw_in[g], x);
      unpack8(__ldg(bias + idx), b);
      unpack8(raw_skip[g], s);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = x[j] + b[j];
        t = ACT < 0 ? activate_rt(t, p.activation) : activate<(ACT < 0 ? 0 : ACT)>(t);
        if (has_skip) t = alpha * t + s[j];
        v[g][j] = t;
        sum += t;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[g][j] = 0.0f;
    }
  }
  const float inv_width = 1.0f / static_cast<float>(p.width);
  const float mean = warp_sum(sum) * inv_width;
  float sq = 0.0f;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    if (lane + 32 * g < groups) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = v[g][j] - mean;
        v[g][j] = c;
        sq += c * c;
      }
    }
  }
  const float var = warp_sum(sq) * inv_width;
  const float rstd = 1.0f / sqrtf(var + p.epsilon);

  const uint4* gamma = reinterpret_cast<const uint4*>(p.gamma);
  const uint4* beta = reinterpret_cast<const uint4*>(p.beta);
  uint4* out = reinterpret_cast<uint4*>(p.out + row * p.width);
  float amax = 0.0f;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = lane + 32 * g;
    if (idx < groups) {
      float ga[8], be[8];
      unpack8(__ldg(gamma + idx), ga);
      unpack8(__ldg(beta + idx), be);
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float y0 = v[g][2 * j] * rstd * ga[2 * j] + be[2 * j];
        const float y1 = v[g][2 * j + 1] * rstd * ga[2 * j + 1] + be[2 * j + 1];
        w[j] = pack_bf16x2(y0, y1);
        if (quant) {
          // Keep the bf16-rounded result: the quantiser below must see what is stored.
          const float2 r = unpack_bf16x2(w[j]);
          v[g][2 * j] = r.x;
          v[g][2 * j + 1] = r.y;
          amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
        }
      }
      if (p.out != nullptr) out[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (quant) {
    amax = warp_max(amax);
    const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 1.0f;
    if (lane == 0) p.q_scale[row] = s;
    uint2* qdst = reinterpret_cast<uint2*>(p.q_out + row * p.width);
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const int idx = lane + 32 * g;
      if (idx < groups) {
        qdst[idx] = make_uint2(quantize4_s8(v[g][0], v[g][1], v[g][2], v[g][3], inv),
                               quantize4_s8(v[g][4], v[g][5], v[g][6], v[g][7], inv));
      }
    }
  }
}

template <int GROUPS, int ACT, int SKIP, int QUANT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layer_norm_warp_kernel(const LnParams p) {
  grid_dependency_release();
  grid_dependency_wait();
  layer_norm_warp_body<GROUPS, ACT, SKIP, QUANT>(p);
}

// One CTA per row, row cached in shared memory as fp32 (any width, any alignment).
__global__ void __launch_bounds__(256) layer_norm_block_kernel(const LnParams p) {
  grid_dependency_release();
  grid_dependency_wait();
  extern __shared__ float row_cache[];
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16* in = p.in + row * p.width;
  const bf16* skip = p.has_skip ? p.skip + row * p.width : nullptr;
  const float alpha = p.has_skip ? __bfloat162float(*p.alpha) : 1.0f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  auto block_sum = [&](float x) -> float {
    x = warp_sum(x);
    __syncthreads();
    if (lane == 0) red[warp] = x;
    __syncthreads();
    float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.0f;
    if (warp == 0) {
      t = warp_sum(t);
      if (lane == 0) red[0] = t;
    }
    __syncthreads();
    return red[0];
  };

  float sum = 0.0f;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    float t = activate_rt(__bfloat162float(in[c]) + __bfloat162float(p.bias[c]), p.activation);
    if (p.has_skip) t = alpha * t + __bfloat162float(skip[c]);
    row_cache[c] = t;
    sum += t;
  }
  const float mean = block_sum(sum) / static_cast<float>(p.width);
  float sq = 0.0f;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    const float d = row_cache[c] - mean;
    sq += d * d;
  }
  const float var = block_sum(sq) / static_cast<float>(p.width);
  const float rstd = 1.0f / sqrtf(var + p.epsilon);
  bf16* out = p.out + row * p.width;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    const float y = (row_cache[c] - mean) * rstd * __bfloat162float(p.gamma[c]) + __bfloat162float(p.beta[c]);
    out[c] = __float2bfloat16_rn(y);
  }
}

// Wide rows (the 8192-wide smolgen LayerNorm): one CTA of 256 threads per row, the row held in
// registers as GROUPS 16-byte groups per thread, two block reductions through shared memory.  ACT / SKIP as in
// the one-warp kernel: fixed at compile time for what the forward pass runs (swish, no skip), -1 = run time.
template <int GROUPS, int ACT, int SKIP>
__global__ void __launch_bounds__(256) layer_norm_wide_kernel(const LnParams p) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ float red[2][8];
  const long long row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = p.width >> 3;
  const bool has_skip = SKIP < 0 ? p.has_skip != 0 : SKIP != 0;
  const uint4* in = reinterpret_cast<const uint4*>(p.in + row * p.width);
  const uint4* skip = reinterpret_cast<const uint4*>(p.skip + row * p.width);
  const uint4* bias = reinterpret_cast<const uint4*>(p.bias);
  uint4 raw_in[GROUPS], raw_skip[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {  // every load of the row before any arithmetic
    const int idx = threadIdx.x + 256 * g;
    raw_in[g] = make_uint4(0u, 0u, 0u, 0u);
    raw_skip[g] = make_uint4(0u, 0u, 0u, 0u);
    if (idx < groups) {
      raw_in[g] = in[idx];
      if (has_skip) raw_skip[g] = skip[idx];
    }
  }
  const float alpha = has_skip ? __bfloat162float(*p.alpha) : 1.0f;
  float v[GROUPS][8];
  float sum = 0.0f;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = threadIdx.x + 256 * g;
    if (idx < groups) {
      float x[8], b[8], s[8];
      unpack8(raw_in[g], x);
      unpack8(__ldg(bias + idx), b);
      unpack8(raw_skip[g], s);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = x[j] + b[j];
        t = ACT < 0 ? activate_rt(t, p.activation) : activate<(ACT < 0 ? 0 : ACT)>(t);
        if (has_skip) t = alpha * t + s[j];
        v[g][j] = t;
        sum += t;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[g][j] = 0.0f;
    }
  }
  sum = warp_sum(sum);
  if (lane == 0) red[0][warp] = sum;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += red[0][w];
  const float inv_width = 1.0f / static_cast<float>(p.width);
  const float mean = total * inv_width;
  float sq = 0.0f;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    if (threadIdx.x + 256 * g < groups) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = v[g][j] - mean;
        v[g][j] = c;
        sq += c * c;
      }
    }
  }
  sq = warp_sum(sq);
  if (lane == 0) red[1][warp] = sq;
  __syncthreads();
  float total_sq = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total_sq += red[1][w];
  const float rstd = 1.0f / sqrtf(total_sq * inv_width + p.epsilon);
  const uint4* gamma = reinterpret_cast<const uint4*>(p.gamma);
  const uint4* beta = reinterpret_cast<const uint4*>(p.beta);
  uint4* out = reinterpret_cast<uint4*>(p.out + row * p.width);
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = threadIdx.x + 256 * g;
    if (idx < groups) {
      float ga[8], be[8];
      unpack8(__ldg(gamma + idx), ga);
      unpack8(__ldg(beta + idx), be);
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        w[j] = pack_bf16x2(v[g][2 * j] * rstd * ga[2 * j] + be[2 * j],
                           v[g][2 * j + 1] * rstd * ga[2 * j + 1] + be[2 * j + 1]);
      }
      out[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

template <int GROUPS>
int launch_warp(const LnParams& p, cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>(ceil_div_ll(p.rows, kWarpsPerBlock));
  constexpr int kThreads = kWarpsPerBlock * 32;
  const bool quant = p.q_out != nullptr;
  // The combinations the forward pass runs, decided at compile time; the rest at run time.
  if (p.activation == LC0B200_ACT_NONE && p.has_skip && !quant) {
    launch_dependent(layer_norm_warp_kernel<GROUPS, LC0B200_ACT_NONE, 1, 0>, dim3(blocks), dim3(kThreads), 0, st, p);
  } else if (p.activation == LC0B200_ACT_NONE && p.has_skip && quant) {
    launch_dependent(layer_norm_warp_kernel<GROUPS, LC0B200_ACT_NONE, 1, 1>, dim3(blocks), dim3(kThreads), 0, st, p);
  } else if (p.activation == LC0B200_ACT_NONE && !p.has_skip && !quant) {
    launch_dependent(layer_norm_warp_kernel<GROUPS, LC0B200_ACT_NONE, 0, 0>, dim3(blocks), dim3(kThreads), 0, st, p);
  } else if (p.activation == LC0B200_ACT_MISH && !p.has_skip && !quant) {
    launch_dependent(layer_norm_warp_kernel<GROUPS, LC0B200_ACT_MISH, 0, 0>, dim3(blocks), dim3(kThreads), 0, st, p);
  } else if (p.activation == LC0B200_ACT_SWISH && !p.has_skip && !quant) {
    launch_dependent(layer_norm_warp_kernel<GROUPS, LC0B200_ACT_SWISH, 0, 0>, dim3(blocks), dim3(kThreads), 0, st, p);
  } else {
    launch_dependent(layer_norm_warp_kernel<GROUPS, -1, -1, -1>, dim3(blocks), dim3(kThreads), 0, st, p);
  }
  return launch_status();
}

// Deferred-LayerNorm rows straight to per-row int8: y = (z - mean) * rstd * gamma + beta with mean / rstd
// from the partial row sums a residual GEMM wrote (lc0b200_gemm_args::stats_out), rounded to bf16 (what a
// LayerNorm kernel would have stored), then s = max|y| / 127, q = rint(y * (127 / max|y|)).  One warp per
// row, the row in registers between the two passes; nothing but z is read at full width.
template <int GROUPS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
normalize_quantize_kernel(int8_t* __restrict__ q_out, float* __restrict__ q_scale, const bf16* __restrict__ z,
                          const float2* __restrict__ stats, int parts, const bf16* __restrict__ gamma,
                          const bf16* __restrict__ beta, long long rows, int width, float epsilon) {
  grid_dependency_release();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * static_cast<long long>(kWarpsPerBlock) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int groups = width >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(z + row * width);
  // The row first (its loads are in flight while the statistics arrive: one memory round trip, not two).
  uint4 raw[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = lane + 32 * g;
    raw[g] = idx < groups ? __ldg(src + idx) : make_uint4(0u, 0u, 0u, 0u);
  }
  // mean and 1/sqrt(var + eps) from the partials (lanes share the loads, a shuffle sums them)
  float s = 0.0f, q = 0.0f;
  for (int i = lane; i < parts; i += 32) {
    const float2 t = __ldg(stats + static_cast<long long>(i) * rows + row);
    s += t.x;
    q += t.y;
  }
  s = warp_sum(s);
  q = warp_sum(q);
  const float inv_width = 1.0f / static_cast<float>(width);
  const float mean = s * inv_width;
  const float rstd = rsqrtf(fmaxf(q * inv_width - mean * mean, 0.0f) + epsilon);
  const float shift = -mean * rstd;
  float y[GROUPS][8];
  float amax = 0.0f;
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = lane + 32 * g;
    if (idx < groups) {
      float v[8], ga[8], be[8];
      unpack8(raw[g], v);
      unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + idx), ga);
      unpack8(__ldg(reinterpret_cast<const uint4*>(beta) + idx), be);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float y0 = fmaf(fmaf(v[2 * j], rstd, shift), ga[2 * j], be[2 * j]);
        const float y1 = fmaf(fmaf(v[2 * j + 1], rstd, shift), ga[2 * j + 1], be[2 * j + 1]);
        const float2 r = unpack_bf16x2(pack_bf16x2(y0, y1));  // the quantiser sees bf16 values
        y[g][2 * j] = r.x;
        y[g][2 * j + 1] = r.y;
        amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
      }
    }
  }
  amax = warp_max(amax);
  const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 1.0f;
  if (lane == 0) q_scale[row] = scale;
  uint2* dst = reinterpret_cast<uint2*>(q_out + row * width);
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int idx = lane + 32 * g;
    if (idx < groups) {
      dst[idx] = make_uint2(quantize4_s8(y[g][0], y[g][1], y[g][2], y[g][3], inv),
                            quantize4_s8(y[g][4], y[g][5], y[g][6], y[g][7], inv));
    }
  }
}

}  // namespace

int normalize_quantize_rows(void* q_out, float* q_scale, const void* z, const float* stats, int parts, const void* gamma,
                            const void* beta, long long rows, int width, float epsilon, cudaStream_t st) {
  if (rows == 0) return LC0B200_OK;
  if ((width % 8) != 0 || width > 256 * kMaxGroups) return LC0B200_ERR_UNSUPPORTED;
  if (!aligned16(q_out) || !aligned16(z) || !aligned16(gamma) || !aligned16(beta) || (reinterpret_cast<uintptr_t>(stats) & 7u)) {
    return LC0B200_ERR_MISALIGNED;
  }
  const unsigned blocks = static_cast<unsigned>(ceil_div_ll(rows, kWarpsPerBlock));
  const dim3 block(kWarpsPerBlock * 32);
  auto* qo = reinterpret_cast<int8_t*>(q_out);
  const auto* zz = reinterpret_cast<const bf16*>(z);
  const auto* st2 = reinterpret_cast<const float2*>(stats);
  const auto* ga = reinterpret_cast<const bf16*>(gamma);
  const auto* be = reinterpret_cast<const bf16*>(beta);
  const int g = (width + 255) / 256;
  if (g <= 1) launch_dependent(normalize_quantize_kernel<1>, dim3(blocks), dim3(block), 0, st, qo, q_scale, zz, st2, parts, ga, be, rows, width, epsilon);
  else if (g <= 2) launch_dependent(normalize_quantize_kernel<2>, dim3(blocks), dim3(block), 0, st, qo, q_scale, zz, st2, parts, ga, be, rows, width, epsilon);
  else if (g <= 4) launch_dependent(normalize_quantize_kernel<4>, dim3(blocks), dim3(block), 0, st, qo, q_scale, zz, st2, parts, ga, be, rows, width, epsilon);
  else launch_dependent(normalize_quantize_kernel<8>, dim3(blocks), dim3(block), 0, st, qo, q_scale, zz, st2, parts, ga, be, rows, width, epsilon);
  return launch_status();
}

namespace {
}  // namespace

int layer_norm(void* out, const void* in, const void* bias, const void* skip, const void* gamma, const void* beta,
               const void* alpha, long long rows, int width, int activation, int has_skip, float epsilon,
               void* q_out, float* q_scale, cudaStream_t st) {
  LnParams p;
  p.out = reinterpret_cast<bf16*>(out);
  p.in = reinterpret_cast<const bf16*>(in);
  p.bias = reinterpret_cast<const bf16*>(bias);
  p.skip = reinterpret_cast<const bf16*>(skip);
  p.gamma = reinterpret_cast<const bf16*>(gamma);
  p.beta = reinterpret_cast<const bf16*>(beta);
  p.alpha = reinterpret_cast<const bf16*>(alpha);
  p.q_out = reinterpret_cast<int8_t*>(q_out);
  p.q_scale = q_scale;
  p.rows = rows;
  p.width = width;
  p.activation = activation;
  p.has_skip = has_skip;
  p.epsilon = epsilon;
  if (out == nullptr && q_out == nullptr) return LC0B200_ERR_NULL_POINTER;
  const bool vec = (width % 8 == 0) && width <= 256 * kMaxGroups && aligned16(out) && aligned16(in) &&
                   aligned16(bias) && aligned16(gamma) && aligned16(beta) && (!has_skip || aligned16(skip)) &&
                   (q_out == nullptr || aligned16(q_out));
  if (vec) {
    const int g = (width + 255) / 256;
    if (g <= 1) return launch_warp<1>(p, st);
    if (g <= 2) return launch_warp<2>(p, st);
    if (g <= 3) return launch_warp<3>(p, st);
    if (g <= 4) return launch_warp<4>(p, st);
    if (g <= 6) return launch_warp<6>(p, st);
    return launch_warp<8>(p, st);
  }
  if (q_out != nullptr) return LC0B200_ERR_UNSUPPORTED;
  const bool wide_vec = (width % 8 == 0) && width <= 256 * 8 * 8 && aligned16(out) && aligned16(in) && aligned16(bias) &&
                        aligned16(gamma) && aligned16(beta) && (!has_skip || aligned16(skip)) && rows <= 0x7FFFFFFFLL;
  if (wide_vec) {
    const int g = (width / 8 + 255) / 256;
    const unsigned grid = static_cast<unsigned>(rows);
    const bool swish_plain = activation == LC0B200_ACT_SWISH && !has_skip;  // the smolgen LayerNorms
    if (g <= 2) {
      if (swish_plain) launch_dependent(layer_norm_wide_kernel<2, LC0B200_ACT_SWISH, 0>, dim3(grid), dim3(256), 0, st, p);
      else launch_dependent(layer_norm_wide_kernel<2, -1, -1>, dim3(grid), dim3(256), 0, st, p);
    } else if (g <= 4) {
      if (swish_plain) launch_dependent(layer_norm_wide_kernel<4, LC0B200_ACT_SWISH, 0>, dim3(grid), dim3(256), 0, st, p);
      else launch_dependent(layer_norm_wide_kernel<4, -1, -1>, dim3(grid), dim3(256), 0, st, p);
    } else {
      if (swish_plain) launch_dependent(layer_norm_wide_kernel<8, LC0B200_ACT_SWISH, 0>, dim3(grid), dim3(256), 0, st, p);
      else launch_dependent(layer_norm_wide_kernel<8, -1, -1>, dim3(grid), dim3(256), 0, st, p);
    }
    return launch_status();
  }
  const size_t smem = static_cast<size_t>(width) * sizeof(float);
  if (smem > 200 * 1024) return LC0B200_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(layer_norm_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess) {
      return LC0B200_ERR_CUDA;
    }
  }
  if (rows > 0x7FFFFFFFLL) return LC0B200_ERR_BAD_SHAPE;
  launch_dependent(layer_norm_block_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), smem, st, p);
  return launch_status();
}

}  // namespace lc0b200
