// Layout, element-wise and quantisation kernels (all HBM-bound; one pass, 64-bit indexing).
// Each kernel names the reference Triton kernel it replaces; paths are relative to
// packages/lczero-triton/src/lczero_triton/bt4/kernels/.
// Kernels with a reference counterpart are written as a __device__ body plus a thin __global__ entry:
// lc0ex_bridge.py wraps the same body in an extern "C" entry point whose parameters are pointers only and
// whose shapes are compile-time constants (the contract of an lc0ex kernel artifact).
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lc0b200 {

namespace {

constexpr int kBlock = 256;

inline unsigned grid_for(long long elements, int per_block = kBlock) {
  long long g = ceil_div_ll(elements, per_block);
  const long long cap = static_cast<long long>(sm_count()) * 32;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<unsigned>(g);
}

// expand_planes.py:26-42
__device__ __forceinline__ void expand_planes_body(bf16* __restrict__ out, const uint64_t* __restrict__ masks,
                                                   const float* __restrict__ values, long long plane_count) {
  const long long total = plane_count * 64;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long plane = i >> 6;
    const int sq = static_cast<int>(i & 63);
    const bf16 v = __float2bfloat16_rn(values[plane]);
    out[i] = ((masks[plane] >> sq) & 1ull) ? v : __float2bfloat16_rn(0.0f);
  }
}
__global__ void expand_planes_kernel(bf16* __restrict__ out, const uint64_t* __restrict__ masks,
                                     const float* __restrict__ values, long long plane_count) {
  grid_dependency_release();
  grid_dependency_wait();
  expand_planes_body(out, masks, values, plane_count);
}

// nchw_to_nhwc.py:26-44
__device__ __forceinline__ void nchw_to_nhwc_body(bf16* __restrict__ out, const bf16* __restrict__ in, long long total,
                                                  int input_channels, int output_channels, int hw) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % output_channels);
    const long long rest = i / output_channels;
    const int s = static_cast<int>(rest % hw);
    const long long b = rest / hw;
    out[i] = in[(b * input_channels + c) * hw + s];
  }
}
__global__ void nchw_to_nhwc_kernel(bf16* __restrict__ out, const bf16* __restrict__ in, long long total,
                                    int input_channels, int output_channels, int hw) {
  grid_dependency_release();
  grid_dependency_wait();
  nchw_to_nhwc_body(out, in, total, input_channels, output_channels, hw);
}

// preprocess_attention_body.py:26-61
__device__ __forceinline__ void preprocess_attention_body_body(bf16* __restrict__ out, const bf16* __restrict__ planes,
                                                               const bf16* __restrict__ encoding, long long total,
                                                               int input_channels, int encoding_channels) {
  const int width = input_channels + encoding_channels;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % width);
    const long long token = i / width;
    const long long b = token >> 6;
    const int sq = static_cast<int>(token & 63);
    out[i] = c < input_channels ? planes[(b * input_channels + c) * 64 + sq]
                                : encoding[token * encoding_channels + (c - input_channels)];
  }
}
__global__ void preprocess_attention_body_kernel(bf16* __restrict__ out, const bf16* __restrict__ planes,
                                                 const bf16* __restrict__ encoding, long long total,
                                                 int input_channels, int encoding_channels) {
  grid_dependency_release();
  grid_dependency_wait();
  preprocess_attention_body_body(out, planes, encoding, total, input_channels, encoding_channels);
}

// input_gating.py:26-51
__device__ __forceinline__ void input_gating_body(bf16* out, const bf16* in, const bf16* __restrict__ mult,
                                                  const bf16* __restrict__ add, long long total, long long gate_elements) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long g = i % gate_elements;
    const float x = __bfloat162float(in[i]);
    out[i] = __float2bfloat16_rn(x * __bfloat162float(mult[g]) + __bfloat162float(add[g]));
  }
}
__global__ void input_gating_kernel(bf16* out, const bf16* in, const bf16* __restrict__ mult,
                                    const bf16* __restrict__ add, long long total, long long gate_elements) {
  grid_dependency_release();
  grid_dependency_wait();
  input_gating_body(out, in, mult, add, total, gate_elements);
}

// Same, eight channels per thread with 16-byte accesses (gate_elements a multiple of 8).
__global__ void input_gating_vec_kernel(uint4* out, const uint4* in, const uint4* __restrict__ mult,
                                        const uint4* __restrict__ add, long long groups, long long gate_groups) {
  grid_dependency_release();
  grid_dependency_wait();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < groups;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long g = i % gate_groups;
    const uint4 x = in[i], m = __ldg(mult + g), a = __ldg(add + g);
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ms[4] = {m.x, m.y, m.z, m.w}, as[4] = {a.x, a.y, a.z, a.w};
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = unpack_bf16x2(xs[j]), mf = unpack_bf16x2(ms[j]), af = unpack_bf16x2(as[j]);
      r[j] = pack_bf16x2(xf.x * mf.x + af.x, xf.y * mf.y + af.y);
    }
    out[i] = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

// add_vectors.py:37-66 (period = bias_element_count, rows = 1) and
// add_bias_batched.py:35-66 (bias row chosen by i / (row_count * channel_count)).
__device__ __forceinline__ void add_bias_body(bf16* out, const bf16* in, const bf16* __restrict__ bias, long long total,
                                              int channels, long long elements_per_batch, int activation) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long bt = i / elements_per_batch;
    const int c = static_cast<int>(i % channels);
    const float x = __bfloat162float(in[i]) + __bfloat162float(bias[bt * channels + c]);
    out[i] = __float2bfloat16_rn(activate_rt(x, activation));
  }
}
__global__ void add_bias_kernel(bf16* out, const bf16* in, const bf16* __restrict__ bias, long long total,
                                int channels, long long elements_per_batch, int activation) {
  grid_dependency_release();
  grid_dependency_wait();
  add_bias_body(out, in, bias, total, channels, elements_per_batch, activation);
}

// fused_qkv.py:132-183: three independent row-broadcast bias adds in one launch.
struct QkvBiasParams {
  bf16* out[3];
  const bf16* in[3];
  const bf16* bias[3];
  int width[3];
  long long rows;
};
__device__ __forceinline__ void fused_qkv_bias_body(const QkvBiasParams p) {
  const int which = blockIdx.y;
  const long long total = p.rows * p.width[which];
  bf16* out = p.out[which];
  const bf16* in = p.in[which];
  const bf16* bias = p.bias[which];
  const int w = p.width[which];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    out[i] = __float2bfloat16_rn(__bfloat162float(in[i]) + __bfloat162float(bias[i % w]));
  }
}
__global__ void fused_qkv_bias_kernel(const QkvBiasParams p) {
  grid_dependency_release();
  grid_dependency_wait();
  fused_qkv_bias_body(p);
}

// copy_type_converted.py:26-34
__device__ __forceinline__ void widen_body(float* __restrict__ out, const bf16* __restrict__ in, long long total) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    out[i] = __bfloat162float(in[i]);
  }
}
__global__ void widen_kernel(float* __restrict__ out, const bf16* __restrict__ in, long long total) {
  grid_dependency_release();
  grid_dependency_wait();
  widen_body(out, in, total);
}

// policy_map.py:28-49
__device__ __forceinline__ void policy_map_body(bf16* __restrict__ out, const bf16* __restrict__ in,
                                                const int32_t* __restrict__ table, long long total, int in_count, int out_count) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(i % out_count);
    const long long b = i / out_count;
    const int src = table[o];
    out[i] = (src >= 0 && src < in_count) ? in[b * in_count + src] : __float2bfloat16_rn(0.0f);
  }
}
__global__ void policy_map_kernel(bf16* __restrict__ out, const bf16* __restrict__ in,
                                  const int32_t* __restrict__ table, long long total, int in_count, int out_count) {
  grid_dependency_release();
  grid_dependency_wait();
  policy_map_body(out, in, table, total, in_count, out_count);
}

// dst[c, r] = src[r, c] through a padded shared-memory tile.
template <typename T>
__global__ void transpose_kernel(T* __restrict__ dst, const T* __restrict__ src, int rows, int cols) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ T tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[static_cast<long long>(r) * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[static_cast<long long>(c) * rows + r] = tile[threadIdx.x][j];
  }
}

// Fused plane expansion + NHWC extraction of the 12 current-position piece planes
// (expand_planes.py + nchw_to_nhwc.py; network.py:458-484).
__global__ void embed_position_input_kernel(bf16* __restrict__ out, const uint64_t* __restrict__ masks,
                                            const float* __restrict__ values, long long total) {
  grid_dependency_release();
  grid_dependency_wait();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % 12);
    const long long rest = i / 12;
    const int sq = static_cast<int>(rest & 63);
    const long long b = rest >> 6;
    const long long plane = b * 112 + c;
    const bf16 v = __float2bfloat16_rn(values[plane]);
    out[i] = ((masks[plane] >> sq) & 1ull) ? v : __float2bfloat16_rn(0.0f);
  }
}

// Fused plane expansion + per-token concat with the positional encoding
// (expand_planes.py + preprocess_attention_body.py; network.py:458-465,521-533).
// One CTA per position; each thread moves 16-byte groups of 8 channels.
__global__ void __launch_bounds__(kBlock) embed_concat_kernel(bf16* __restrict__ out,
                                                              const uint64_t* __restrict__ masks,
                                                              const float* __restrict__ values,
                                                              const bf16* __restrict__ position, int enc) {
  grid_dependency_release();
  grid_dependency_wait();
  __shared__ uint64_t s_mask[112];
  __shared__ uint16_t s_val[112];
  const long long b = blockIdx.x;
  if (threadIdx.x < 112) {
    s_mask[threadIdx.x] = masks[b * 112 + threadIdx.x];
    const bf16 v = __float2bfloat16_rn(values[b * 112 + threadIdx.x]);
    s_val[threadIdx.x] = *reinterpret_cast<const uint16_t*>(&v);
  }
  __syncthreads();
  const int width = 112 + enc;
  if ((enc & 7) == 0) {
    const int groups = width >> 3;
    const uint4* pos = reinterpret_cast<const uint4*>(position + b * 64 * enc);
    uint4* dst = reinterpret_cast<uint4*>(out + b * 64 * width);
    for (int i = threadIdx.x; i < 64 * groups; i += kBlock) {
      const int sq = i / groups, g = i % groups;
      uint4 v;
      if (g < 14) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = g * 8 + j * 2;
          const uint32_t lo = ((s_mask[c] >> sq) & 1ull) ? s_val[c] : 0u;
          const uint32_t hi = ((s_mask[c + 1] >> sq) & 1ull) ? s_val[c + 1] : 0u;
          w[j] = lo | (hi << 16);
        }
        v = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
        v = pos[sq * (enc >> 3) + (g - 14)];
      }
      dst[i] = v;
    }
  } else {
    uint16_t* dst = reinterpret_cast<uint16_t*>(out + b * 64 * width);
    const uint16_t* pos = reinterpret_cast<const uint16_t*>(position + b * 64 * enc);
    for (int i = threadIdx.x; i < 64 * width; i += kBlock) {
      const int sq = i / width, c = i % width;
      dst[i] = c < 112 ? (((s_mask[c] >> sq) & 1ull) ? s_val[c] : uint16_t(0)) : pos[sq * enc + (c - 112)];
    }
  }
}

// Symmetric per-row int8 quantisation, one warp per row:
// s = max|x| / 127 (1 when the row is all zero); q = clamp(rint(x * (127 / max|x|)), -127, 127).
// Rows up to 2048 wide stay in registers between the two passes.
__device__ __forceinline__ uint2 quantize8(const uint4& raw, float inv) {
  const float2 f0 = unpack_bf16x2(raw.x), f1 = unpack_bf16x2(raw.y), f2 = unpack_bf16x2(raw.z), f3 = unpack_bf16x2(raw.w);
  return make_uint2(quantize4_s8(f0.x, f0.y, f1.x, f1.y, inv), quantize4_s8(f2.x, f2.y, f3.x, f3.y, inv));
}

__device__ __forceinline__ float amax8(const uint4& raw, float amax) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(w[j]);
    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  return amax;
}

// The common case - aligned rows of up to 2048 columns, a multiple of 8 - with the number of 16-byte groups a
// lane keeps fixed at compile time, so that a 1024-wide row costs 4 registers of data per lane, not 8 (the
// kernel is bound by how many rows the SM has in flight, i.e. by registers per thread).
// Two rows (warps) per CTA: small CTAs keep more rows in flight and shorten the tail of the launch.
constexpr int kQuantWarps = 2;

template <int GROUPS>
__global__ void __launch_bounds__(kQuantWarps * 32) quantize_rows_held_kernel(int8_t* __restrict__ out, float* __restrict__ scale,
                                                                              const bf16* __restrict__ in, long long rows,
                                                                              int width, long long ld_in) {
  grid_dependency_release();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * static_cast<long long>(kQuantWarps) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint4* src = reinterpret_cast<const uint4*>(in + row * ld_in);
  uint2* dst = reinterpret_cast<uint2*>(out + row * width);
  const int groups = width >> 3;
  uint4 keep[GROUPS];
#pragma unroll
  for (int i = 0; i < GROUPS; ++i) {
    const int g = lane + 32 * i;
    keep[i] = g < groups ? __ldg(src + g) : make_uint4(0u, 0u, 0u, 0u);
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < GROUPS; ++i) amax = amax8(keep[i], amax);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 1.0f;
  if (lane == 0) scale[row] = s;
#pragma unroll
  for (int i = 0; i < GROUPS; ++i) {
    const int g = lane + 32 * i;
    if (g < groups) dst[g] = quantize8(keep[i], inv);
  }
}

// Any width, pitch and alignment.
__global__ void __launch_bounds__(kBlock) quantize_rows_kernel(int8_t* __restrict__ out, float* __restrict__ scale,
                                                               const bf16* __restrict__ in, long long rows,
                                                               int width, long long ld_in) {
  grid_dependency_release();
  grid_dependency_wait();
  constexpr int kHeld = 8;  // 16-byte groups a lane keeps in registers: 8 * 32 lanes * 8 values = 2048 columns
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * static_cast<long long>(kBlock / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const bf16* src = in + row * ld_in;
  int8_t* dst = out + row * width;
  const bool vec = ((width & 7) == 0) && ((ld_in & 7) == 0) && aligned16_dev(in) && aligned16_dev(out);
  const int groups = width >> 3;
  const bool held = vec && groups <= kHeld * 32;
  uint4 keep[kHeld];
  float amax = 0.0f;
  if (held) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int g = lane + 32 * i;
      keep[i] = g < groups ? __ldg(reinterpret_cast<const uint4*>(src) + g) : make_uint4(0u, 0u, 0u, 0u);
      amax = amax8(keep[i], amax);
    }
  } else if (vec) {
    for (int g = lane; g < groups; g += 32) amax = amax8(__ldg(reinterpret_cast<const uint4*>(src) + g), amax);
  } else {
    for (int c = lane; c < width; c += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[c])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 1.0f;
  if (lane == 0) scale[row] = s;
  if (held) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int g = lane + 32 * i;
      if (g < groups) reinterpret_cast<uint2*>(dst)[g] = quantize8(keep[i], inv);
    }
  } else if (vec) {
    for (int g = lane; g < groups; g += 32) {
      reinterpret_cast<uint2*>(dst)[g] = quantize8(__ldg(reinterpret_cast<const uint4*>(src) + g), inv);
    }
  } else {
    for (int c = lane; c < width; c += 32) {
      const int q = max(-127, min(127, __float2int_rn(__bfloat162float(src[c]) * inv)));
      dst[c] = static_cast<int8_t>(q);
    }
  }
}

}  // namespace

#define LC0_STREAM(s) reinterpret_cast<cudaStream_t>(s)

int expand_planes(void* out, const uint64_t* masks, const float* values, long long plane_count, cudaStream_t st) {
  launch_dependent(expand_planes_kernel, dim3(grid_for(plane_count * 64)), dim3(kBlock), 0, st, reinterpret_cast<bf16*>(out), masks, values,
                                                                     plane_count);
  return launch_status();
}

int nchw_to_nhwc(void* out, const void* in, int batch, int in_ch, int out_ch, int hw, cudaStream_t st) {
  const long long total = static_cast<long long>(batch) * hw * out_ch;
  launch_dependent(nchw_to_nhwc_kernel, dim3(grid_for(total)), dim3(kBlock), 0, st, reinterpret_cast<bf16*>(out),
                                                          reinterpret_cast<const bf16*>(in), total, in_ch, out_ch, hw);
  return launch_status();
}

int preprocess_attention_body(void* out, const void* planes, const void* enc, int batch, int in_ch, int enc_ch,
                              cudaStream_t st) {
  const long long total = static_cast<long long>(batch) * 64 * (in_ch + enc_ch);
  launch_dependent(preprocess_attention_body_kernel, dim3(grid_for(total)), dim3(kBlock), 0, st, 
      reinterpret_cast<bf16*>(out), reinterpret_cast<const bf16*>(planes), reinterpret_cast<const bf16*>(enc), total,
      in_ch, enc_ch);
  return launch_status();
}

int input_gating(void* out, const void* in, const void* mult, const void* add, int batch, int squares, int channels,
                 cudaStream_t st) {
  const long long gate = static_cast<long long>(squares) * channels;
  const long long total = gate * batch;
  if (gate % 8 == 0 && aligned16(out) && aligned16(in) && aligned16(mult) && aligned16(add)) {
    launch_dependent(input_gating_vec_kernel, dim3(grid_for(total / 8)), dim3(kBlock), 0, st, 
        reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(in), reinterpret_cast<const uint4*>(mult),
        reinterpret_cast<const uint4*>(add), total / 8, gate / 8);
    return launch_status();
  }
  launch_dependent(input_gating_kernel, dim3(grid_for(total)), dim3(kBlock), 0, st, reinterpret_cast<bf16*>(out),
                                                          reinterpret_cast<const bf16*>(in),
                                                          reinterpret_cast<const bf16*>(mult),
                                                          reinterpret_cast<const bf16*>(add), total, gate);
  return launch_status();
}

int add_bias(void* out, const void* in, const void* bias, long long total, int channels, long long per_batch,
             int activation, cudaStream_t st) {
  launch_dependent(add_bias_kernel, dim3(grid_for(total)), dim3(kBlock), 0, st, reinterpret_cast<bf16*>(out), reinterpret_cast<const bf16*>(in),
                                                      reinterpret_cast<const bf16*>(bias), total, channels, per_batch,
                                                      activation);
  return launch_status();
}

int fused_qkv_bias(void* const out[3], const void* const in[3], const void* const bias[3], const int width[3],
                   long long rows, cudaStream_t st) {
  QkvBiasParams p;
  int wmax = 0;
  for (int i = 0; i < 3; ++i) {
    p.out[i] = reinterpret_cast<bf16*>(out[i]);
    p.in[i] = reinterpret_cast<const bf16*>(in[i]);
    p.bias[i] = reinterpret_cast<const bf16*>(bias[i]);
    p.width[i] = width[i];
    wmax = width[i] > wmax ? width[i] : wmax;
  }
  p.rows = rows;
  dim3 grid(grid_for(rows * wmax), 3);
  launch_dependent(fused_qkv_bias_kernel, dim3(grid), dim3(kBlock), 0, st, p);
  return launch_status();
}

int widen(float* out, const void* in, long long total, cudaStream_t st) {
  launch_dependent(widen_kernel, dim3(grid_for(total)), dim3(kBlock), 0, st, out, reinterpret_cast<const bf16*>(in), total);
  return launch_status();
}

int policy_map(void* out, const void* in, const int32_t* table, int batch, int in_count, int out_count,
               cudaStream_t st) {
  const long long total = static_cast<long long>(batch) * out_count;
  launch_dependent(policy_map_kernel, dim3(grid_for(total)), dim3(kBlock), 0, st, reinterpret_cast<bf16*>(out),
                                                        reinterpret_cast<const bf16*>(in), table, total, in_count,
                                                        out_count);
  return launch_status();
}

int transpose(void* dst, const void* src, int rows, int cols, int element_size, cudaStream_t st) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (element_size == 1) {
    launch_dependent(transpose_kernel<uint8_t>, dim3(grid), dim3(block), 0, st, reinterpret_cast<uint8_t*>(dst),
                                                      reinterpret_cast<const uint8_t*>(src), rows, cols);
  } else {
    launch_dependent(transpose_kernel<uint16_t>, dim3(grid), dim3(block), 0, st, reinterpret_cast<uint16_t*>(dst),
                                                       reinterpret_cast<const uint16_t*>(src), rows, cols);
  }
  return launch_status();
}

int embed_position_input(void* out, const uint64_t* masks, const float* values, int batch, cudaStream_t st) {
  const long long total = static_cast<long long>(batch) * 64 * 12;
  launch_dependent(embed_position_input_kernel, dim3(grid_for(total)), dim3(kBlock), 0, st, reinterpret_cast<bf16*>(out), masks, values, total);
  return launch_status();
}

int embed_concat(void* out, const uint64_t* masks, const float* values, const void* position, int batch, int enc,
                 cudaStream_t st) {
  launch_dependent(embed_concat_kernel, dim3(batch), dim3(kBlock), 0, st, reinterpret_cast<bf16*>(out), masks, values,
                                                reinterpret_cast<const bf16*>(position), enc);
  return launch_status();
}

int quantize_rows(void* out, float* scale, const void* in, long long rows, int width, long long ld_in,
                  cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>(ceil_div_ll(rows, kBlock / 32));
  const unsigned held_blocks = static_cast<unsigned>(ceil_div_ll(rows, kQuantWarps));
  constexpr int kHeldThreads = kQuantWarps * 32;
  auto* q = reinterpret_cast<int8_t*>(out);
  const auto* x = reinterpret_cast<const bf16*>(in);
  const bool held = (width % 8) == 0 && (ld_in % 8) == 0 && width <= 2048 && aligned16(in) && aligned16(out) &&
                    rows <= 0x7FFFFFFFLL;
  if (held) {
    const int g = (width + 255) / 256;
    if (g <= 1) launch_dependent(quantize_rows_held_kernel<1>, dim3(held_blocks), dim3(kHeldThreads), 0, st, q, scale, x, rows, width, ld_in);
    else if (g <= 2) launch_dependent(quantize_rows_held_kernel<2>, dim3(held_blocks), dim3(kHeldThreads), 0, st, q, scale, x, rows, width, ld_in);
    else if (g <= 4) launch_dependent(quantize_rows_held_kernel<4>, dim3(held_blocks), dim3(kHeldThreads), 0, st, q, scale, x, rows, width, ld_in);
    else if (g <= 6) launch_dependent(quantize_rows_held_kernel<6>, dim3(held_blocks), dim3(kHeldThreads), 0, st, q, scale, x, rows, width, ld_in);
    else launch_dependent(quantize_rows_held_kernel<8>, dim3(held_blocks), dim3(kHeldThreads), 0, st, q, scale, x, rows, width, ld_in);
  } else {
    launch_dependent(quantize_rows_kernel, dim3(blocks), dim3(kBlock), 0, st, q, scale, x, rows, width, ld_in);
  }
  return launch_status();
}

}  // namespace lc0b200
