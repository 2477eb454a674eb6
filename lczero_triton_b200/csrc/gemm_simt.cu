// CUDA-core GEMM with the same contract as the tensor-core kernel.  It takes any shape,
// pitch and alignment, so it serves the layers TMA cannot address (output widths 1, 3 and 4 of
// the value, moves-left and promotion layers) and is the independent on-device cross-check
// of the tcgen05 kernel in the tests.  64 x 64 output tile per CTA, 4 x 4 per thread.
#include <cuda_runtime.h>

#include "common.cuh"
#include "gemm.h"

namespace lc0b200 {

namespace {

constexpr int kTile = 64;
constexpr int kTileK = 16;

struct SimtParams {
  void* out;
  const void* a;
  const void* w;
  const bf16* bias;
  const float* row_scale;
  const float* col_scale;
  long long m, lda, ldw, ldc;
  int n, k, out_kind, activation, w_kn;
};

template <bool INT8>
__device__ __forceinline__ float load_elem(const void* base, long long idx) {
  if (INT8) return static_cast<float>(reinterpret_cast<const int8_t*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const bf16*>(base)[idx]);
}

template <bool INT8>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  __shared__ float sa[kTileK][kTile + 1];
  __shared__ float sw[kTileK][kTile + 1];
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;
  const long long m0 = static_cast<long long>(blockIdx.y) * kTile;
  const int n0 = blockIdx.x * kTile;
  // int8 inputs accumulate exactly in s32; bf16 inputs in f32.
  float accf[4][4] = {};
  int acci[4][4] = {};
  for (int k0 = 0; k0 < p.k; k0 += kTileK) {
    for (int i = threadIdx.x; i < kTile * kTileK; i += 256) {
      const int r = i / kTileK, c = i % kTileK;  // A: r = row in tile, c = k
      const long long gm = m0 + r;
      const int gk = k0 + c;
      sa[c][r] = (gm < p.m && gk < p.k) ? load_elem<INT8>(p.a, gm * p.lda + gk) : 0.0f;
    }
    for (int i = threadIdx.x; i < kTile * kTileK; i += 256) {
      int kk, nn;
      if (p.w_kn) { kk = i / kTile; nn = i % kTile; } else { nn = i / kTileK; kk = i % kTileK; }
      const int gk = k0 + kk, gn = n0 + nn;
      float v = 0.0f;
      if (gk < p.k && gn < p.n) {
        v = p.w_kn ? load_elem<INT8>(p.w, static_cast<long long>(gk) * p.ldw + gn)
                   : load_elem<INT8>(p.w, static_cast<long long>(gn) * p.ldw + gk);
      }
      sw[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = sw[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (INT8) {
            acci[i][j] += static_cast<int>(av[i]) * static_cast<int>(wv[j]);
          } else {
            accf[i][j] = fmaf(av[i], wv[j], accf[i][j]);
          }
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long gm = m0 + ty * 4 + i;
    if (gm >= p.m) continue;
    const float rs = (INT8 && p.row_scale != nullptr) ? p.row_scale[gm] : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= p.n) continue;
      const long long o = gm * p.ldc + gn;
      if (p.out_kind == LC0B200_OUT_S32) {
        reinterpret_cast<int*>(p.out)[o] = INT8 ? acci[i][j] : __float_as_int(accf[i][j]);
        continue;
      }
      float y;
      if (INT8) {
        y = static_cast<float>(acci[i][j]) * rs;
        if (p.col_scale != nullptr) y *= p.col_scale[gn];
      } else {
        y = accf[i][j];
      }
      if (p.bias != nullptr) y += __bfloat162float(p.bias[gn]);
      y = activate_rt(y, p.activation);
      if (p.out_kind == LC0B200_OUT_F32) {
        reinterpret_cast<float*>(p.out)[o] = y;
      } else {
        reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(y);
      }
    }
  }
}

}  // namespace

int gemm_simt(const lc0b200_gemm_args& g, cudaStream_t stream) {
  SimtParams p;
  p.out = g.out;
  p.a = g.a;
  p.w = g.w;
  p.bias = reinterpret_cast<const bf16*>(g.bias_bf16);
  p.row_scale = g.row_scale;
  p.col_scale = g.col_scale;
  p.m = g.m;
  p.lda = g.lda;
  p.ldw = g.ldw;
  p.ldc = g.ldc;
  p.n = g.n;
  p.k = g.k;
  p.out_kind = g.out_kind;
  p.activation = g.activation;
  p.w_kn = g.w_layout == LC0B200_W_KN;
  const long long grid_y = ceil_div_ll(g.m, kTile);
  if (grid_y > 65535) {
    // Split very tall problems into slabs that fit the y-dimension limit.
    const long long slab = 65535LL * kTile;
    for (long long r0 = 0; r0 < g.m; r0 += slab) {
      lc0b200_gemm_args part = g;
      const long long rows = (g.m - r0 < slab) ? g.m - r0 : slab;
      const int in_eb = g.in_type == LC0B200_IN_INT8 ? 1 : 2;
      const int out_eb = g.out_kind == LC0B200_OUT_BF16 ? 2 : 4;
      part.m = rows;
      part.a = reinterpret_cast<const uint8_t*>(g.a) + r0 * g.lda * in_eb;
      part.out = reinterpret_cast<uint8_t*>(g.out) + r0 * g.ldc * out_eb;
      part.row_scale = g.row_scale != nullptr ? g.row_scale + r0 : nullptr;
      const int st = gemm_simt(part, stream);
      if (st != LC0B200_OK) return st;
    }
    return LC0B200_OK;
  }
  dim3 grid(static_cast<unsigned>(ceil_div_ll(g.n, kTile)), static_cast<unsigned>(grid_y));
  if (g.in_type == LC0B200_IN_INT8) {
    gemm_simt_kernel<true><<<grid, 256, 0, stream>>>(p);
  } else {
    gemm_simt_kernel<false><<<grid, 256, 0, stream>>>(p);
  }
  return launch_status();
}

}  // namespace lc0b200
