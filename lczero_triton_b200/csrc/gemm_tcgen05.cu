// Tensor-core GEMM for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma with the
// accumulator in TMEM, fused epilogue.  Replaces the reference's Triton _matmul_kernel
// (bt4/kernels/matmul.py:57-116) and, through the fused epilogue, the bias/activation kernels
// that follow it in the graph (bt4/kernels/add_bias_batched.py, add_vectors.py) and the
// LayerNorm launches (bt4/kernels/layer_norm.py) via the deferred-LayerNorm epilogues.
//
// One persistent CTA per SM walks output tiles of 128 x BN; for the large GEMMs two CTAs on the
// two SMs of a TPC form a cluster and share 256 x 256 tiles (tcgen05 cta_group::2: each CTA stages
// its own 128 rows of A and its own half of the weight tile, the leader CTA issues MMAs that read
// both shared memories, each CTA's TMEM receives its 128 rows of the accumulator).  No load is
// multicast: every CTA fetches its own operands with plain per-CTA TMA.  Warp roles:
//   warp 0      TMA producer   (the whole warp follows the loop, one elected lane issues the
//                               cp.async.bulk.tensor loads)
//   warp 1      MMA issuer     (likewise; one elected lane issues tcgen05.mma; owns the TMEM allocation)
//   warps 2..   epilogue       (eight warps for BN >= 128: two per TMEM lane quarter, each taking
//                               half of the tile's columns in groups of 64)
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps the
// main loop of tile i+1.  The epilogue is organised so that nothing it needs from global memory is
// on the critical path after the accumulator arrives: per-row LayerNorm statistics are read while
// the tile is still being multiplied, the per-column vectors of the tile wait in shared memory (put
// there one tile ahead), the residual operand of a 32 x 64 group is brought into the warp's swizzled
// staging buffer by TMA ahead of time, the result overwrites it in place and leaves by TMA store.  The
// accumulator goes back to the MMA warp as soon as its last columns are in registers.
// f32 / raw s32 results, narrow tiles and unaligned outputs use direct stores.  Operands are staged
// K-major with the 128-byte swizzle; the weight operand may instead be staged MN-major straight from
// the reference's [K,N] layout.
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "gemm.h"
#include "ptx.cuh"
#include "tensormap.h"

namespace lc0b200 {

namespace {

constexpr int kBM = 128;          // tile rows per CTA = TMEM lanes
constexpr int kRowBytes = 128;    // one swizzle row: 64 bf16 or 128 int8 along K
constexpr int kGroupBytes = 32 * kRowBytes;  // staging for 32 rows x 64 bf16 columns

// Epilogue flavours (compile-time, so that the hot loop carries no dead code):
//   kPlain: y = act(dequant(acc) + bias)
//   kLnIn : y = act(rstd[m] * (acc - mean[m] * c[n]) + d[n])        LayerNorm of the A rows folded in
//   kRes  : y = alpha * (dequant(acc) + bias) + skip, skip plain or a deferred LayerNorm; row sums out
enum : int { kPlain = 0, kLnIn = 1, kRes = 2 };

// The grouped epilogue (bf16 results, 64-column groups) stages a tile in shared memory and stores it by
// TMA (any row length a tensor map takes; asynchronous).  Stores straight from registers (32 bytes per
// lane) and a half-and-half mix were measured too: they win short bursts where the main loop is long,
// but launched back to back under the power cap the TMA store costs the least energy per launch for
// every shape of the forward pass, so it is the only form kept.
template <int BN, int CTAS, int MODE>
struct TileCfg {
  static_assert(CTAS == 1 || (CTAS == 2 && BN == 256), "CTA pairs are used for 256 x 256 tiles only");
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBRows = BN / CTAS;          // weight-tile rows (N) staged by each CTA
  static constexpr int kBBytes = kBRows * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;  // power of two for BN in {32,64,128,256}
  static constexpr int kEpilogueWarps = (BN >= 128) ? 8 : 4;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
  static constexpr bool kTmaStore = BN >= 128;      // each epilogue warp then owns whole 64-column groups
  static constexpr int kColsPerWarp = BN / (kEpilogueWarps / 4);
  static constexpr int kGroups = kColsPerWarp / 64; // 64-column groups per warp and tile (TMA-store path)
  // One staging buffer of 32 rows x 64 columns per epilogue warp and group: the residual flavour
  // lands the skip operand of the whole tile in them ahead of time, and every flavour parks the
  // whole tile's results there so that copying them out happens after the accumulator is released.
  static constexpr int kBuffersPerWarp = !kTmaStore ? 0 : kGroups;
  static constexpr int kStagingBytes = kEpilogueWarps * kBuffersPerWarp * kGroupBytes;
  // Per-column epilogue vectors of the current tile, refreshed once per tile (two fp32 vectors and,
  // for the residual flavour, one bf16 vector: see ColRegs).
  static constexpr int kVecBytes = (MODE == kRes ? 10 : 8) * BN;
  // The dynamic shared-memory window is declared 1024-byte aligned (the kernel checks), so no slack.
  static constexpr int kFixedBytes = kStagingBytes + 512 /*barriers*/ + kVecBytes;
  // As many pipeline stages as fit below the 227 KB per-CTA limit (at most 8).
  static constexpr int kFit = (227 * 1024 - kFixedBytes) / kStageBytes;
  static constexpr int kStages = kFit > 8 ? 8 : kFit;
  static_assert(kStages >= 3, "pipeline too shallow");
  static constexpr int kSmemBytes = kStages * kStageBytes + kFixedBytes;
};

struct KernelParams {
  void* out;
  // Columns [n_main, n) of the product go to a second bf16 matrix (a projection that shares A with the main
  // one: smolgen's compression rides on the QKV GEMM).  n_main is a multiple of 256, so a tile is wholly main
  // or wholly tail; n_main == n when there is no tail.
  bf16* out_tail;
  long long ldc_tail;
  int n_main;
  const bf16* bias;
  const float* row_scale;
  const float* col_scale;
  long long m;
  long long ldc;
  int n;
  int k;
  int out_kind;
  int activation;
  int vec_ok;     // out / bias / scales / fold vectors are 16-byte aligned and ldc keeps rows aligned
  int tma_store;  // bf16 output that a tensor map can address (map_out is valid)
  unsigned int* status;
  // Deferred LayerNorm (see lc0b200_gemm_args).
  const float2* ln_in_stats;
  const float* ln_in_c;
  const float* ln_in_d;
  int ln_in_parts;
  float ln_in_inv_width;
  float ln_eps;
  const bf16* res_skip;
  long long ld_skip;
  const float2* res_stats;
  const bf16* res_gamma;
  const bf16* res_beta;
  int res_parts;
  float res_inv_width;
  float res_alpha;
  float2* stats_out;
};

// Per-thread (= per output row) values the epilogue needs.
struct RowCtx {
  float rs;       // int8: activation scale of this row
  float mean;     // kLnIn: mean and 1/sqrt(var + eps) of this row of A;  kRes: of this row of the skip operand
  float rstd;
  float nmean;    // kLnIn: -mean;  kRes: -mean * rstd  (the fused multiply-add forms of finish32_sv)
  bool row_ok;
};

__device__ __forceinline__ void row_stats(const float2* stats, int parts, long long m, long long row, float inv_width,
                                          float eps, float& mean, float& rstd) {
  float s = 0.0f, q = 0.0f;
  for (int i = 0; i < parts; ++i) {
    const float2 t = __ldg(stats + i * m + row);
    s += t.x;
    q += t.y;
  }
  mean = s * inv_width;
  const float var = fmaxf(q * inv_width - mean * mean, 0.0f);
  rstd = rsqrtf(var + eps);
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  float2 t;
  t = unpack_bf16x2(raw.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16x2(raw.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16x2(raw.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16x2(raw.w); f[6] = t.x; f[7] = t.y;
}

template <bool VEC>
__device__ __forceinline__ void load8_bf16(const bf16* ptr, int valid, float (&f)[8]) {
  if (VEC) {
    unpack8(__ldg(reinterpret_cast<const uint4*>(ptr)), f);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = j < valid ? __bfloat162float(ptr[j]) : 0.0f;
  }
}

template <bool VEC>
__device__ __forceinline__ void load8_f32(const float* ptr, int valid, float fill, float (&f)[8]) {
  if (VEC) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(ptr));
    const float4 b = __ldg(reinterpret_cast<const float4*>(ptr) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = j < valid ? ptr[j] : fill;
  }
}

// Per-column vectors of one output column, as one epilogue thread carries them from global memory
// to the shared-memory vector area (a tile ahead, so the load latency is never waited for).
// They are pre-combined so that the per-element arithmetic is a short chain of fused multiply-adds:
//   kLnIn : f0 = c, f1 = d                       y = rstd * (acc - mean * c) + d
//   kPlain: f0 = int8 scale, f1 = bias           y = acc * f0 + f1
//   kRes  : f0 = int8 scale, f1 = beta + alpha * bias, g = gamma
//                                               y = alpha * acc * f0 + ((skip - mean) * rstd * g + f1)
// Columns past the matrix edge carry zeros (scale 1), so they produce exact zeros and need no guard.
struct ColRegs {
  float f0, f1;
  uint16_t g;  // bf16 bits
};

template <int MODE, bool INT8>
__device__ __forceinline__ ColRegs load_cols(const KernelParams& p, int col) {
  ColRegs r;
  r.f0 = INT8 ? 1.0f : 0.0f;
  r.f1 = 0.0f;
  r.g = 0;
  if (col < p.n) {
    if (MODE == kLnIn) {
      r.f0 = __ldg(p.ln_in_c + col);
      r.f1 = __ldg(p.ln_in_d + col);
    } else {
      if (INT8 && p.col_scale != nullptr) r.f0 = __ldg(p.col_scale + col);
      const float b = p.bias != nullptr ? __bfloat162float(p.bias[col]) : 0.0f;
      if (MODE == kRes) {
        r.f1 = p.res_alpha * b;
        r.g = 0x3F80u;  // 1.0: a skip operand that is added as it is
        if (p.res_stats != nullptr) {
          r.f1 += __bfloat162float(p.res_beta[col]);
          r.g = __ldg(reinterpret_cast<const uint16_t*>(p.res_gamma) + col);
        }
      } else {
        r.f1 = b;
      }
    }
  }
  return r;
}

// Layout of the vector area: [f0 f32 x BN][f1 f32 x BN][g bf16 x BN (kRes)].  `i` is the column inside the tile.
template <int BN, int MODE, bool INT8>
__device__ __forceinline__ void store_cols(uint32_t vec, int i, const ColRegs& r) {
  if (MODE == kLnIn || INT8) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(vec + 4 * i), "r"(__float_as_uint(r.f0)) : "memory");
  }
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(vec + 4 * BN + 4 * i), "r"(__float_as_uint(r.f1)) : "memory");
  if (MODE == kRes) asm volatile("st.shared.b16 [%0], %1;" ::"r"(vec + 8 * BN + 2 * i), "h"(r.g) : "memory");
}

__device__ __forceinline__ void lds8_f32(uint32_t addr, float (&f)[8]) {
  uint4 a, b;
  ptx::ld_shared_v4(addr, a);
  ptx::ld_shared_v4(addr + 16, b);
  f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
  f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
}
__device__ __forceinline__ void lds8_bf16(uint32_t addr, float (&f)[8]) {
  uint4 a;
  ptx::ld_shared_v4(addr, a);
  unpack8(a, f);
}

// mish(x) = x * n / (n + 2) with n = e^x (e^x + 2) (reference formula: bt4/kernels/layer_norm.py:61-69,
// which switches between n*q and x - 2q by range; with x clamped to <= 20 in the exponential the single
// form is accurate everywhere: n / (n + 2) rounds to 1 from x = 9 on and tends to n / 2 for x -> -inf).
// 32 values at a time; one reciprocal serves two elements (1/da = db / (da db)).  (Moving exponentials
// to a polynomial on the FMA pipe was measured slower: every extra instruction issued by the epilogue
// warps costs more than the transcendental unit saves.)
__device__ __forceinline__ void mish32(float (&y)[32]) {
  constexpr float kLog2e = 1.4426950408889634f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float a = y[2 * j], b = y[2 * j + 1];
    float ea, eb;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ea) : "f"(fminf(a, 20.0f) * kLog2e));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(eb) : "f"(fminf(b, 20.0f) * kLog2e));
    const float na = ea * (ea + 2.0f), nb = eb * (eb + 2.0f);
    const float da = na + 2.0f, db = nb + 2.0f;  // in [2, 2.4e17]: the product stays finite
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(da * db));
    y[2 * j] = a * (na * (db * r));
    y[2 * j + 1] = b * (nb * (da * r));
  }
}

// The TMA-store epilogue's form of finish32 (below): per-column vectors come pre-combined from the
// shared-memory vector area at `vec` (tile column `tcol`), see ColRegs.
template <int MODE, bool INT8, int BN>
__device__ __forceinline__ void finish32_sv(const uint32_t* v, uint32_t* packed, const uint32_t* skip, const RowCtx& r,
                                            const KernelParams& p, float& sum, float& sumsq, uint32_t vec, int tcol) {
  if (MODE == kPlain && !INT8) {
    // A bf16 product with neither bias nor activation (the smolgen shared projection: K = 256, one
    // gigabyte of output per layer at batch 4096) is all epilogue: round and pack, nothing else.
    if (p.bias == nullptr && p.activation == LC0B200_ACT_NONE) {
#pragma unroll
      for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
      return;
    }
  }
  float y[32];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float f0[8], f1[8];
    if (MODE == kLnIn || INT8) lds8_f32(vec + 4 * (tcol + g * 8), f0);
    lds8_f32(vec + 4 * BN + 4 * (tcol + g * 8), f1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = g * 8 + j;
      float a = INT8 ? static_cast<float>(static_cast<int>(v[e])) * r.rs : __uint_as_float(v[e]);
      if (MODE == kLnIn) {
        y[e] = fmaf(r.rstd, fmaf(r.nmean, f0[j], a), f1[j]);
      } else {
        if (INT8) a *= f0[j];
        if (MODE == kPlain) y[e] = a + f1[j];
        else y[e] = a;  // finished below, once the skip values are unpacked
      }
    }
    if (MODE == kRes) {
      float ga[8];
      lds8_bf16(vec + 8 * BN + 2 * (tcol + g * 8), ga);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack_bf16x2(skip[g * 4 + j]);
        const int e = g * 8 + 2 * j;
        y[e] = fmaf(p.res_alpha, y[e], fmaf(fmaf(t.x, r.rstd, r.nmean), ga[2 * j], f1[2 * j]));
        y[e + 1] = fmaf(p.res_alpha, y[e + 1], fmaf(fmaf(t.y, r.rstd, r.nmean), ga[2 * j + 1], f1[2 * j + 1]));
      }
    }
  }
  // The activation code is uniform for the launch: branch once per chunk, not per element.
  if (p.activation == LC0B200_ACT_MISH) {
    mish32(y);
  } else if (p.activation == LC0B200_ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = fmaxf(y[j], 0.0f);
  } else if (p.activation == LC0B200_ACT_SWISH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = act_swish(y[j]);
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(y[2 * j], y[2 * j + 1]);
  if (MODE == kRes) {
    if (p.stats_out != nullptr) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 f = unpack_bf16x2(packed[j]);  // what the consumer will read
        sum += f.x + f.y;
        sumsq = fmaf(f.x, f.x, fmaf(f.y, f.y, sumsq));
      }
    }
  }
}

// 32 output columns of one row: from raw accumulator words to packed bf16, plus the row's partial
// sums of what is stored.  `skip` holds the 32 skip values as packed bf16 pairs (kRes).  VEC selects
// 16-byte loads of the per-column vectors (whole, aligned groups) or guarded scalar loads (matrix
// edge, odd alignment).  The work is laid out as whole-chunk phases, each over 32 independent
// values, so that loads are issued together and the transcendental pipe sees long independent runs.
template <int MODE, bool INT8, bool VEC>
__device__ __forceinline__ void finish32(const uint32_t* v, uint32_t* packed, int col0, const uint32_t* skip,
                                         const RowCtx& r, const KernelParams& p, float& sum, float& sumsq) {
  float y[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    y[j] = INT8 ? static_cast<float>(static_cast<int>(v[j])) * r.rs : __uint_as_float(v[j]);
  }
  if (INT8) {
    if (p.col_scale != nullptr) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float cs[8];
        load8_f32<VEC>(p.col_scale + col0 + g * 8, p.n - col0 - g * 8, 1.0f, cs);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[g * 8 + j] *= cs[j];
      }
    }
  }
  if (MODE == kLnIn) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float c[8];
      load8_f32<VEC>(p.ln_in_c + col0 + g * 8, p.n - col0 - g * 8, 0.0f, c);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[g * 8 + j] = r.rstd * (y[g * 8 + j] - r.mean * c[j]);
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float d[8];
      load8_f32<VEC>(p.ln_in_d + col0 + g * 8, p.n - col0 - g * 8, 0.0f, d);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[g * 8 + j] += d[j];
    }
  } else if (p.bias != nullptr) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float b[8];
      load8_bf16<VEC>(p.bias + col0 + g * 8, p.n - col0 - g * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[g * 8 + j] += b[j];
    }
  }
  if (MODE == kRes) {
    float t[32];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 f = unpack_bf16x2(skip[j]);
      t[2 * j] = f.x;
      t[2 * j + 1] = f.y;
    }
    if (p.res_stats != nullptr) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float ga[8];
        load8_bf16<VEC>(p.res_gamma + col0 + g * 8, p.n - col0 - g * 8, ga);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[g * 8 + j] = (t[g * 8 + j] - r.mean) * r.rstd * ga[j];
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float be[8];
        load8_bf16<VEC>(p.res_beta + col0 + g * 8, p.n - col0 - g * 8, be);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[g * 8 + j] += be[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = p.res_alpha * y[j] + t[j];
  }
  // The activation code is uniform for the launch: branch once per chunk, not per element.
  if (p.activation == LC0B200_ACT_MISH) {
    mish32(y);
  } else if (p.activation == LC0B200_ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = fmaxf(y[j], 0.0f);
  } else if (p.activation == LC0B200_ACT_SWISH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = act_swish(y[j]);
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(y[2 * j], y[2 * j + 1]);
  if (MODE == kRes) {
    if (p.stats_out != nullptr) {
      const int valid = VEC ? 32 : p.n - col0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 f = unpack_bf16x2(packed[j]);  // what the consumer will read
        if (2 * j < valid) { sum += f.x; sumsq += f.x * f.x; }
        if (2 * j + 1 < valid) { sum += f.y; sumsq += f.y * f.y; }
      }
    }
  }
}

template <bool INT8>
__device__ __forceinline__ float acc_value(uint32_t raw, float rs, const float* __restrict__ cs, int col) {
  if (INT8) {
    float y = static_cast<float>(static_cast<int>(raw)) * rs;
    return cs != nullptr ? y * __ldg(cs + col) : y;
  }
  return __uint_as_float(raw);
}

// Width (N) of the MMAs of the n-tile that starts at column `tile_n0`: the whole tile width, or, for a bf16
// product with K-major weights whose last tile is ragged, the columns that exist rounded up to 32 - the
// tensor core then spends time on 32 columns instead of 256 for a 32-wide tail.  (32 is a valid N for both
// the single-CTA M = 128 and the CTA-pair M = 256 shapes; a pair splits it 16 + 16 between its CTAs.)
template <int BN, bool INT8, bool W_KN>
__device__ __forceinline__ int mma_width(int n, int tile_n0) {
  if (INT8 || W_KN || BN < 32) return BN;
  const int left = n - tile_n0;
  return left >= BN ? BN : ((left + 31) & ~31);
}

template <int BN, bool INT8, bool W_KN, int CTAS, int MODE>
__global__ void __launch_bounds__(TileCfg<BN, CTAS, MODE>::kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_skip,
                    const __grid_constant__ CUtensorMap map_tail, const KernelParams p) {
  using Cfg = TileCfg<BN, CTAS, MODE>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kElemsPerRow = INT8 ? 128 : 64;   // K elements per 128-byte row
  constexpr int kUmmaK = INT8 ? 32 : 16;          // K per tcgen05.mma (32 bytes)
  constexpr int kMmaPerStage = kElemsPerRow / kUmmaK;  // 4
  constexpr int kPanelN = INT8 ? 128 : 64;        // N elements per 128-byte row (MN-major weight staging)
  constexpr int kPanels = (Cfg::kBRows + kPanelN - 1) / kPanelN;
  constexpr int kPanelBytes = kElemsPerRow * kRowBytes;  // K rows x 128 B
  constexpr int kTileM = kBM * CTAS;              // rows of C per tile (per CTA pair when CTAS == 2)
  static_assert(!W_KN || (Cfg::kBRows % kPanelN == 0), "MN-major weight staging needs whole 128-byte panels");
  static_assert(MODE != kRes || Cfg::kTmaStore, "the residual epilogue needs the TMA-store layout");

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = ptx::smem_u32(smem_raw);  // 1024-byte aligned (checked below): the swizzle needs it
  const uint32_t smem_a = smem_base;
  const uint32_t smem_b = smem_base + kStages * Cfg::kABytes;
  const uint32_t staging_base = smem_base + kStages * Cfg::kStageBytes;  // 1024-byte aligned
  const uint32_t bar_base = staging_base + Cfg::kStagingBytes;
  const uint32_t bar_full = bar_base;                   // [kStages]  (used in the leader CTA only)
  const uint32_t bar_empty = bar_base + 8 * kStages;    // [kStages]
  const uint32_t bar_acc_full = bar_base + 16 * kStages;       // [2]
  const uint32_t bar_acc_empty = bar_base + 16 * kStages + 16; // [2]  (used in the leader CTA only)
  const uint32_t bar_skip = bar_base + 16 * kStages + 32;      // [kEpilogueWarps] skip tile landed (kRes)
  const uint32_t bar_vec_ready = bar_skip + 8 * Cfg::kEpilogueWarps;  // this tile's column vectors are in place
  const uint32_t bar_vec_free = bar_vec_ready + 8;                    // ... and have been read by every warp
  const uint32_t tmem_slot = bar_vec_free + 8;
  const uint32_t vec_base = bar_base + 512;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (tmem_slot + 4 - smem_base));
  static_assert(16 * 8 + 32 + 8 * 8 + 16 + 8 <= 512, "barrier area too small");
  grid_dependency_release();  // the next kernel on the stream may be scheduled as blocks of this one retire
  if ((smem_base & 1023u) != 0u) {  // never seen; refuse loudly rather than mis-swizzle
    if (threadIdx.x == 0 && atomicCAS(&p.status[0], 0u, kDeviceSmemMisaligned) == 0u) p.status[1] = smem_base;
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Rank inside the CTA pair: rank 0 is the leader (issues the MMAs, owns the full / acc-empty barriers).
  const uint32_t rank = (CTAS == 2) ? ptx::cluster_ctarank() : 0u;
  const uint32_t group = blockIdx.x / CTAS;       // CTA pair (or CTA) index
  const uint32_t num_groups = gridDim.x / CTAS;

  const long long m_tiles = (p.m + kTileM - 1) / kTileM;
  const int n_tiles = (p.n + BN - 1) / BN;
  const long long num_tiles = m_tiles * n_tiles;
  const int k_blocks = (p.k + kElemsPerRow - 1) / kElemsPerRow;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(bar_vec_ready, Cfg::kEpilogueWarps);
    ptx::mbar_init(bar_vec_free, Cfg::kEpilogueWarps);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(bar_acc_full + 8 * a, 1);
      ptx::mbar_init(bar_acc_empty + 8 * a, Cfg::kEpilogueWarps * CTAS);
    }
    for (int w = 0; w < Cfg::kEpilogueWarps; ++w) ptx::mbar_init(bar_skip + 8 * w, 1);
    ptx::mbar_init_fence();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_w);
    if (p.tma_store) ptx::prefetch_tensormap(&map_out);
    if (p.tma_store && p.n_main < p.n) ptx::prefetch_tensormap(&map_tail);
    if (MODE == kRes) ptx::prefetch_tensormap(&map_skip);
  }
  if (warp == 1) {
    if (CTAS == 2) {
      ptx::tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (CTAS == 2) ptx::cluster_sync();  // the peer's barriers exist before anything signals them
  ptx::tc_fence_after_sync();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  // Barriers, tensor memory and descriptors are ready; nothing in global memory has been touched.  From here
  // on every role reads or writes what the previous kernel on the stream produced or may still be reading.
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (every CTA loads its own operands)
    // The whole warp follows the loop; one elected lane issues the copies.
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (long long tile = group; tile < num_tiles && ok; tile += num_groups) {
      const int m0 = static_cast<int>(tile / n_tiles) * kTileM + static_cast<int>(rank) * kBM;
      // This CTA's share of the weight tile: rows [rank * width / CTAS, ...) of the tile, where width is what
      // the MMAs of this tile cover (the box is always kBRows rows; rows past the share are not read).
      const int tile_n0 = static_cast<int>(tile % n_tiles) * BN;
      const int n0 = tile_n0 + static_cast<int>(rank) * (mma_width<BN, INT8, W_KN>(p.n, tile_n0) / CTAS);
      for (int kb = 0; kb < k_blocks; ++kb) {
        ok = ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, 0x100u + stage);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        if (ptx::elect_one()) {
          // Transaction bytes of both CTAs complete on the leader's barrier.
          const uint32_t full = (CTAS == 2) ? ptx::map_to_cta(bar_full + 8 * stage, 0u) : bar_full + 8 * stage;
          if (rank == 0) ptx::mbar_expect_tx(bar_full + 8 * stage, Cfg::kStageBytes * CTAS);
          const int k0 = kb * kElemsPerRow;
          ptx::tma_load_2d<CTAS>(smem_a + stage * Cfg::kABytes, &map_a, k0, m0, full);
          if (W_KN) {
#pragma unroll
            for (int pnl = 0; pnl < kPanels; ++pnl) {
              ptx::tma_load_2d<CTAS>(smem_b + stage * Cfg::kBBytes + pnl * kPanelBytes, &map_w, n0 + pnl * kPanelN,
                                     k0, full);
            }
          } else {
            ptx::tma_load_2d<CTAS>(smem_b + stage * Cfg::kBBytes, &map_w, k0, n0, full);
          }
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t local = 0;
      bool ok = true;
      for (long long tile = group; tile < num_tiles && ok; tile += num_groups, ++local) {
        const uint32_t acc = local & 1u;
        const uint32_t acc_phase = (local >> 1) & 1u;
        ok = ptx::mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, 0x200u + acc);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        const int tile_n0 = static_cast<int>(tile % n_tiles) * BN;
        const uint32_t idesc = ptx::instr_desc(INT8 ? 2u : 1u, 1u, W_KN ? 1u : 0u, static_cast<uint32_t>(kTileM),
                                               static_cast<uint32_t>(mma_width<BN, INT8, W_KN>(p.n, tile_n0)));
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = ptx::mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 0x300u + stage);
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = smem_a + stage * Cfg::kABytes;
          const uint32_t b_addr = smem_b + stage * Cfg::kBBytes;
          if (ptx::elect_one()) {
#pragma unroll
            for (int j = 0; j < kMmaPerStage; ++j) {
              // A: K-major, 8-row groups 1024 B apart; K advance = 32 B inside the swizzle row.
              const uint64_t da = ptx::smem_desc_sw128(a_addr + j * 32, 16, 1024);
              // W: K-major as A, or MN-major: 128-byte rows run along N, one row per K index,
              //    8-row groups 1024 B apart (SBO), N panels kPanelBytes apart (LBO).
              const uint64_t db = W_KN ? ptx::smem_desc_sw128(b_addr + j * kUmmaK * kRowBytes, kPanelBytes, 1024)
                                       : ptx::smem_desc_sw128(b_addr + j * 32, 16, 1024);
              const uint32_t accumulate = (kb > 0 || j > 0) ? 1u : 0u;
              ptx::mma<INT8, CTAS>(tmem_d, da, db, idesc, accumulate);
            }
            // Free the smem stage (in both CTAs) once these MMAs have read it.
            ptx::tc_commit<CTAS>(bar_empty + 8 * stage);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (ptx::elect_one()) ptx::tc_commit<CTAS>(bar_acc_full + 8 * acc);  // accumulator complete -> epilogue (both CTAs)
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int ew = warp - 2;
    const int quarter = warp & 3;              // TMEM lane quarter this warp may access
    const int half = ew >> 2;                  // which share of the tile's columns (eight-warp layout)
    constexpr int kColsPerWarp = Cfg::kColsPerWarp;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t staging_warp = staging_base + ew * Cfg::kBuffersPerWarp * kGroupBytes;
    const uint32_t skip_bar = bar_skip + 8 * ew;
    const bool tma_path = Cfg::kTmaStore && p.tma_store && p.out_kind == LC0B200_OUT_BF16;  // grouped epilogue
    uint32_t local = 0;
    uint32_t skip_phase = 0;  // parity of this warp's skip barrier; flips each time the barrier is used
    bool ok = true;
    // Column of the tile this thread carries to the vector area (threads past BN carry none).
    const int vec_col = static_cast<int>(threadIdx.x) - 64;
    ColRegs cols = {};
    if (tma_path && vec_col < BN && group < num_tiles) {
      cols = load_cols<MODE, INT8>(p, static_cast<int>(group % n_tiles) * BN + vec_col);
    }
    for (long long tile = group; tile < num_tiles && ok; tile += num_groups, ++local) {
      const long long m0 = (tile / n_tiles) * kTileM + rank * kBM;
      const int n0 = static_cast<int>(tile % n_tiles) * BN + half * kColsPerWarp;
      const uint32_t acc = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      const long long row = m0 + row_in_tile;
      const bool row_ok = row < p.m;
      const uint32_t staging = staging_warp;

      if (tma_path) {
        // Column vectors: wait until every warp is done with the previous tile's, put this tile's in
        // place, then start the next tile's on their way.
        if (local > 0) {
          ok = ptx::mbar_wait(bar_vec_free, (local - 1u) & 1u, abort_flag, p.status, 0x600u);
          if (!ok) break;
        }
        if (vec_col < BN) store_cols<BN, MODE, INT8>(vec_base, vec_col, cols);
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_vec_ready);
        const long long next = tile + num_groups;
        if (vec_col < BN && next < num_tiles) {
          cols = load_cols<MODE, INT8>(p, static_cast<int>(next % n_tiles) * BN + vec_col);
        }
      }

      // ---- everything that can be fetched before the accumulator is complete
      RowCtx rc;
      rc.row_ok = row_ok;
      rc.rs = (INT8 && p.row_scale != nullptr && row_ok) ? __ldg(p.row_scale + row) : 1.0f;
      rc.mean = 0.0f;
      rc.rstd = 1.0f;
      if (row_ok) {
        if (MODE == kLnIn) {
          row_stats(p.ln_in_stats, p.ln_in_parts, p.m, row, p.ln_in_inv_width, p.ln_eps, rc.mean, rc.rstd);
        } else if (MODE == kRes) {
          if (p.res_stats != nullptr) {
            row_stats(p.res_stats, p.res_parts, p.m, row, p.res_inv_width, p.ln_eps, rc.mean, rc.rstd);
          }
        }
      }
      rc.nmean = (MODE == kRes) ? -rc.mean * rc.rstd : -rc.mean;
      if (tma_path) {
        // TMA-store flavours: the staging buffers are free once the previous tile's stores have
        // finished reading them.
        if (lane == 0) ptx::bulk_wait_read<0>();
        __syncwarp();
      }
      if constexpr (MODE == kRes) {
        // Bring this warp's part of the skip operand (32 rows x kColsPerWarp columns) into its staging
        // buffers, one 32 x 64 box per group.
        if (lane == 0) {
          int boxes = 0;
#pragma unroll
          for (int g = 0; g < Cfg::kGroups; ++g) boxes += (n0 + g * 64 < p.n) ? 1 : 0;
          if (boxes > 0) {
            ptx::mbar_expect_tx(skip_bar, boxes * kGroupBytes);
#pragma unroll
            for (int g = 0; g < Cfg::kGroups; ++g) {
              if (n0 + g * 64 < p.n) {
                ptx::tma_load_2d<1>(staging + g * kGroupBytes, &map_skip, n0 + g * 64,
                                    static_cast<int>(m0) + quarter * 32, skip_bar);
              }
            }
          }
        }
        __syncwarp();
      }

      ok = ptx::mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, p.status, 0x400u + acc);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      if constexpr (MODE == kRes) {
        if (n0 < p.n) {
          ok = ptx::mbar_wait(skip_bar, skip_phase, abort_flag, p.status, 0x500u + ew);
          if (!ok) break;
          skip_phase ^= 1u;
        }
      }
      if (tma_path) {
        ok = ptx::mbar_wait(bar_vec_ready, local & 1u, abort_flag, p.status, 0x700u);
        if (!ok) break;
      }
      const uint32_t taddr_row =
          tmem_base + acc * BN + half * kColsPerWarp + (static_cast<uint32_t>(quarter * 32) << 16);
      bool released = false;  // accumulator already handed back to the MMA issuer
      if (tma_path) {
        if constexpr (Cfg::kTmaStore) {
          int groups_here = (p.n - n0 + 63) >> 6;  // groups of this warp that reach into the matrix
          groups_here = groups_here < 0 ? 0 : (groups_here > Cfg::kGroups ? Cfg::kGroups : groups_here);
          if (groups_here == 0) {  // nothing to read: hand the accumulator straight back
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if (CTAS == 2) ptx::mbar_arrive_cluster(ptx::map_to_cta(bar_acc_empty + 8 * acc, 0u));
              else ptx::mbar_arrive(bar_acc_empty + 8 * acc);
            }
          }
#pragma unroll 1
          for (int g = 0; g < groups_here; ++g) {
            const int col0 = n0 + g * 64;  // a partly outside group is clipped by the store
            uint32_t v[64];
            ptx::tmem_ld_32x32(taddr_row + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
            ptx::tmem_ld_32x32(taddr_row + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
            ptx::tc_wait_ld();
            if (g == groups_here - 1) {
              // The last of this warp's accumulator columns are in registers: hand the accumulator
              // back to the MMA issuer before the arithmetic and the stores of this group.
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) {
                if (CTAS == 2) {
                  ptx::mbar_arrive_cluster(ptx::map_to_cta(bar_acc_empty + 8 * acc, 0u));  // the leader's barrier
                } else {
                  ptx::mbar_arrive(bar_acc_empty + 8 * acc);
                }
              }
            }
            float sum = 0.0f, sumsq = 0.0f;
            // Row `lane` of this group's 32 x 128-byte staging buffer (skip operand in, results out)
            // in the 128-byte swizzle the tensor maps use: 16-byte chunk c of row r lives at
            // chunk (c ^ (r & 7)).
            const uint32_t buf = staging + g * kGroupBytes;
            const uint32_t row_addr = buf + lane * kRowBytes;
#pragma unroll
            for (int h = 0; h < 2; ++h) {  // two 32-column halves of the group
              uint32_t skip_raw[16];
              if (MODE == kRes) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  uint4 raw;
                  ptx::ld_shared_v4(row_addr + (((h * 4 + c) ^ (lane & 7)) << 4), raw);
                  skip_raw[4 * c] = raw.x; skip_raw[4 * c + 1] = raw.y;
                  skip_raw[4 * c + 2] = raw.z; skip_raw[4 * c + 3] = raw.w;
                }
              }
              uint32_t pk[16];
              finish32_sv<MODE, INT8, BN>(&v[h * 32], pk, skip_raw, rc, p, sum, sumsq, vec_base,
                                          half * kColsPerWarp + g * 64 + h * 32);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                ptx::st_shared_v4(row_addr + (((h * 4 + c) ^ (lane & 7)) << 4), pk[4 * c], pk[4 * c + 1],
                                  pk[4 * c + 2], pk[4 * c + 3]);
              }
            }
            if (MODE == kRes) {
              // One partial per 64 output columns: part index col0 / 64, layout [part][row].
              if (p.stats_out != nullptr && row_ok) p.stats_out[(col0 >> 6) * p.m + row] = make_float2(sum, sumsq);
            }
          }
          // The column vectors have been read for the last time.
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_vec_free);
          released = true;
          if (n0 < p.n) {
            // One proxy fence per tile and warp (by far the most expensive instruction here), then
            // the stores of all groups; a group partly outside the matrix is clipped by the store.
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
#pragma unroll
              for (int g = 0; g < Cfg::kGroups; ++g) {
                if (n0 + g * 64 < p.n) {
                  const bool tail = n0 >= p.n_main;  // tiles never straddle n_main
                  ptx::tma_store_2d(tail ? &map_tail : &map_out, staging + g * kGroupBytes,
                                    n0 + g * 64 - (tail ? p.n_main : 0), static_cast<int>(m0) + quarter * 32);
                }
              }
              ptx::bulk_commit();
            }
          }
        }
      } else if constexpr (MODE != kRes) {
#pragma unroll 1
        for (int c = 0; c < kColsPerWarp / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.n) break;  // warp-uniform
          uint32_t v[32];
          ptx::tmem_ld_32x32(taddr_row + c * 32, v);
          ptx::tc_wait_ld();
          if (!row_ok) continue;
          const bool full_chunk = (col0 + 32 <= p.n) && p.vec_ok;
          if (p.out_kind == LC0B200_OUT_BF16) {
            uint32_t packed[16];
            float unused_sum = 0.0f, unused_sumsq = 0.0f;
            finish32<MODE, INT8, false>(v, packed, col0, nullptr, rc, p, unused_sum, unused_sumsq);
            bf16* dst = col0 >= p.n_main ? p.out_tail + row * p.ldc_tail + (col0 - p.n_main)
                                         : reinterpret_cast<bf16*>(p.out) + row * p.ldc + col0;
            if (full_chunk) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                *reinterpret_cast<uint4*>(dst + g * 8) =
                    make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.n) {
                  const uint32_t w = packed[j >> 1];
                  reinterpret_cast<uint16_t*>(dst)[j] = static_cast<uint16_t>((j & 1) ? (w >> 16) : (w & 0xFFFFu));
                }
              }
            }
          } else if (p.out_kind == LC0B200_OUT_F32) {
            float* dst = reinterpret_cast<float*>(p.out) + row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < p.n) {
                float y = acc_value<INT8>(v[j], rc.rs, p.col_scale, col0 + j);
                if (p.bias != nullptr) y += __bfloat162float(p.bias[col0 + j]);
                dst[j] = activate_rt(y, p.activation);
              }
            }
          } else {  // raw accumulator bits (s32 for int8 inputs)
            uint32_t* dst = reinterpret_cast<uint32_t*>(p.out) + row * p.ldc + col0;
            if (full_chunk) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                *reinterpret_cast<uint4*>(dst + g * 4) =
                    make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.n) dst[j] = v[j];
              }
            }
          }
        }
      }
      if (!released) {
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2) {
          ptx::mbar_arrive_cluster(ptx::map_to_cta(bar_acc_empty + 8 * acc, 0u));  // the leader's barrier
        } else {
          ptx::mbar_arrive(bar_acc_empty + 8 * acc);
        }
      }
      }
    }
    if (tma_path && lane == 0) ptx::bulk_wait_read<0>();  // staging must outlive the last store's read
    __syncwarp();
  }

  // ------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  // Neither CTA of a pair may leave while the other can still signal its barriers or read its smem.
  if (CTAS == 2) ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if (CTAS == 2) {
      ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    } else {
      ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
  }
}

// ---------------------------------------------------------------- host side

// 2-D row-major tensor [rows, cols] with a row pitch, tiled into [box_rows, box_cols] boxes
// whose inner extent is exactly 128 bytes (the swizzle span).
bool make_map(CUtensorMap* map, const void* base, int elem_bytes, long long rows, long long cols,
              long long pitch_elems, int box_rows, int box_cols) {
  return make_tensormap_2d(map, base, elem_bytes, rows, cols, pitch_elems, box_rows, box_cols,
                           CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BN, bool INT8, bool W_KN, int CTAS, int MODE>
int launch(const lc0b200_gemm_args& g, cudaStream_t stream) {
  using Cfg = TileCfg<BN, CTAS, MODE>;
  constexpr int kElemsPerRow = INT8 ? 128 : 64;
  constexpr int kPanelN = INT8 ? 128 : 64;
  const int eb = INT8 ? 1 : 2;
  CUtensorMap map_a, map_w;
  if (!make_map(&map_a, g.a, eb, g.m, g.k, g.lda, kBM, kElemsPerRow)) return LC0B200_ERR_CUDA;
  if (W_KN) {
    if (!make_map(&map_w, g.w, eb, g.k, g.n, g.ldw, kElemsPerRow, kPanelN)) return LC0B200_ERR_CUDA;
  } else {
    if (!make_map(&map_w, g.w, eb, g.n, g.k, g.ldw, Cfg::kBRows, kElemsPerRow)) return LC0B200_ERR_CUDA;
  }
  const int out_eb = g.out_kind == LC0B200_OUT_BF16 ? 2 : 4;
  const bool tma_store = Cfg::kTmaStore && g.out_kind == LC0B200_OUT_BF16 && aligned16(g.out) &&
                         ((g.ldc * out_eb) % 16 == 0);
  const bool has_tail = g.out_tail_bf16 != nullptr;
  const int n_main = has_tail ? g.n_main : g.n;
  if (has_tail && (MODE == kRes || n_main % BN != 0)) return LC0B200_ERR_UNSUPPORTED;
  CUtensorMap map_out = map_a, map_skip = map_a, map_tail = map_a;  // placeholders when unused
  if (tma_store && !make_map(&map_out, g.out, 2, g.m, n_main, g.ldc, 32, 64)) return LC0B200_ERR_CUDA;
  if (has_tail && tma_store) {
    // The tail shares the grouped epilogue with the main output, so it must be addressable the same way.
    if (!aligned16(g.out_tail_bf16) || (g.ldc_tail % 8) != 0) return LC0B200_ERR_MISALIGNED;
    if (!make_map(&map_tail, g.out_tail_bf16, 2, g.m, g.n - n_main, g.ldc_tail, 32, 64)) return LC0B200_ERR_CUDA;
  }
  if (MODE == kRes) {
    if (!tma_store) return LC0B200_ERR_UNSUPPORTED;
    if (!aligned16(g.res_skip_bf16) || (g.ld_skip % 8) != 0) return LC0B200_ERR_MISALIGNED;
    if (!make_map(&map_skip, g.res_skip_bf16, 2, g.m, g.n, g.ld_skip, 32, 64)) return LC0B200_ERR_CUDA;
  }
  auto kernel = gemm_tcgen05_kernel<BN, INT8, W_KN, CTAS, MODE>;
  static PerDeviceOnce smem_opt_in;  // per instantiation
  if (allow_dynamic_smem(smem_opt_in, kernel, Cfg::kSmemBytes) != LC0B200_OK) return LC0B200_ERR_CUDA;
  KernelParams p;
  p.out = g.out;
  p.out_tail = reinterpret_cast<bf16*>(g.out_tail_bf16);
  p.ldc_tail = g.ldc_tail;
  p.n_main = n_main;
  p.bias = reinterpret_cast<const bf16*>(g.bias_bf16);
  p.row_scale = g.row_scale;
  p.col_scale = g.col_scale;
  p.m = g.m;
  p.ldc = g.ldc;
  p.n = g.n;
  p.k = g.k;
  p.out_kind = g.out_kind;
  p.activation = g.activation;
  p.status = device_status_words();
  if (p.status == nullptr) return LC0B200_ERR_CUDA;
  p.vec_ok = aligned16(g.out) && ((g.ldc * out_eb) % 16 == 0) && (!has_tail || (aligned16(g.out_tail_bf16) && g.ldc_tail % 8 == 0)) && (g.bias_bf16 == nullptr || aligned16(g.bias_bf16)) &&
             (g.col_scale == nullptr || aligned16(g.col_scale)) &&
             (g.ln_in_stats == nullptr || (aligned16(g.ln_in_c) && aligned16(g.ln_in_d))) &&
             (g.res_stats == nullptr || (aligned16(g.res_gamma_bf16) && aligned16(g.res_beta_bf16)));
  p.tma_store = tma_store ? 1 : 0;
  p.ln_in_stats = reinterpret_cast<const float2*>(g.ln_in_stats);
  p.ln_in_c = g.ln_in_c;
  p.ln_in_d = g.ln_in_d;
  p.ln_in_parts = g.ln_in_parts;
  p.ln_in_inv_width = 1.0f / static_cast<float>(g.k);
  p.ln_eps = g.ln_eps;
  p.res_skip = reinterpret_cast<const bf16*>(g.res_skip_bf16);
  p.ld_skip = g.ld_skip;
  p.res_stats = reinterpret_cast<const float2*>(g.res_stats);
  p.res_gamma = reinterpret_cast<const bf16*>(g.res_gamma_bf16);
  p.res_beta = reinterpret_cast<const bf16*>(g.res_beta_bf16);
  p.res_parts = g.res_parts;
  p.res_inv_width = 1.0f / static_cast<float>(g.n);
  p.res_alpha = g.res_alpha;
  p.stats_out = reinterpret_cast<float2*>(g.stats_out);
  const long long tiles = ceil_div_ll(g.m, kBM * CTAS) * ceil_div_ll(g.n, BN);
  const long long max_groups = sm_count() / CTAS;
  const unsigned grid = static_cast<unsigned>((tiles < max_groups ? tiles : max_groups) * CTAS);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0] = dependent_launch_attribute();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = CTAS;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CTAS == 2 ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kernel, map_a, map_w, map_out, map_skip, map_tail, p) != cudaSuccess) {
    (void)cudaGetLastError();  // reported here; do not leave it for an unrelated later call
    return LC0B200_ERR_CUDA;
  }
  return LC0B200_OK;
}

// Rows at and above which the 256-wide tiles are shared by CTA pairs.  bf16: whenever the tile width is 256
// at all (measured from 24 positions up: 2 % faster at batch 32, 4 % at 64, 6 % at 120, level below); int8:
// from 8192 rows (below that the two forms measure the same within half a percent).
constexpr long long kPairMinRowsBf16 = 256;
constexpr long long kPairMinRowsInt8 = 8192;

template <bool INT8, bool W_KN, int MODE>
int dispatch_bn(const lc0b200_gemm_args& g, cudaStream_t stream) {
  // Tile width: the widest of 256 / 128 / 64 / 32 that still gives most SMs a tile, so that small
  // problems (batch 64: a 64 x 256 output) spread over several CTAs instead of one.
  // MN-major weight staging needs whole 128-byte panels (64 bf16 or 128 int8 columns); the residual
  // epilogue needs the TMA-store layout (BN >= 128).
  constexpr int kMinBn = (MODE == kRes) ? 128 : (W_KN ? (INT8 ? 128 : 64) : 32);
  const long long rows128 = ceil_div_ll(g.m, kBM);
  const long long enough = sm_count() * 3LL / 5;
  auto tiles = [&](int bn) { return rows128 * ceil_div_ll(g.n, bn); };
  int bn = 256;
  while (bn > kMinBn && (bn / 2 >= g.n || tiles(bn) < enough)) bn /= 2;
  if (bn == 256) {
    // (Short main loops are paced by the output and measured faster on single CTAs.)
    if (g.m >= (INT8 ? kPairMinRowsInt8 : kPairMinRowsBf16) && g.k > 512) return launch<256, INT8, W_KN, 2, MODE>(g, stream);
    return launch<256, INT8, W_KN, 1, MODE>(g, stream);
  }
  if constexpr (kMinBn <= 128) {
    if (bn == 128) return launch<128, INT8, W_KN, 1, MODE>(g, stream);
  }
  if constexpr (kMinBn <= 64) {
    if (bn == 64) return launch<64, INT8, W_KN, 1, MODE>(g, stream);
  }
  if constexpr (kMinBn <= 32) {
    if (bn == 32) return launch<32, INT8, W_KN, 1, MODE>(g, stream);
  }
  return LC0B200_ERR_UNSUPPORTED;
}

template <bool INT8, bool W_KN>
int dispatch_mode(const lc0b200_gemm_args& g, cudaStream_t stream) {
  const bool ln_in = g.ln_in_stats != nullptr;
  const bool res = g.res_skip_bf16 != nullptr;
  if (ln_in && res) return LC0B200_ERR_UNSUPPORTED;
  if ((ln_in || res || g.stats_out != nullptr) && g.out_kind != LC0B200_OUT_BF16) return LC0B200_ERR_UNSUPPORTED;
  if (g.stats_out != nullptr && !res) return LC0B200_ERR_UNSUPPORTED;
  if constexpr (INT8) {
    // An int8 GEMM cannot fold the LayerNorm of its input (the input is already quantised); it can
    // produce the residual form.  Only the pre-transposed weight layout is instantiated for it.
    if (ln_in) return LC0B200_ERR_UNSUPPORTED;
    if (res) {
      if constexpr (W_KN) {
        return LC0B200_ERR_UNSUPPORTED;
      } else {
        return dispatch_bn<INT8, W_KN, kRes>(g, stream);
      }
    }
    return dispatch_bn<INT8, W_KN, kPlain>(g, stream);
  } else {
    if (ln_in) return dispatch_bn<INT8, W_KN, kLnIn>(g, stream);
    if (res) return dispatch_bn<INT8, W_KN, kRes>(g, stream);
    return dispatch_bn<INT8, W_KN, kPlain>(g, stream);
  }
}

}  // namespace

bool gemm_tcgen05_supported(const lc0b200_gemm_args& g) {
  const int eb = g.in_type == LC0B200_IN_INT8 ? 1 : 2;
  if (g.m <= 0 || g.n <= 0 || g.k <= 0) return false;
  if (!aligned16(g.a) || !aligned16(g.w)) return false;
  if ((g.lda * eb) % 16 != 0 || (g.ldw * eb) % 16 != 0) return false;
  if (g.m > 0x7FFFFF00LL) return false;  // tile coordinates are 32-bit
  return true;
}

int gemm_tcgen05(const lc0b200_gemm_args& g, cudaStream_t stream) {
  const bool int8 = g.in_type == LC0B200_IN_INT8;
  const bool w_kn = g.w_layout == LC0B200_W_KN;
  if (int8) return w_kn ? dispatch_mode<true, true>(g, stream) : dispatch_mode<true, false>(g, stream);
  return w_kn ? dispatch_mode<false, true>(g, stream) : dispatch_mode<false, false>(g, stream);
}

}  // namespace lc0b200
