// Attention for the 64-token board.
//
// attention_kernel fuses the reference's three launches per encoder layer
//   _qk_kernel (bt4/kernels/batched_matmul.py:68-141)  S = scale * Q_h K_h^T
//   _softmax_64_kernel (bt4/kernels/softmax_64.py:45-71)  P = softmax(clamp(S + smolgen))
//   _attention_v_kernel (bt4/kernels/batched_matmul.py:150-210)  O = P V_h, written merged
// into one kernel: the 64 x 64 scores of a head never leave the SM.  The operator is HBM-bound
// (Q, K, V, the 64 x 64 bias and O are each touched once: 24 KB per head for ~1 MFLOP), so the
// design goal is bytes in flight: every CTA streams a run of heads through a two-stage
// cp.async pipeline while its four warps (16 query rows each) do the small tensor-core products
// on the previous stage.
//
// The remaining kernels are the stand-alone forms of the same ops for per-op parity with the
// reference (softmax_64, body_qk / policy_qk, attention_v); policy_qk (K = policy width) is also
// what the policy head uses.
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lc0b200 {

namespace {

constexpr float kClamp = 131008.0f;  // twice the fp16 maximum, softmax_64.py:62-65
constexpr int kRowStride = 80;       // bytes; 64-byte rows padded so ldmatrix is conflict-free
constexpr int kBiasStride = 144;     // bytes; 128-byte rows padded so fragment reads are conflict-free
constexpr int kTileBytes = 64 * kRowStride;            // one 64 x 32 bf16 operand tile
constexpr int kBiasBytes = 64 * kBiasStride;
constexpr int kStageBytes = 3 * kTileBytes + kBiasBytes;  // 24576

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// clamp(v, -131008, 131008) that keeps NaN (min.NaN / max.NaN return NaN if an input is NaN).
__device__ __forceinline__ float clamp_keep_nan(float v) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(v), "f"(-kClamp));
  asm("min.NaN.f32 %0, %0, %1;" : "+f"(r) : "f"(kClamp));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

struct AttnParams {
  bf16* out;
  const bf16* q;
  const bf16* k;
  const bf16* v;
  const bf16* bias;
  long long ldq, ldk, ldv, ldo;
  long long items;  // batch * heads
  int heads;
  float scale;
};

__device__ __forceinline__ void load_head(uint8_t* stage, const AttnParams& p, long long item) {
  const long long b = item / p.heads;
  const int h = static_cast<int>(item % p.heads);
  const uint32_t s = smem_addr(stage);
  // 3 tiles x 64 rows x 4 chunks of 16 bytes: thread t moves chunks t and t + 128 of each tile.
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int rc = threadIdx.x + it * 128, row = rc >> 2, ch = rc & 3;
    const long long tok = b * 64 + row;
    const uint32_t dst = s + row * kRowStride + ch * 16;
    const int col = h * 32 + ch * 8;
    cp_async16(dst, p.q + tok * p.ldq + col);
    cp_async16(dst + kTileBytes, p.k + tok * p.ldk + col);
    cp_async16(dst + 2 * kTileBytes, p.v + tok * p.ldv + col);
  }
  if (p.bias != nullptr) {
    const bf16* src = p.bias + item * 4096;
#pragma unroll
    for (int it = 0; it < 4; ++it) {  // 64 rows x 8 chunks = 512 chunks
      const int c = threadIdx.x + it * 128;
      const int row = c >> 3, ch = c & 7;
      cp_async16(s + 3 * kTileBytes + row * kBiasStride + ch * 16, src + row * 64 + ch * 8);
    }
  }
}

// HPB = consecutive heads streamed by one CTA.
template <int HPB>
__global__ void __launch_bounds__(128) attention_kernel(const AttnParams p) {
  grid_dependency_release();
  grid_dependency_wait();
  constexpr int kHeadsPerBlock = HPB;
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const long long first = static_cast<long long>(blockIdx.x) * kHeadsPerBlock;
  const long long remaining = p.items - first;
  const int count = remaining < kHeadsPerBlock ? static_cast<int>(remaining) : kHeadsPerBlock;

  load_head(smem, p, first);
  cp_async_commit();
  for (int i = 0; i < count; ++i) {
    uint8_t* stage = smem + (i & 1) * kStageBytes;
    if (i + 1 < count) load_head(smem + ((i + 1) & 1) * kStageBytes, p, first + i + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const uint32_t qs = smem_addr(stage), ks = qs + kTileBytes, vs = qs + 2 * kTileBytes;
    const uint8_t* bs = stage + 3 * kTileBytes;
    const int mi = lane >> 3, ri = lane & 7;  // ldmatrix: matrix index and row within it

    // ---- S = Q K^T for this warp's 16 query rows
    uint32_t qa[2][4];
    ldmatrix_x4(qa[0], qs + (16 * warp + (mi & 1) * 8 + ri) * kRowStride + (mi >> 1) * 16);
    ldmatrix_x4(qa[1], qs + (16 * warp + (mi & 1) * 8 + ri) * kRowStride + 32 + (mi >> 1) * 16);
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
      uint32_t kb[4];
      ldmatrix_x4(kb, ks + (8 * j + ri) * kRowStride + mi * 16);
      mma_16816(s[j], qa[0], kb[0], kb[1]);
      mma_16816(s[j], qa[1], kb[2], kb[3]);
    }
    // ---- scale, edge bias, clamp, softmax over the 64 keys (rows g and g + 8 of the warp's slab)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2 b0 = make_float2(0.f, 0.f), b1 = make_float2(0.f, 0.f);
      if (p.bias != nullptr) {
        const int col = 8 * j + 2 * t;
        b0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(bs + (16 * warp + g) * kBiasStride + col * 2));
        b1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(bs + (16 * warp + g + 8) * kBiasStride + col * 2));
      }
      // Scores stay in fp32 from the tensor-core accumulator to the softmax (the reference rounds
      // them to its 16-bit storage type in between only because it materialises them).
      s[j][0] = clamp_keep_nan(s[j][0] * p.scale + b0.x);
      s[j][1] = clamp_keep_nan(s[j][1] * p.scale + b0.y);
      s[j][2] = clamp_keep_nan(s[j][2] * p.scale + b1.x);
      s[j][3] = clamp_keep_nan(s[j][3] * p.scale + b1.y);
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
    // exp(v - max) as exp2(v * log2e - max * log2e): one fused multiply-add and one ex2 per score.
    // P stays un-normalised (values in (0, 1]) for the second product; the 16 x 32 result is scaled
    // by 1 / sum afterwards, which costs half as many multiplies as scaling P.
    constexpr float kLog2e = 1.4426950408889634f;
    const float off0 = mx0 * kLog2e, off1 = mx1 * kLog2e;
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j][0] = fast_exp2(fmaf(s[j][0], kLog2e, -off0));
      s[j][1] = fast_exp2(fmaf(s[j][1], kLog2e, -off0));
      s[j][2] = fast_exp2(fmaf(s[j][2], kLog2e, -off1));
      s[j][3] = fast_exp2(fmaf(s[j][3], kLog2e, -off1));
      sum0 += s[j][0] + s[j][1];
      sum1 += s[j][2] + s[j][3];
    }
    sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 1);
    sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 2);
    sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 1);
    sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 2);
    const float inv0 = 1.0f / sum0, inv1 = 1.0f / sum1;

    // ---- O = P V
    float o[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
#pragma unroll
    for (int step = 0; step < 4; ++step) {  // 16 keys per step
      uint32_t pa[4];
      pa[0] = pack_bf16x2(s[2 * step][0], s[2 * step][1]);
      pa[1] = pack_bf16x2(s[2 * step][2], s[2 * step][3]);
      pa[2] = pack_bf16x2(s[2 * step + 1][0], s[2 * step + 1][1]);
      pa[3] = pack_bf16x2(s[2 * step + 1][2], s[2 * step + 1][3]);
#pragma unroll
      for (int jj = 0; jj < 4; jj += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vs + (16 * step + (mi & 1) * 8 + ri) * kRowStride + (8 * jj + (mi >> 1) * 8) * 2);
        mma_16816(o[jj], pa, vb[0], vb[1]);
        mma_16816(o[jj + 1], pa, vb[2], vb[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j][0] *= inv0;
      o[j][1] *= inv0;
      o[j][2] *= inv1;
      o[j][3] *= inv1;
    }
    // ---- stage O through this warp's own (now dead) Q rows, then 16-byte coalesced stores
    __syncwarp();
    uint8_t* orow = stage + (16 * warp) * kRowStride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      *reinterpret_cast<uint32_t*>(orow + g * kRowStride + (8 * j + 2 * t) * 2) = pack_bf16x2(o[j][0], o[j][1]);
      *reinterpret_cast<uint32_t*>(orow + (g + 8) * kRowStride + (8 * j + 2 * t) * 2) = pack_bf16x2(o[j][2], o[j][3]);
    }
    __syncwarp();
    const long long item = first + i;
    const long long b = item / p.heads;
    const int h = static_cast<int>(item % p.heads);
#pragma unroll
    for (int c = lane; c < 64; c += 32) {
      const int row = c >> 2, ch = c & 3;
      const uint4 val = *reinterpret_cast<const uint4*>(orow + row * kRowStride + ch * 16);
      *reinterpret_cast<uint4*>(p.out + (b * 64 + 16 * warp + row) * p.ldo + h * 32 + ch * 8) = val;
    }
    __syncthreads();
  }
  cp_async_wait<0>();
}

// softmax_64.py:45-71, one warp per row of 64, two columns per lane.  (A device function: the kernel
// below and the pointer-only entry points generated by lc0ex_bridge.py both wrap it.)
__device__ __forceinline__ void softmax_64_body(bf16* out, const bf16* qk, const bf16* smolgen, long long rows) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float2 a = unpack_bf16x2(reinterpret_cast<const uint32_t*>(qk + row * 64)[lane]);
  const float2 b = unpack_bf16x2(reinterpret_cast<const uint32_t*>(smolgen + row * 64)[lane]);
  const float v0 = clamp_keep_nan(a.x + b.x), v1 = clamp_keep_nan(a.y + b.y);
  float mx = fmaxf(v0, v1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  const float e0 = __expf(v0 - mx), e1 = __expf(v1 - mx);
  float sum = e0 + e1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  const float inv = 1.0f / sum;
  reinterpret_cast<uint32_t*>(out + row * 64)[lane] = pack_bf16x2(e0 * inv, e1 * inv);
}

__global__ void __launch_bounds__(256) softmax_64_kernel(bf16* out, const bf16* qk, const bf16* smolgen,
                                                         long long rows) {
  grid_dependency_release();
  grid_dependency_wait();
  softmax_64_body(out, qk, smolgen, rows);
}

// Tensor-core QK^T for 64 x 64 outputs with any K that is a multiple of 32: body_qk (heads
// interleaved, K = head depth) and policy_qk (contiguous, K = policy width, record stride 4288).
struct QkParams {
  bf16* out;
  const bf16* q;
  const bf16* k;
  const bf16* scale;
  long long out_stride;
  int depth;
  int heads;
  int interleaved;
};

__device__ __forceinline__ void load_qk_chunk(uint8_t* stage, const QkParams& p, long long matrix, int k0) {
  long long base, ld;
  if (p.interleaved) {
    const long long b = matrix / p.heads;
    const int h = static_cast<int>(matrix % p.heads);
    ld = static_cast<long long>(p.heads) * p.depth;
    base = b * 64 * ld + static_cast<long long>(h) * p.depth;
  } else {
    ld = p.depth;
    base = matrix * 64 * ld;
  }
  const uint32_t s = smem_addr(stage);
#pragma unroll
  for (int it = 0; it < 4; ++it) {  // 2 tiles x 64 rows x 4 chunks
    const int c = threadIdx.x + it * 128;
    const int which = c >> 8, rc = c & 255, row = rc >> 2, ch = rc & 3;
    const bf16* src = (which ? p.k : p.q) + base + row * ld + k0 + ch * 8;
    cp_async16(s + which * kTileBytes + row * kRowStride + ch * 16, src);
  }
}

__device__ __forceinline__ void qk_mma_body(const QkParams p) {
  __shared__ __align__(16) uint8_t smem[2 * 2 * kTileBytes];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3, mi = lane >> 3, ri = lane & 7;
  const long long matrix = blockIdx.x;
  const int chunks = p.depth / 32;
  float s[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
  load_qk_chunk(smem, p, matrix, 0);
  cp_async_commit();
  for (int i = 0; i < chunks; ++i) {
    uint8_t* stage = smem + (i & 1) * 2 * kTileBytes;
    if (i + 1 < chunks) load_qk_chunk(smem + ((i + 1) & 1) * 2 * kTileBytes, p, matrix, (i + 1) * 32);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t qs = smem_addr(stage), ks = qs + kTileBytes;
    uint32_t qa[2][4];
    ldmatrix_x4(qa[0], qs + (16 * warp + (mi & 1) * 8 + ri) * kRowStride + (mi >> 1) * 16);
    ldmatrix_x4(qa[1], qs + (16 * warp + (mi & 1) * 8 + ri) * kRowStride + 32 + (mi >> 1) * 16);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t kb[4];
      ldmatrix_x4(kb, ks + (8 * j + ri) * kRowStride + mi * 16);
      mma_16816(s[j], qa[0], kb[0], kb[1]);
      mma_16816(s[j], qa[1], kb[2], kb[3]);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  const float scale = p.scale != nullptr ? __bfloat162float(*p.scale) : 1.0f;
  bf16* out = p.out + matrix * p.out_stride;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int col = 8 * j + 2 * t;
    *reinterpret_cast<uint32_t*>(out + (16 * warp + g) * 64 + col) = pack_bf16x2(s[j][0] * scale, s[j][1] * scale);
    *reinterpret_cast<uint32_t*>(out + (16 * warp + g + 8) * 64 + col) = pack_bf16x2(s[j][2] * scale, s[j][3] * scale);
  }
}
__global__ void __launch_bounds__(128) qk_mma_kernel(const QkParams p) {
  grid_dependency_release();
  grid_dependency_wait();
  qk_mma_body(p);
}

// Generic CUDA-core forms of the three batched products (any m, n, k): one thread per output.
struct BmmParams {
  bf16* out;
  const bf16* a;
  const bf16* b;
  const bf16* scale;
  long long batch_count;
  int operation, m, n, k, heads;
};

__global__ void __launch_bounds__(256) bmm_generic_kernel(const BmmParams p) {
  grid_dependency_release();
  grid_dependency_wait();
  const long long per = static_cast<long long>(p.m) * p.n;
  const long long total = p.batch_count * per;
  const float scale = (p.operation != LC0B200_BMM_BODY_ATTENTION_V && p.scale != nullptr)
                          ? __bfloat162float(*p.scale) : 1.0f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long matrix = i / per;
    const int r = static_cast<int>((i % per) / p.n), c = static_cast<int>(i % p.n);
    const long long sample = matrix / p.heads;
    const int head = static_cast<int>(matrix % p.heads);
    float acc = 0.0f;
    if (p.operation == LC0B200_BMM_BODY_ATTENTION_V) {
      // a = attention [matrix, m, k]; b = values [sample, k, heads * n]; out merged [sample, m, heads * n]
      const long long vw = static_cast<long long>(p.heads) * p.n;
      const bf16* arow = p.a + (matrix * p.m + r) * p.k;
      const bf16* bcol = p.b + sample * p.k * vw + static_cast<long long>(head) * p.n + c;
      for (int kk = 0; kk < p.k; ++kk) acc = fmaf(__bfloat162float(arow[kk]), __bfloat162float(bcol[kk * vw]), acc);
      p.out[(sample * p.m + r) * vw + static_cast<long long>(head) * p.n + c] = __float2bfloat16_rn(acc);
    } else {
      long long abase, bbase, ld, ostride;
      if (p.operation == LC0B200_BMM_BODY_QK) {
        ld = static_cast<long long>(p.heads) * p.k;
        abase = sample * p.m * ld + static_cast<long long>(head) * p.k;
        bbase = sample * p.n * ld + static_cast<long long>(head) * p.k;
        ostride = per;
      } else {
        ld = p.k;
        abase = matrix * p.m * ld;
        bbase = matrix * p.n * ld;
        ostride = 4288;
      }
      const bf16* arow = p.a + abase + r * ld;
      const bf16* brow = p.b + bbase + c * ld;
      for (int kk = 0; kk < p.k; ++kk) acc = fmaf(__bfloat162float(arow[kk]), __bfloat162float(brow[kk]), acc);
      p.out[matrix * ostride + static_cast<long long>(r) * p.n + c] = __float2bfloat16_rn(acc * scale);
    }
  }
}

}  // namespace

int softmax_64(void* out, const void* qk, const void* smolgen, long long rows, cudaStream_t st) {
  const long long blocks = ceil_div_ll(rows, 8);
  launch_dependent(softmax_64_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, st, reinterpret_cast<bf16*>(out),
                                                                 reinterpret_cast<const bf16*>(qk),
                                                                 reinterpret_cast<const bf16*>(smolgen), rows);
  return launch_status();
}

int attention(void* out, const void* q, const void* k, const void* v, const void* bias, float scale,
              long long batch, int heads, long long ldq, long long ldk, long long ldv, long long ldo,
              cudaStream_t st) {
  if (attention_tc_supported(out, q, k, v, bias, batch, heads, ldq, ldk, ldv, ldo)) {
    return attention_tc(out, q, k, v, bias, scale, batch, heads, ldq, ldk, ldv, ldo, st);
  }
  AttnParams p;
  p.out = reinterpret_cast<bf16*>(out);
  p.q = reinterpret_cast<const bf16*>(q);
  p.k = reinterpret_cast<const bf16*>(k);
  p.v = reinterpret_cast<const bf16*>(v);
  p.bias = reinterpret_cast<const bf16*>(bias);
  p.ldq = ldq;
  p.ldk = ldk;
  p.ldv = ldv;
  p.ldo = ldo;
  p.items = batch * heads;
  p.heads = heads;
  p.scale = scale;
  // Heads per CTA: long runs amortise the pipeline prologue; short runs keep all SMs busy when the
  // batch is small.
  const int hpb = p.items >= 64LL * 8 * sm_count() ? 16 : (p.items >= 16LL * 8 * sm_count() ? 8 : 4);
  auto run = [&](auto kernel, PerDeviceOnce& once, int heads_per_block) -> int {
    if (allow_dynamic_smem(once, kernel, 2 * kStageBytes) != LC0B200_OK) return LC0B200_ERR_CUDA;
    const long long blocks = ceil_div_ll(p.items, heads_per_block);
    if (blocks > 0x7FFFFFFFLL) return LC0B200_ERR_BAD_SHAPE;
    launch_dependent(kernel, dim3(static_cast<unsigned>(blocks)), dim3(128), 2 * kStageBytes, st, p);
    return launch_status();
  };
  static PerDeviceOnce once16, once8, once4;
  if (hpb >= 16) return run(attention_kernel<16>, once16, 16);
  if (hpb >= 8) return run(attention_kernel<8>, once8, 8);
  return run(attention_kernel<4>, once4, 4);
}

int batched_matmul(void* out, const void* a, const void* b, const void* scale, int operation, long long batch_count,
                   int m, int n, int k, int heads, cudaStream_t st) {
  const bool qk_op = operation == LC0B200_BMM_BODY_QK || operation == LC0B200_BMM_POLICY_QK;
  if (qk_op && m == 64 && n == 64 && k % 32 == 0 && aligned16(a) && aligned16(b) && aligned16(out) &&
      batch_count <= 0x7FFFFFFFLL) {
    QkParams p;
    p.out = reinterpret_cast<bf16*>(out);
    p.q = reinterpret_cast<const bf16*>(a);
    p.k = reinterpret_cast<const bf16*>(b);
    p.scale = reinterpret_cast<const bf16*>(scale);
    p.out_stride = operation == LC0B200_BMM_POLICY_QK ? 4288 : 4096;
    p.depth = k;
    p.heads = heads;
    p.interleaved = operation == LC0B200_BMM_BODY_QK;
    launch_dependent(qk_mma_kernel, dim3(static_cast<unsigned>(batch_count)), dim3(128), 0, st, p);
    return launch_status();
  }
  BmmParams p;
  p.out = reinterpret_cast<bf16*>(out);
  p.a = reinterpret_cast<const bf16*>(a);
  p.b = reinterpret_cast<const bf16*>(b);
  p.scale = reinterpret_cast<const bf16*>(scale);
  p.batch_count = batch_count;
  p.operation = operation;
  p.m = m;
  p.n = n;
  p.k = k;
  p.heads = heads;
  long long blocks = ceil_div_ll(batch_count * m * n, 256);
  const long long cap = static_cast<long long>(sm_count()) * 32;
  if (blocks > cap) blocks = cap;
  launch_dependent(bmm_generic_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, st, p);
  return launch_status();
}

}  // namespace lc0b200
