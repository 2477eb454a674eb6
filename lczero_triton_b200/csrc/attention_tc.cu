// Fused edge-biased attention on the 5th-generation tensor cores: QK^T, smolgen bias, softmax and
// PV for the 64-token board with the scores held in TMEM and the probabilities in shared memory.
// Same math as attention_kernel in attention.cu (reference: bt4/kernels/batched_matmul.py:68-141,
// softmax_64.py:45-71, batched_matmul.py:150-210), different machine mapping:
//
//  * a persistent CTA streams PAIRS of heads; the two heads are stacked into one 128-row problem
//        S[128 x 128] = [Q_a; Q_b] [K_a; K_b]^T        (tcgen05.mma M=128, N=128, K=32)
//    whose diagonal 64 x 64 blocks are the two score matrices (the off-diagonal blocks are never read:
//    tensor work is free here, the operator is HBM-bound);
//  * 128 softmax threads own one score row each: tcgen05.ld brings the 64 scores of the row into
//    registers, so max / exp / sum need no shuffles; the un-normalised probabilities go to shared
//    memory as the K-major A operand of
//        O[128 x 32] = P[128 x 128] [V_a; V_b]          (M=128, N=32, K=128, P block-diagonal)
//    and the 1 / sum scaling is applied to the 32 outputs of the row;
//  * operands arrive by TMA (64-byte swizzle for the 64 x 32 Q, K, V tiles, 128-byte swizzle for the
//    64 x 64 bias tiles) through a three-stage ring, results leave by TMA stores;
//  * two softmax warpgroups alternate pairs (even pairs / odd pairs), each with its own score and
//    output accumulators in TMEM and its own P buffer, so that one group's TMEM reads, exponentials
//    and stores overlap the other group's.
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer (and TMEM owner), warps 2..5 and 6..9 softmax.
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include "tensormap.h"

namespace lc0b200 {

namespace {

constexpr float kClamp = 131008.0f;  // twice the fp16 maximum, softmax_64.py:62-65
constexpr int kStages = 3;
constexpr int kTileQ = 64 * 64;            // 64 rows x 64 bytes
constexpr int kTileBias = 64 * 128;        // 64 rows x 128 bytes
constexpr int kOffQ = 0, kOffK = 2 * kTileQ, kOffV = 4 * kTileQ, kOffBias = 6 * kTileQ;
constexpr int kStageBytes = 6 * kTileQ + 2 * kTileBias;  // 40960
constexpr int kPOne = 2 * 128 * 128;       // one P buffer: two K-blocks of 128 rows x 128 bytes
constexpr int kPBytes = 2 * kPOne;         // one per softmax warpgroup
constexpr int kOutBytes = 8 * 32 * 64;     // per softmax warp: 32 rows x 64 bytes
constexpr int kSmemBytes = kStages * kStageBytes + kPBytes + kOutBytes + 1024 + 256;
constexpr int kThreads = 64 + 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;  // S buffers at 0 / 128, O buffers at 256 / 288

struct TcParams {
  long long pairs;     // number of head pairs
  int heads;
  int has_bias;
  float scale;
  unsigned int* status;
};

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

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_bias,
                    const __grid_constant__ CUtensorMap map_out, const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_base = base;
  const uint32_t p_base = base + kStages * kStageBytes;      // 1024-aligned (40960 = 40 * 1024)
  const uint32_t out_base = p_base + kPBytes;
  const uint32_t bar = out_base + kOutBytes;
  const uint32_t bar_in_full = bar, bar_in_empty = bar + 8 * kStages;
  const uint32_t bar_s_full = bar + 16 * kStages, bar_s_empty = bar_s_full + 16;
  const uint32_t bar_o_full = bar_s_empty + 16, bar_o_empty = bar_o_full + 16;
  const uint32_t bar_p_full = bar_o_empty + 16, bar_p_empty = bar_p_full + 16;
  const uint32_t tmem_slot = bar_p_empty + 16;
  __shared__ int abort_flag_storage;
  volatile int* abort_flag = &abort_flag_storage;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  grid_dependency_release();
  if (threadIdx.x == 0) {
    abort_flag_storage = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(bar_in_full + 8 * s, 1);
      ptx::mbar_init(bar_in_empty + 8 * s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(bar_s_full + 8 * t, 1);
      ptx::mbar_init(bar_s_empty + 8 * t, 4);
      ptx::mbar_init(bar_o_full + 8 * t, 1);
      ptx::mbar_init(bar_o_empty + 8 * t, 4);
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(bar_p_full + 8 * t, 4);
      ptx::mbar_init(bar_p_empty + 8 * t, 1);
    }
    ptx::mbar_init_fence();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    ptx::prefetch_tensormap(&map_out);
    if (p.has_bias) ptx::prefetch_tensormap(&map_bias);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  // The off-diagonal blocks of P (rows of one head x keys of the other) stay zero for the whole
  // kernel: block 0 rows 64..127 and block 1 rows 0..63, 8 KB each, contiguous from +8192, in both buffers.
  for (int i = threadIdx.x; i < 2 * (16384 / 16); i += kThreads) {
    const int buf = i / (16384 / 16), c = i % (16384 / 16);
    ptx::st_shared_v4(p_base + buf * kPOne + 8192 + c * 16, 0u, 0u, 0u, 0u);
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  grid_dependency_wait();  // set-up done; Q, K, V and the bias come from the kernels before this one

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // (The whole warp follows the loop and one elected lane issues: warp-uniform control flow lets
    // the compiler keep addresses and descriptors in uniform registers.)
    bool ok = true;
    uint32_t i = 0;
    for (long long pair = blockIdx.x; pair < p.pairs && ok; pair += gridDim.x, ++i) {
      const uint32_t s = i % kStages, ph = (i / kStages) & 1u;
      ok = ptx::mbar_wait(bar_in_empty + 8 * s, ph ^ 1u, abort_flag, p.status, 0x610u + s);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      if (ptx::elect_one()) {
        const uint32_t full = bar_in_full + 8 * s;
        ptx::mbar_expect_tx(full, 6 * kTileQ + (p.has_bias ? 2 * kTileBias : 0));
        const uint32_t st = stage_base + s * kStageBytes;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const long long item = 2 * pair + e;
          const int b = static_cast<int>(item / p.heads), h = static_cast<int>(item % p.heads);
          ptx::tma_load_2d<1>(st + kOffQ + e * kTileQ, &map_q, h * 32, b * 64, full);
          ptx::tma_load_2d<1>(st + kOffK + e * kTileQ, &map_k, h * 32, b * 64, full);
          ptx::tma_load_2d<1>(st + kOffV + e * kTileQ, &map_v, h * 32, b * 64, full);
          if (p.has_bias) {
            ptx::tma_load_2d<1>(st + kOffBias + e * kTileBias, &map_bias, 0, static_cast<int>(item) * 64, full);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (whole warp, one elected lane)
    constexpr uint32_t idesc_s = ptx::instr_desc(1u, 1u, 0u, 128u, 128u);  // bf16 -> f32, A and B K-major
    constexpr uint32_t idesc_o = ptx::instr_desc(1u, 1u, 1u, 128u, 32u);   // B (= V) MN-major
    bool ok = true;
    auto second_product = [&](uint32_t k) -> bool {
      const uint32_t s = k % kStages, t = k & 1u;
      bool good = ptx::mbar_wait(bar_p_full + 8 * t, (k >> 1) & 1u, abort_flag, p.status, 0x640u + t);
      good = good && ptx::mbar_wait(bar_o_empty + 8 * t, ((k >> 1) & 1u) ^ 1u, abort_flag, p.status, 0x650u + t);
      if (!__all_sync(0xFFFFFFFFu, good)) return false;
      ptx::tc_fence_after_sync();
      const uint32_t v_addr = stage_base + s * kStageBytes + kOffV;
      if (ptx::elect_one()) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // 16 keys per step; the two heads' keys are stacked
          const uint64_t da = ptx::smem_desc_sw128(p_base + t * kPOne + (j >> 2) * 16384 + (j & 3) * 32, 16, 1024);
          const uint64_t db = ptx::smem_desc_sw64(v_addr + j * 1024, 512, 512);
          ptx::mma_bf16(tmem_base + kColO + t * 32, da, db, idesc_o, j > 0 ? 1u : 0u);
        }
        ptx::tc_commit(bar_o_full + 8 * t);
        ptx::tc_commit(bar_in_empty + 8 * s);  // Q, K, V and the bias tiles of this stage are dead
        ptx::tc_commit(bar_p_empty + 8 * t);
      }
      return true;
    };
    uint32_t i = 0;
    for (long long pair = blockIdx.x; pair < p.pairs && ok; pair += gridDim.x, ++i) {
      const uint32_t s = i % kStages, t = i & 1u;
      ok = ptx::mbar_wait(bar_in_full + 8 * s, (i / kStages) & 1u, abort_flag, p.status, 0x620u + s);
      ok = ok && ptx::mbar_wait(bar_s_empty + 8 * t, ((i >> 1) & 1u) ^ 1u, abort_flag, p.status, 0x630u + t);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t st = stage_base + s * kStageBytes;
      if (ptx::elect_one()) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {  // depth 32 = two K steps of 16
          const uint64_t da = ptx::smem_desc_sw64(st + kOffQ + j * 32, 16, 512);
          const uint64_t db = ptx::smem_desc_sw64(st + kOffK + j * 32, 16, 512);
          ptx::mma_bf16(tmem_base + kColS + t * 128, da, db, idesc_s, j > 0 ? 1u : 0u);
        }
        ptx::tc_commit(bar_s_full + 8 * t);
      }
      if (i > 0) ok = second_product(i - 1);
    }
    if (ok && i > 0) second_product(i - 1);
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax / epilogue: one score row per thread
    const uint32_t wg = static_cast<uint32_t>(warp - 2) >> 2;  // softmax warpgroup: pairs with (i & 1) == wg
    const int quarter = warp & 3;              // TMEM lane quarter
    const int row = quarter * 32 + lane;       // row of the stacked problem
    const int e = row >> 6;                    // which head of the pair
    const int r = row & 63;                    // token within the head
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t out_buf = out_base + (warp - 2) * (32 * 64);
    constexpr float kLog2e = 1.4426950408889634f;
    bool ok = true;
    // O row of pair `j_pair` (the j-th pair of this CTA): 32 outputs, scaled by 1 / sum, to this warp's
    // staging box, then a TMA store.
    auto finish_output = [&](long long j_pair, uint32_t j, float row_sum) -> bool {
      const uint32_t t = j & 1u;
      if (!ptx::mbar_wait(bar_o_full + 8 * t, (j >> 1) & 1u, abort_flag, p.status, 0x680u + t)) return false;
      ptx::tc_fence_after_sync();
      uint32_t oraw[32];
      ptx::tmem_ld_32x32(tmem_base + kColO + t * 32 + lane_sel, oraw);
      ptx::tc_wait_ld();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(bar_o_empty + 8 * t);
        ptx::bulk_wait_read<0>();  // the previous store of this warp has read the staging box
      }
      __syncwarp();
      const float inv = 1.0f / row_sum;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) {
          w[k2] = pack_bf16x2(__uint_as_float(oraw[c * 8 + 2 * k2]) * inv, __uint_as_float(oraw[c * 8 + 2 * k2 + 1]) * inv);
        }
        // 32 rows x 64 bytes in the 64-byte swizzle: 16-byte chunk c of row q lives at chunk c ^ ((q >> 1) & 3)
        ptx::st_shared_v4(out_buf + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4), w[0], w[1], w[2], w[3]);
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const long long item = 2 * j_pair + e;
        const int b = static_cast<int>(item / p.heads), h = static_cast<int>(item % p.heads);
        ptx::tma_store_2d(&map_out, out_buf, h * 32, b * 64 + (quarter & 1) * 32);
        ptx::bulk_commit();
      }
      return true;
    };
    bool have_pending = false;
    long long pending_pair = 0;
    uint32_t pending_i = 0;
    float pending_sum = 1.0f;
    uint32_t i = 0;
    for (long long pair = blockIdx.x; pair < p.pairs && ok; pair += gridDim.x, ++i) {
      const uint32_t s = i % kStages, t = i & 1u;
      if (t != wg) continue;
      ok = ptx::mbar_wait(bar_s_full + 8 * t, (i >> 1) & 1u, abort_flag, p.status, 0x660u + t);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      uint32_t sraw[64];
      ptx::tmem_ld_32x64(tmem_base + kColS + t * 128 + e * 64 + lane_sel, sraw);
      ptx::tc_wait_ld();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_s_empty + 8 * t);

      // The bias tile was written by TMA: observe its barrier directly (already complete by now).
      if (p.has_bias) {
        ok = ptx::mbar_wait(bar_in_full + 8 * s, (i / kStages) & 1u, abort_flag, p.status, 0x690u + s);
        if (!ok) break;
      }
      // scores * scale + bias, clamp, row max
      float v[64];
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one of 64
      const uint32_t bias_row = stage_base + s * kStageBytes + kOffBias + e * kTileBias + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (p.has_bias) {
          uint4 raw;
          ptx::ld_shared_v4(bias_row + ((c ^ (r & 7)) << 4), raw);
          float2 f;
          f = unpack_bf16x2(raw.x); b[0] = f.x; b[1] = f.y;
          f = unpack_bf16x2(raw.y); b[2] = f.x; b[3] = f.y;
          f = unpack_bf16x2(raw.z); b[4] = f.x; b[5] = f.y;
          f = unpack_bf16x2(raw.w); b[6] = f.x; b[7] = f.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float x = fmaf(__uint_as_float(sraw[c * 8 + j]), p.scale, b[j]);
          v[c * 8 + j] = x;
          mx4[j & 3] = fmaxf(mx4[j & 3], x);
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The reference clamps every score to +-131008 (softmax_64.py:45-71).  The clamp changes the result
      // only when the row maximum is above the range, or so close to its lower end that a score clamped
      // up to -131008 would still get a non-zero weight (exp2 of less than -256 * log2(e) is zero either
      // way); such rows, infinities included, take the per-element clamp.  NaN scores pass through and
      // make the row NaN in both cases.
      if (mx > kClamp || mx < -kClamp + 256.0f) {
#pragma unroll
        for (int j = 0; j < 64; ++j) v[j] = clamp_keep_nan(v[j]);
        mx = fmaxf(fminf(mx, kClamp), -kClamp);
      }
      const float off = mx * kLog2e;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float p0 = fast_exp2(fmaf(v[2 * j], kLog2e, -off));
        const float p1 = fast_exp2(fmaf(v[2 * j + 1], kLog2e, -off));
        sum4[j & 3] += p0 + p1;
        pk[j] = pack_bf16x2(p0, p1);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // P row into the K-major, 128-byte-swizzled A operand of the second product: K block e.
      ok = ptx::mbar_wait(bar_p_empty + 8 * t, ((i >> 1) & 1u) ^ 1u, abort_flag, p.status, 0x670u + t);
      if (!ok) break;
      const uint32_t p_row = p_base + t * kPOne + e * 16384 + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        ptx::st_shared_v4(p_row + ((c ^ (row & 7)) << 4), pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_p_full + 8 * t);

      // The O rows of this pair are finished one round later, after the next softmax of this
      // warpgroup: the second product and its barrier round trip then never make it wait.
      if (have_pending) {
        ok = finish_output(pending_pair, pending_i, pending_sum);
        if (!ok) break;
      }
      have_pending = true;
      pending_pair = pair;
      pending_i = i;
      pending_sum = sum;
    }
    if (ok && have_pending) finish_output(pending_pair, pending_i, pending_sum);
    if (lane == 0) ptx::bulk_wait_read<0>();
    __syncwarp();
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

bool attention_tc_supported(const void* out, const void* q, const void* k, const void* v, const void* bias,
                            long long batch, int heads, long long ldq, long long ldk, long long ldv, long long ldo) {
  if ((heads & 1) != 0 || batch <= 0) return false;
  if (!aligned16(out) || !aligned16(q) || !aligned16(k) || !aligned16(v) || (bias != nullptr && !aligned16(bias))) {
    return false;
  }
  if ((ldq % 8) != 0 || (ldk % 8) != 0 || (ldv % 8) != 0 || (ldo % 8) != 0) return false;
  if (batch * 64 > 0x7FFFFF00LL || batch * heads * 64 > 0x7FFFFF00LL) return false;  // 32-bit TMA coordinates
  return true;
}

int attention_tc(void* out, const void* q, const void* k, const void* v, const void* bias, float scale,
                 long long batch, int heads, long long ldq, long long ldk, long long ldv, long long ldo,
                 cudaStream_t st) {
  const long long rows = batch * 64;
  const long long width = static_cast<long long>(heads) * 32;
  CUtensorMap mq, mk, mv, mb, mo;
  if (!make_tensormap_2d(&mq, q, 2, rows, width, ldq, 64, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return LC0B200_ERR_CUDA;
  if (!make_tensormap_2d(&mk, k, 2, rows, width, ldk, 64, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return LC0B200_ERR_CUDA;
  if (!make_tensormap_2d(&mv, v, 2, rows, width, ldv, 64, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return LC0B200_ERR_CUDA;
  if (!make_tensormap_2d(&mo, out, 2, rows, width, ldo, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return LC0B200_ERR_CUDA;
  mb = mq;
  if (bias != nullptr &&
      !make_tensormap_2d(&mb, bias, 2, batch * heads * 64, 64, 64, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return LC0B200_ERR_CUDA;
  }
  static PerDeviceOnce smem_opt_in;
  if (allow_dynamic_smem(smem_opt_in, attention_tc_kernel, kSmemBytes) != LC0B200_OK) return LC0B200_ERR_CUDA;
  TcParams p;
  p.pairs = batch * heads / 2;
  p.heads = heads;
  p.has_bias = bias != nullptr ? 1 : 0;
  p.scale = scale;
  p.status = device_status_words();
  if (p.status == nullptr) return LC0B200_ERR_CUDA;
  const long long grid = p.pairs < sm_count() ? p.pairs : sm_count();
  launch_dependent(attention_tc_kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), kSmemBytes, st, mq, mk, mv, mb, mo, p);
  return launch_status();
}

}  // namespace lc0b200
