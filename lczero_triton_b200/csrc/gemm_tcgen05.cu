// Tensor-core GEMM for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma with the
// accumulator in TMEM, fused epilogue.  Replaces the reference's Triton _matmul_kernel
// (bt4/kernels/matmul.py:57-116) and, through the fused epilogue, the bias/activation kernels
// that follow it in the graph (bt4/kernels/add_bias_batched.py, add_vectors.py).
//
// One persistent CTA per SM walks output tiles of 128 x BN; for the large GEMMs two CTAs on the
// two SMs of a TPC form a cluster and share 256 x 256 tiles (tcgen05 cta_group::2: each CTA stages
// its own 128 rows of A and its own half of the weight tile, the leader CTA issues MMAs that read
// both shared memories, each CTA's TMEM receives its 128 rows of the accumulator).  That halves the
// weight traffic per CTA and deepens the pipeline from 4 to 6 stages.  No load is multicast: every
// CTA fetches its own operands with plain per-CTA TMA.  Warp roles:
//   warp 0      TMA producer   (one elected lane issues cp.async.bulk.tensor loads)
//   warp 1      MMA issuer     (one elected lane issues tcgen05.mma; owns the TMEM allocation)
//   warps 2..    epilogue      (tcgen05.ld -> bias / dequant / activation -> bf16 -> swizzled
//                              shared-memory staging -> TMA store; eight warps for BN >= 128:
//                              two per TMEM lane quarter, each taking half of the columns)
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.  bf16 results leave through cp.async.bulk.tensor stores
// (full 128-byte lines, clipped at the matrix edge by the tensor map); f32 / raw s32 results and
// unaligned outputs use direct stores.  Operands are staged K-major with the 128-byte swizzle;
// the weight operand may instead be staged MN-major straight from the reference's [K,N] layout.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "common.cuh"
#include "gemm.h"
#include "ptx.cuh"

namespace lc0b200 {

namespace {

constexpr int kBM = 128;          // tile rows = TMEM lanes
constexpr int kRowBytes = 128;    // one swizzle row: 64 bf16 or 128 int8 along K
constexpr int kStagingBytesPerWarp = 32 * kRowBytes;  // 32 rows x 64 bf16 columns

template <int BN, int CTAS>
struct TileCfg {
  static_assert(CTAS == 1 || (CTAS == 2 && BN == 256), "CTA pairs are used for 256 x 256 tiles only");
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBRows = BN / CTAS;          // weight-tile rows (N) staged by each CTA
  static constexpr int kBBytes = kBRows * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;  // power of two for BN in {32,64,128,256}
  static constexpr int kEpilogueWarps = (BN >= 128) ? 8 : 4;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
  static constexpr bool kTmaStore = BN >= 128;  // each epilogue warp then owns at least one 64-column group
  static constexpr int kStagingBytes = kTmaStore ? kEpilogueWarps * kStagingBytesPerWarp : 0;
  static constexpr int kFixedBytes = kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;
  // As many pipeline stages as fit below the 227 KB per-CTA limit (at most 8).
  static constexpr int kFit = (227 * 1024 - kFixedBytes) / kStageBytes;
  static constexpr int kStages = kFit > 8 ? 8 : kFit;
  static constexpr int kSmemBytes = kStages * kStageBytes + kFixedBytes;
};

struct KernelParams {
  void* out;
  const bf16* bias;
  const float* row_scale;
  const float* col_scale;
  long long m;
  long long ldc;
  int n;
  int k;
  int out_kind;
  int activation;
  int vec_ok;     // out / bias / col_scale are 16-byte aligned and ldc keeps rows aligned
  int tma_store;  // bf16 output that a tensor map can address (map_out is valid)
  unsigned int* status;
};

template <bool INT8>
__device__ __forceinline__ float acc_value(uint32_t raw, float rs, const float* __restrict__ cs, int col) {
  if (INT8) {
    float y = static_cast<float>(static_cast<int>(raw)) * rs;
    return cs != nullptr ? y * __ldg(cs + col) : y;
  }
  return __uint_as_float(raw);
}

// One 32-column chunk of one accumulator row: dequantise, add bias, activate, pack to bf16.
template <bool INT8>
__device__ __forceinline__ void finish_chunk_bf16(const uint32_t (&v)[32], uint32_t (&packed)[16], int col0, float rs,
                                                  const KernelParams& p) {
  const bool vec = p.vec_ok && (col0 + 32 <= p.n);
  float b[32], cs[32];
  if (vec) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint4 braw = make_uint4(0u, 0u, 0u, 0u);
      if (p.bias != nullptr) braw = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + g * 8));
      float2 t;
      t = unpack_bf16x2(braw.x); b[g * 8 + 0] = t.x; b[g * 8 + 1] = t.y;
      t = unpack_bf16x2(braw.y); b[g * 8 + 2] = t.x; b[g * 8 + 3] = t.y;
      t = unpack_bf16x2(braw.z); b[g * 8 + 4] = t.x; b[g * 8 + 5] = t.y;
      t = unpack_bf16x2(braw.w); b[g * 8 + 6] = t.x; b[g * 8 + 7] = t.y;
    }
    if (INT8) {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float4 c = make_float4(1.f, 1.f, 1.f, 1.f);
        if (p.col_scale != nullptr) c = __ldg(reinterpret_cast<const float4*>(p.col_scale + col0 + g * 4));
        cs[g * 4 + 0] = c.x; cs[g * 4 + 1] = c.y; cs[g * 4 + 2] = c.z; cs[g * 4 + 3] = c.w;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const bool in = col0 + j < p.n;
      b[j] = (in && p.bias != nullptr) ? __bfloat162float(p.bias[col0 + j]) : 0.0f;
      if (INT8) cs[j] = (in && p.col_scale != nullptr) ? p.col_scale[col0 + j] : 1.0f;
    }
  }
  float y[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float x;
    if (INT8) {
      x = (static_cast<float>(static_cast<int>(v[j])) * rs) * cs[j];
    } else {
      x = __uint_as_float(v[j]);
    }
    y[j] = x + b[j];
  }
  // The activation code is uniform for the launch: branch once per chunk, not per element.
  if (p.activation == LC0B200_ACT_MISH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = act_mish(y[j]);
  } else if (p.activation == LC0B200_ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = fmaxf(y[j], 0.0f);
  } else if (p.activation == LC0B200_ACT_SWISH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) y[j] = act_swish(y[j]);
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(y[2 * j], y[2 * j + 1]);
}

template <int BN, bool INT8, bool W_KN, int CTAS>
__global__ void __launch_bounds__(TileCfg<BN, CTAS>::kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, const KernelParams p) {
  using Cfg = TileCfg<BN, CTAS>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kElemsPerRow = INT8 ? 128 : 64;   // K elements per 128-byte row
  constexpr int kUmmaK = INT8 ? 32 : 16;          // K per tcgen05.mma (32 bytes)
  constexpr int kMmaPerStage = kElemsPerRow / kUmmaK;  // 4
  constexpr int kPanelN = INT8 ? 128 : 64;        // N elements per 128-byte row (MN-major weight staging)
  constexpr int kPanels = (Cfg::kBRows + kPanelN - 1) / kPanelN;
  constexpr int kPanelBytes = kElemsPerRow * kRowBytes;  // K rows x 128 B
  constexpr int kTileM = kBM * CTAS;              // rows of C per tile (per CTA pair when CTAS == 2)
  static_assert(!W_KN || (Cfg::kBRows % kPanelN == 0), "MN-major weight staging needs whole 128-byte panels");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = smem_base;
  const uint32_t smem_b = smem_base + kStages * Cfg::kABytes;
  const uint32_t staging_base = smem_base + kStages * Cfg::kStageBytes;  // 1024-byte aligned
  const uint32_t bar_base = staging_base + Cfg::kStagingBytes;
  const uint32_t bar_full = bar_base;                   // [kStages]  (used in the leader CTA only)
  const uint32_t bar_empty = bar_base + 8 * kStages;    // [kStages]
  const uint32_t bar_acc_full = bar_base + 16 * kStages;       // [2]
  const uint32_t bar_acc_empty = bar_base + 16 * kStages + 16; // [2]  (used in the leader CTA only)
  const uint32_t tmem_slot = bar_base + 16 * kStages + 32;
  __shared__ int abort_flag_storage;
  volatile int* abort_flag = &abort_flag_storage;

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
    abort_flag_storage = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(bar_acc_full + 8 * a, 1);
      ptx::mbar_init(bar_acc_empty + 8 * a, Cfg::kEpilogueWarps * CTAS);
    }
    ptx::mbar_init_fence();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_w);
    if (p.tma_store) ptx::prefetch_tensormap(&map_out);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (every CTA loads its own operands)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = group; tile < num_tiles && ok; tile += num_groups) {
        const int m0 = static_cast<int>(tile / n_tiles) * kTileM + static_cast<int>(rank) * kBM;
        const int n0 = static_cast<int>(tile % n_tiles) * BN + static_cast<int>(rank) * Cfg::kBRows;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = ptx::mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, 0x100u + stage);
          if (!ok) break;
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
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = ptx::instr_desc(INT8 ? 2u : 1u, 1u, W_KN ? 1u : 0u, static_cast<uint32_t>(kTileM),
                                                 static_cast<uint32_t>(BN));
      int stage = 0;
      uint32_t phase = 0;
      uint32_t local = 0;
      bool ok = true;
      for (long long tile = group; tile < num_tiles && ok; tile += num_groups, ++local) {
        const uint32_t acc = local & 1u;
        const uint32_t acc_phase = (local >> 1) & 1u;
        ok = ptx::mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, 0x200u + acc);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = ptx::mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 0x300u + stage);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = smem_a + stage * Cfg::kABytes;
          const uint32_t b_addr = smem_b + stage * Cfg::kBBytes;
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
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::tc_commit<CTAS>(bar_acc_full + 8 * acc);   // accumulator complete -> epilogue (both CTAs)
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int ew = warp - 2;
    const int quarter = warp & 3;              // TMEM lane quarter this warp may access
    const int half = ew >> 2;                  // which share of the tile's columns (eight-warp layout)
    constexpr int kColsPerWarp = BN / (Cfg::kEpilogueWarps / 4);
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t staging = staging_base + ew * kStagingBytesPerWarp;
    const bool tma_path = Cfg::kTmaStore && p.tma_store && p.out_kind == LC0B200_OUT_BF16;
    uint32_t local = 0;
    bool ok = true;
    for (long long tile = group; tile < num_tiles && ok; tile += num_groups, ++local) {
      const long long m0 = (tile / n_tiles) * kTileM + rank * kBM;
      const int n0 = static_cast<int>(tile % n_tiles) * BN + half * kColsPerWarp;
      const uint32_t acc = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      ok = ptx::mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, p.status, 0x400u + acc);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const long long row = m0 + row_in_tile;
      const bool row_ok = row < p.m;
      const float rs = (INT8 && p.row_scale != nullptr && row_ok) ? __ldg(p.row_scale + row) : 1.0f;
      const uint32_t taddr_row =
          tmem_base + acc * BN + half * kColsPerWarp + (static_cast<uint32_t>(quarter * 32) << 16);
      if (tma_path) {
        if constexpr (Cfg::kTmaStore) {
#pragma unroll 1
          for (int g = 0; g < kColsPerWarp / 64; ++g) {
            const int col0 = n0 + g * 64;
            if (col0 >= p.n) break;  // warp-uniform; a partly outside group is clipped by the store
            uint32_t v0[32], v1[32];
            ptx::tmem_ld_32x32(taddr_row + g * 64, v0);
            ptx::tmem_ld_32x32(taddr_row + g * 64 + 32, v1);
            ptx::tc_wait_ld();
            uint32_t packed[32];
            finish_chunk_bf16<INT8>(v0, *reinterpret_cast<uint32_t(*)[16]>(&packed[0]), col0, rs, p);
            finish_chunk_bf16<INT8>(v1, *reinterpret_cast<uint32_t(*)[16]>(&packed[16]), col0 + 32, rs, p);
            // The staging buffer is free once the previous store has finished reading it.
            if (lane == 0) ptx::bulk_wait_read<0>();
            __syncwarp();
            // Row `lane` of a 32 x 128-byte tile in the 128-byte swizzle the tensor map expects:
            // 16-byte chunk c of row r lives at chunk (c ^ (r & 7)).
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint32_t addr = staging + lane * kRowBytes + ((c ^ (lane & 7)) << 4);
              ptx::st_shared_v4(addr, packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_2d(&map_out, staging, col0, static_cast<int>(m0) + quarter * 32);
              ptx::bulk_commit();
            }
          }
        }
      } else {
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
            finish_chunk_bf16<INT8>(v, packed, col0, rs, p);
            bf16* dst = reinterpret_cast<bf16*>(p.out) + row * p.ldc + col0;
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
                float y = acc_value<INT8>(v[j], rs, p.col_scale, col0 + j);
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
      // TMEM has been read out: hand the accumulator back before the stores drain.
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

// LC0B200_GEMM_PAIRS=0 in the environment keeps every GEMM on the single-CTA kernel (measurement aid).
bool pair_kernels_enabled() {
  static const bool enabled = []() {
    const char* v = getenv("LC0B200_GEMM_PAIRS");
    return !(v != nullptr && v[0] == '0');
  }();
  return enabled;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// 2-D row-major tensor [rows, cols] with a row pitch, tiled into [box_rows, box_cols] boxes
// whose inner extent is exactly 128 bytes (the swizzle span).
bool make_map(CUtensorMap* map, const void* base, int elem_bytes, long long rows, long long cols,
              long long pitch_elems, int box_rows, int box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, bool INT8, bool W_KN, int CTAS>
int launch(const lc0b200_gemm_args& g, cudaStream_t stream) {
  using Cfg = TileCfg<BN, CTAS>;
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
  CUtensorMap map_out = map_a;  // placeholder when the direct-store epilogue is used
  if (tma_store && !make_map(&map_out, g.out, 2, g.m, g.n, g.ldc, 32, 64)) return LC0B200_ERR_CUDA;
  auto kernel = gemm_tcgen05_kernel<BN, INT8, W_KN, CTAS>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) {
      return LC0B200_ERR_CUDA;
    }
    configured = true;
  }
  KernelParams p;
  p.out = g.out;
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
  p.vec_ok = aligned16(g.out) && ((g.ldc * out_eb) % 16 == 0) && (g.bias_bf16 == nullptr || aligned16(g.bias_bf16)) &&
             (g.col_scale == nullptr || aligned16(g.col_scale));
  p.tma_store = tma_store ? 1 : 0;
  const long long tiles = ceil_div_ll(g.m, kBM * CTAS) * ceil_div_ll(g.n, BN);
  const long long max_groups = sm_count() / CTAS;
  const unsigned grid = static_cast<unsigned>((tiles < max_groups ? tiles : max_groups) * CTAS);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CTAS == 2 ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kernel, map_a, map_w, map_out, p) != cudaSuccess) return LC0B200_ERR_CUDA;
  return launch_status();
}

// Rows at and above which the 256-wide tiles are shared by CTA pairs (below it there are too few
// 256 x 256 tiles to fill 74 pairs and the single-CTA kernel balances better).
constexpr long long kPairMinRows = 8192;

template <bool INT8, bool W_KN>
int dispatch_bn(const lc0b200_gemm_args& g, cudaStream_t stream) {
  // MN-major weight staging needs BN to be a whole number of 128-byte panels
  // (64 bf16 or 128 int8 columns); narrower outputs just run a partly empty tile.
  constexpr int kMinBn = W_KN ? (INT8 ? 128 : 64) : 32;
  if (g.n > 128) {
    if (g.m >= kPairMinRows && pair_kernels_enabled()) return launch<256, INT8, W_KN, 2>(g, stream);
    return launch<256, INT8, W_KN, 1>(g, stream);
  }
  if constexpr (kMinBn <= 128) {
    if (g.n > 64 || kMinBn == 128) return launch<128, INT8, W_KN, 1>(g, stream);
  }
  if constexpr (kMinBn <= 64) {
    if (g.n > 32 || kMinBn == 64) return launch<64, INT8, W_KN, 1>(g, stream);
  }
  if constexpr (kMinBn <= 32) {
    return launch<32, INT8, W_KN, 1>(g, stream);
  }
  return LC0B200_ERR_UNSUPPORTED;
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
  if (int8) return w_kn ? dispatch_bn<true, true>(g, stream) : dispatch_bn<true, false>(g, stream);
  return w_kn ? dispatch_bn<false, true>(g, stream) : dispatch_bn<false, false>(g, stream);
}

}  // namespace lc0b200
