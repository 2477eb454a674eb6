// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point, so the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

namespace lc0b200 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tensormap_encode_fn() {
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

// 2-D row-major tensor [rows, cols] with a row pitch (elements), tiled into [box_rows, box_cols]
// boxes; the inner box extent must equal the swizzle span (128 or 64 bytes).
//
// A tensor map is a pure function of these arguments, and a forward pass asks for the same few hundred
// maps on every call (its buffers live at fixed addresses), so each host thread keeps the maps it has
// encoded in a small direct-mapped table: a hit costs a hash and a 48-byte compare instead of a driver
// call per operand and launch.
struct TensorMapKey {
  const void* base;
  long long rows, cols, pitch;
  int elem_bytes, box_rows, box_cols, swizzle;
  bool operator==(const TensorMapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && elem_bytes == o.elem_bytes &&
           box_rows == o.box_rows && box_cols == o.box_cols && swizzle == o.swizzle;
  }
};

inline bool encode_tensormap_2d(CUtensorMap* map, const TensorMapKey& k) {
  EncodeTiledFn fn = tensormap_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k.cols), static_cast<cuuint64_t>(k.rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(k.pitch) * k.elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(k.box_cols), static_cast<cuuint32_t>(k.box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = k.elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return fn(map, dt, 2, const_cast<void*>(k.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            static_cast<CUtensorMapSwizzle>(k.swizzle), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool make_tensormap_2d(CUtensorMap* map, const void* base, int elem_bytes, long long rows, long long cols,
                              long long pitch_elems, int box_rows, int box_cols, CUtensorMapSwizzle swizzle) {
  constexpr int kSlots = 2048;  // a BT4 forward at one batch size uses about 700 distinct maps
  struct Slot {
    TensorMapKey key;
    CUtensorMap map;
    bool used;
  };
  thread_local std::vector<Slot> table;
  if (table.empty()) table.resize(kSlots);  // value-initialised: used == false
  const TensorMapKey key = {base, rows, cols, pitch_elems, elem_bytes, box_rows, box_cols, static_cast<int>(swizzle)};
  uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
  h ^= (static_cast<uint64_t>(rows) * 0xC2B2AE3D27D4EB4Full) ^ (static_cast<uint64_t>(cols) << 17) ^
       (static_cast<uint64_t>(pitch_elems) << 29) ^ (static_cast<uint64_t>(box_rows) << 41) ^
       (static_cast<uint64_t>(box_cols) << 47) ^ (static_cast<uint64_t>(elem_bytes) << 53) ^
       (static_cast<uint64_t>(swizzle) << 57);
  Slot& slot = table[(h ^ (h >> 29)) % kSlots];
  if (slot.used && slot.key == key) {
    *map = slot.map;
    return true;
  }
  if (!encode_tensormap_2d(map, key)) return false;
  slot.key = key;
  slot.map = *map;
  slot.used = true;
  return true;
}

}  // namespace lc0b200
