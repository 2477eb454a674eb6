// lc0b200_linear_int8_static: the int8 dense layer with its temporaries in a fixed device array
// that is part of the library image, for callers that have no way to obtain device memory.
//
// Two kinds of caller are in that position.  An executor in the style of the lc0ex runtime runs
// a buffer plan that was fixed when the network was linked: every kernel gets pointers into that
// plan and nothing can be added to it at run time, so an op that needs a place for its quantised
// activations has nowhere to ask.  And a search thread that evaluates positions in a tight loop
// cannot afford cudaMalloc even where it is available: the call serialises against all work on
// the device and can fail late in a game when memory is fragmented.
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace lc0b200 {

namespace {

constexpr long long kMaxRows = LC0B200_STATIC_MAX_ROWS;
constexpr long long kMaxActBytes = LC0B200_STATIC_MAX_ACT_BYTES;
constexpr long long kScaleBytes = kMaxRows * static_cast<long long>(sizeof(float));

// [0, kScaleBytes): one f32 scale per row.  [kScaleBytes, end): int8 activations, row-major.
// Every GPU that loads the library holds this array (about 8.06 MiB) until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kScaleBytes + kMaxActBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_address[kMaxDevices] = {};

// In host code the array's name is only a handle for the runtime; the address a kernel can use
// has to be asked for, once per device, with that device current.
int scratch_on_current_device(unsigned char** base) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return LC0B200_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_static_scratch) != cudaSuccess || address == nullptr) {
      return LC0B200_ERR_CUDA;
    }
    g_scratch_address[device] = static_cast<unsigned char*>(address);
  }
  *base = g_scratch_address[device];
  return LC0B200_OK;
}

}  // namespace

}  // namespace lc0b200

using namespace lc0b200;

extern "C" LC0B200_API int lc0b200_linear_int8_static(void* out, const void* a, const void* w_nk,
                                                      const float* col_scale, const void* bias, long long m, int n,
                                                      int k, int activation, void* stream) {
  if (out == nullptr || a == nullptr || w_nk == nullptr || col_scale == nullptr) return LC0B200_ERR_NULL_POINTER;
  if (m < 0 || n <= 0 || k <= 0) return LC0B200_ERR_BAD_SHAPE;
  if (activation < LC0B200_ACT_NONE || activation > LC0B200_ACT_SWISH) return LC0B200_ERR_UNSUPPORTED;
  if (m > kMaxRows || m * static_cast<long long>(k) > kMaxActBytes) return LC0B200_ERR_SCRATCH_LIMIT;
  if (m == 0) return LC0B200_OK;
  unsigned char* base = nullptr;
  const int st = scratch_on_current_device(&base);
  if (st != LC0B200_OK) return st;
  float* scales = reinterpret_cast<float*>(base);
  void* quantised = base + kScaleBytes;
  // Nothing in the scratch has to start at zero: the rows this call uses are overwritten in full
  // by the quantiser before the GEMM reads them; rows beyond m keep whatever an earlier call left.
  return linear_int8(out, a, w_nk, col_scale, bias, quantised, scales, m, n, k, activation,
                     reinterpret_cast<cudaStream_t>(stream));
}
