// Internal: the two GEMM back ends behind lc0b200_gemm / lc0b200_matmul.
#pragma once

#include <cuda_runtime.h>

#include "../../include/lc0b200.h"

namespace lc0b200 {

// True when the tensor-core kernel can take the operands (TMA needs 16-byte aligned bases and pitches).
bool gemm_tcgen05_supported(const lc0b200_gemm_args& g);
int gemm_tcgen05(const lc0b200_gemm_args& g, cudaStream_t stream);
// CUDA-core kernel: any shape, pitch and alignment.
int gemm_simt(const lc0b200_gemm_args& g, cudaStream_t stream);

}  // namespace lc0b200
