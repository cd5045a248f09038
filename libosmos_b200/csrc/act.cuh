// The libm-form activations of the f16 path and the store of one value into the tiled f16 activations
// (include/osmos_b200/mm.h: mm_x16_at), shared by the kernels that end in them (moe.cu, mm_tc.cu). Each operation is
// spelled out, so the bits do not depend on how the compiler contracts them (the reference builds with contraction
// off: kernels/block.h:86-87, kernels/mm.h:48-51).
#pragma once
#include <cuda_fp16.h>

#include <cstdint>

namespace osmos {

__device__ __forceinline__ float sigmoidf(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float siluf(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }

// value (token t, column c) of a cols-wide activation into the 16 x 16 tiled f16 layout, a value past f16 flagged
__device__ __forceinline__ void x16_store(__half* x16, int32_t* overflow, uint32_t t, uint32_t c, uint32_t cols, float v) {
  if (!(fabsf(v) <= 65504.0f)) atomicOr(overflow, 1);
  x16[(uint64_t) (t / 16) * 16 * cols + (c / 16) * 256 + (t % 16) * 16 + c % 16] = __float2half_rn(v);
}

}  // namespace osmos
