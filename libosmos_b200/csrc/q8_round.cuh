// The activations' rounding to int8 in blocks of 32 with four lanes a block: a lane holds eight neighbouring values
// (two 16-byte loads), the block's largest magnitude is two shuffles away, and a lane's eight codes leave as one
// 8-byte store. The rules are the contract's (kernels/lane.h:54-56, kernels/q8.h:265-277 in the reference; ggml's Q8_0
// rule: kernels/block.h:88-96): the result does not depend on how the values are spread over lanes, a maximum has no
// order.
#pragma once
#include "common.cuh"

namespace osmos {

// one 32-value block held by four neighbouring lanes (lane % 4 = the block's quarter), eight values each: returns the
// lane's eight codes packed in value order and, in *scale, the block's scale. Every lane of the warp must call it.
// GGML false: q = rint(x * (127 / amax)), scale amax / 127. GGML true: d = amax / 127, q = round(x * (1 / d)) with
// halves away from zero, scale the f16 nearest d (as F32).
template <bool GGML>
__device__ __forceinline__ uint2 round_block8(const float (&v)[8], float* scale) {
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1, kWarp));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2, kWarp));
  int code[8];
  if constexpr (GGML) {
    const float dd = __fdiv_rn(amax, 127.0f), id = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) code[j] = (int) roundf(mul_rn(v[j], id));
    *scale = __half2float(__float2half_rn(dd));
  } else {
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) code[j] = (int) rintf(mul_rn(v[j], inv));
    *scale = __fdiv_rn(amax, 127.0f);
  }
  uint2 out;
  out.x = (uint32_t) (code[0] & 0xFF) | (uint32_t) (code[1] & 0xFF) << 8 | (uint32_t) (code[2] & 0xFF) << 16 | (uint32_t) code[3] << 24;
  out.y = (uint32_t) (code[4] & 0xFF) | (uint32_t) (code[5] & 0xFF) << 8 | (uint32_t) (code[6] & 0xFF) << 16 | (uint32_t) code[7] << 24;
  return out;
}

// eight neighbouring floats: two 16-byte loads when the address allows it
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  if (((uintptr_t) p & 15u) == 0) {
    const float4 a = *(const float4*) p, b = *(const float4*) (p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = p[j];
  }
}

}  // namespace osmos
