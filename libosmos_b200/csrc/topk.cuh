// A warp's top-k pick, shared by both routers: the 32 lanes hold a token's keys in registers (lane l the keys of
// experts l, l + 32, ...), one call returns the greatest key not taken yet - the lowest expert id among equals, a NaN
// key ordered below everything - to every lane, by shuffles only. Same picks, in the same order, as a serial scan in
// expert order (the rule of the reference's kernels/block.h:56-84).
#pragma once
#include "common.cuh"

namespace osmos {

constexpr int kNoPick = 0x7FFFFFFF;

__device__ __forceinline__ float order_key(float x) { return x == x ? x : __int_as_float(0xFF800000); }

// does candidate (bv, bi) lose to (ov, oi)?
__device__ __forceinline__ bool pick_loses(float bv, int bi, float ov, int oi) {
  return oi != kNoPick && (bi == kNoPick || ov > bv || (ov == bv && oi < bi));
}

template <int R>
__device__ __forceinline__ int warp_pick(const float (&v)[R], uint32_t n, uint32_t& taken, float& key) {
  const uint32_t lane = threadIdx.x % kWarp;
  float bv = __int_as_float(0xFF800000);
  int bi = kNoPick;
#pragma unroll
  for (int r = 0; r < R; r++) {
    const uint32_t e = lane + 32u * (uint32_t) r;
    if (e < n && !((taken >> r) & 1u) && (bi == kNoPick || v[r] > bv)) bv = v[r], bi = (int) e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o, kWarp);
    const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o, kWarp);
    if (pick_loses(bv, bi, ov, oi)) bv = ov, bi = oi;
  }
  if (bi != kNoPick && (uint32_t) bi % 32u == lane) taken |= 1u << ((uint32_t) bi / 32u);
  key = bv;
  return bi;
}

}  // namespace osmos
