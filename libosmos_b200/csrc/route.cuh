// Routing with a warp a token: the token's logits live in the warp's registers (lane l holds experts l, l + 32, ...),
// the softmax and the top-k never touch shared memory and a block routes as many tokens as it has warps.
//
// Two rules fix the results and both are kept:
//   - the softmax's sum is the one a 256-slot tree makes (slot i first adds experts i, i + 256, ... in order; then
//     slots i and i + s are added for s = 128, 64, ... 1). With expert e in lane e % 32 the strides 128, 64 and 32 are
//     additions between a lane's own registers and the strides 16 .. 1 are five shuffles, so the warp makes exactly
//     those additions and the probabilities have the bits of the reference's block-wide kernel
//     (kernels/q4x_moe.hip:38-52 with kernels/block.h:9-35 in the reference);
//   - a pick is the greatest key not taken yet, the lowest expert id among equal keys, a NaN key below everything
//     (kernels/block.h:56-84). Here every key becomes a 32-bit integer of the same order once, each lane remembers
//     its own best, and a pick is two warp reductions (the greatest key, then the lowest id that holds it); only the
//     lane that owned the winner looks through its registers again.
#pragma once
#include "common.cuh"

namespace osmos {
namespace route {

constexpr uint32_t kFull = 0xFFFFFFFFu;
constexpr uint32_t kNoId = 0x7FFFFFFFu;

// a float's bits as an unsigned integer of the same order (-inf lowest, +inf highest; -0 below +0)
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  const uint32_t b = __float_as_uint(v);
  return b ^ ((uint32_t) ((int32_t) b >> 31) | 0x80000000u);
}
__device__ __forceinline__ float from_ordered(uint32_t u) {
  return __uint_as_float(u ^ (((u >> 31) - 1u) | 0x80000000u));
}
// the key a value is picked by: a NaN counts as -inf, -0 as +0 (the float comparison's ties), never 0 as an integer
__device__ __forceinline__ uint32_t pick_bits(float v) {
  return ordered_bits(v == v ? __fadd_rn(v, 0.0f) : __int_as_float(0xFF800000));
}

// The warp's picker over keys u[r] (expert lane + 32 r, R registers a lane, n experts in all).
template <int R>
struct Picker {
  uint32_t taken = 0;   // bit r: this lane's expert lane + 32 r is picked
  uint32_t best = 0;    // the lane's greatest key not taken (0: none left)
  uint32_t best_id = kNoId;

  __device__ __forceinline__ void look(const uint32_t (&u)[R], uint32_t n, uint32_t lane) {
    best = 0, best_id = kNoId;
#pragma unroll
    for (int r = 0; r < R; r++) {
      const uint32_t e = lane + 32u * (uint32_t) r;
      const bool open = e < n && !((taken >> r) & 1u);
      if (open && u[r] > best) best = u[r], best_id = e;  // ascending ids, strictly greater: the lowest id among equals
    }
  }
  // the next pick, in every lane: its id, its key's bits in *key; *owner in the lane that held it (before it moves
  // on to its next best)
  __device__ __forceinline__ uint32_t next(const uint32_t (&u)[R], uint32_t n, uint32_t lane, uint32_t* key, bool* owner) {
    const uint32_t top = __reduce_max_sync(kFull, best);
    const uint32_t id = __reduce_min_sync(kFull, best == top ? best_id : kNoId);
    *owner = id == best_id && id != kNoId;
    if (*owner) {
      taken |= 1u << (id >> 5);
      look(u, n, lane);
    }
    *key = top;
    return id;
  }
};

// the 256-slot tree's sum of p[r] (expert lane + 32 r; values past n are not added), the same bits in every lane
template <int R>
__device__ __forceinline__ float tree_sum_256(const float (&p)[R], uint32_t n, uint32_t lane) {
  float slot[8];
#pragma unroll
  for (int a = 0; a < 8; a++) {
    slot[a] = 0.0f;
#pragma unroll
    for (int r = a; r < R; r += 8)
      if (lane + 32u * (uint32_t) r < n) slot[a] = __fadd_rn(slot[a], p[r]);
  }
#pragma unroll
  for (int s = 4; s > 0; s >>= 1)
#pragma unroll
    for (int a = 0; a < s; a++) slot[a] = __fadd_rn(slot[a], slot[a + s]);
  float v = slot[0];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_down_sync(kFull, v, o, kWarp));
  return __shfl_sync(kFull, v, 0, kWarp);
}

constexpr float kSumFloor = 6.103515625e-5f;  // 2^-14: the floor under the picked probabilities' sum

struct Pick {  // lane j's share of a token's result, j < k: the j-th pick
  uint32_t id;
  float w;
};

// One token's softmax router by one warp: logits l[0 .. n) -> the k greatest probabilities in pick order, lane j
// getting pick j's id and p / max(sum of the picked p, 2^-14) (k <= 32).
template <int R>
__device__ __forceinline__ Pick softmax_topk(const float* __restrict__ l, uint32_t n, uint32_t k, uint32_t lane) {
  float p[R];
  float m = __int_as_float(0xFF800000);
#pragma unroll
  for (int r = 0; r < R; r++) {
    const uint32_t e = lane + 32u * (uint32_t) r;
    p[r] = e < n ? l[e] : __int_as_float(0xFF800000);
    m = fmaxf(m, p[r]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFull, m, o, kWarp));
#pragma unroll
  for (int r = 0; r < R; r++) p[r] = lane + 32u * (uint32_t) r < n ? expf(__fsub_rn(p[r], m)) : 0.0f;
  const float inv = __fdiv_rn(1.0f, tree_sum_256<R>(p, n, lane));
  uint32_t u[R];
#pragma unroll
  for (int r = 0; r < R; r++) u[r] = pick_bits(mul_rn(p[r], inv));
  Picker<R> pk;
  pk.look(u, n, lane);
  Pick mine{0u, 0.0f};
  float total = 0.0f;  // the picked probabilities added in pick order, by every lane alike
  for (uint32_t j = 0; j < k; j++) {
    uint32_t key;
    bool owner;
    const uint32_t id = pk.next(u, n, lane, &key, &owner);
    const float v = from_ordered(key);
    total = __fadd_rn(total, v);
    if (lane == j) mine.id = id, mine.w = v;
  }
  mine.w = __fdiv_rn(mine.w, fmaxf(total, kSumFloor));
  return mine;
}

enum Score { kSqrtSoftplus = 0, kSigmoid = 1 };

// One token's scored router by one warp (DeepSeek's form): score = sqrt(softplus(logit)) or sigmoid(logit), picked by
// score + bias, lane j getting pick j's id and score / (sum of the picked scores + 1e-20) * scale
// (kernels/ops.hip:456-484 in the reference).
template <int R, int SCORE>
__device__ __forceinline__ Pick scored_topk(const float* __restrict__ l, const float* __restrict__ bias, uint32_t n,
                                            uint32_t k, float scale, uint32_t lane) {
  float sc[R];
  uint32_t u[R];
#pragma unroll
  for (int r = 0; r < R; r++) {
    const uint32_t e = lane + 32u * (uint32_t) r;
    sc[r] = 0.0f, u[r] = 0u;
    if (e < n) {
      const float x = l[e];
      if constexpr (SCORE == kSigmoid) sc[r] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
      else sc[r] = sqrtf(x > 20.0f ? x : log1pf(expf(x)));
      u[r] = pick_bits(__fadd_rn(sc[r], bias[e]));
    }
  }
  Picker<R> pk;
  pk.look(u, n, lane);
  Pick mine{0u, 0.0f};
  float sum = 0.0f;
  for (uint32_t j = 0; j < k; j++) {
    uint32_t key;
    bool owner;
    const uint32_t id = pk.next(u, n, lane, &key, &owner);
    float s = 0.0f;  // the winner's score, from the lane that holds it
#pragma unroll
    for (int r = 0; r < R; r++)
      if (owner && (uint32_t) r == (id >> 5)) s = sc[r];
    s = __shfl_sync(kFull, s, (int) (id & 31u), kWarp);
    sum = __fadd_rn(sum, s);
    if (lane == j) mine.id = id, mine.w = s;
  }
  mine.w = mul_rn(__fdiv_rn(mine.w, __fadd_rn(sum, 1e-20f)), scale);
  return mine;
}

// registers a lane needs for n experts: 4, 8, 16 or 32
__host__ __device__ inline int regs_for(uint32_t n) { return n <= 128 ? 4 : n <= 256 ? 8 : n <= 512 ? 16 : 32; }

}  // namespace route
}  // namespace osmos
