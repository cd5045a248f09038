// The small steps around the expert FFN (include/osmos_b200/ops.h): routers, activations, gathers, the bounded
// host-flag wait and the MX activation rounding.
#include <cuda/atomic>

#include "decode.cuh"
#include "osmos_b200/mm.h"
#include "osmos_b200/ops.h"
#include "route.cuh"

#include <initializer_list>

namespace osmos {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float sigmoidf(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float siluf(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }

// a warp a token (route.cuh): scores and keys in the warp's registers, four tokens a block
constexpr int kRouteWarps = 4;
template <int R, int SCORE>
__global__ void __launch_bounds__(kRouteWarps* kWarp) router_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                                    uint32_t n_tok, uint32_t n_exp, uint32_t k, float scale,
                                                                    int32_t* __restrict__ idx, float* __restrict__ w) {
  const uint32_t t = blockIdx.x * kRouteWarps + threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
  if (t >= n_tok) return;  // (the whole warp)
  const route::Pick p = route::scored_topk<R, SCORE>(logits + (uint64_t) t * n_exp, bias, n_exp, k, scale, lane);
  if (lane < k) idx[t * k + lane] = (int32_t) p.id, w[t * k + lane] = p.w;
}

template <int SCORE>
bool launch_router(const float* logits, const float* bias, uint32_t n_exp, uint32_t k, float scale, uint32_t n_tok, int32_t* idx,
                   float* w, cudaStream_t s) {
  const dim3 grid(blocks_for(n_tok, kRouteWarps)), block(kRouteWarps * kWarp);
  switch (route::regs_for(n_exp)) {
    case 4: router_kernel<4, SCORE><<<grid, block, 0, s>>>(logits, bias, n_tok, n_exp, k, scale, idx, w); break;
    case 8: router_kernel<8, SCORE><<<grid, block, 0, s>>>(logits, bias, n_tok, n_exp, k, scale, idx, w); break;
    case 16: router_kernel<16, SCORE><<<grid, block, 0, s>>>(logits, bias, n_tok, n_exp, k, scale, idx, w); break;
    default: router_kernel<32, SCORE><<<grid, block, 0, s>>>(logits, bias, n_tok, n_exp, k, scale, idx, w); break;
  }
  return launched();
}

// The elementwise steps take rows of n (or len, dim) values. Where the rows and every address are whole 16-byte words a
// thread handles four neighbouring values of one row (VEC 4: one load / store a tensor), else one (VEC 1). The
// operations on each value are the same either way, so are the bits.
template <int VEC> struct Pack;
template <> struct Pack<1> {
  float v[1];
  __device__ __forceinline__ void load(const float* p) { v[0] = *p; }
  __device__ __forceinline__ void store(float* p) const { *p = v[0]; }
};
template <> struct Pack<4> {
  float v[4];
  __device__ __forceinline__ void load(const float* p) {
    const float4 a = *(const float4*) p;
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
  }
  __device__ __forceinline__ void store(float* p) const { *(float4*) p = make_float4(v[0], v[1], v[2], v[3]); }
};
__host__ inline bool words16(uint32_t row_len, std::initializer_list<const void*> ptrs) {
  if (row_len % 4) return false;
  for (const void* p : ptrs)
    if ((uintptr_t) p & 15u) return false;
  return true;
}

template <bool LANE, int VEC>
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u, uint32_t n,
                                                          float lim, const float* __restrict__ scale, uint64_t total,
                                                          float* __restrict__ h) {
  const uint64_t i = ((uint64_t) blockIdx.x * kThreads + threadIdx.x) * VEC;
  if (i >= total) return;
  Pack<VEC> a, b, o;
  a.load(g + i), b.load(u + i);
  const float sc = scale ? scale[i / n] : 1.0f;
#pragma unroll
  for (int j = 0; j < VEC; j++) {
    if constexpr (LANE) {
      o.v[j] = lane_swiglu(a.v[j], b.v[j], lim, sc);
    } else {
      const float gv = fminf(a.v[j], lim), uv = fminf(fmaxf(b.v[j], -lim), lim);
      const float v = mul_rn(siluf(gv), uv);
      o.v[j] = scale ? mul_rn(v, sc) : v;
    }
  }
  o.store(h + i);
}

// dst[i][:] = src[idx[i]][:] (SCATTER false), or rows idx[i] of src to the same rows of dst (SCATTER true)
template <bool SCATTER, int VEC>
__global__ void __launch_bounds__(kThreads) rows_kernel(float* __restrict__ dst, const float* __restrict__ src,
                                                        const int32_t* __restrict__ idx, uint64_t total, uint32_t len) {
  const uint64_t i = ((uint64_t) blockIdx.x * kThreads + threadIdx.x) * VEC;
  if (i >= total) return;
  const uint64_t from = (uint64_t) idx[i / len] * len + i % len;
  Pack<VEC> v;
  v.load(src + from);
  v.store(dst + (SCATTER ? from : i));
}

template <int VEC>
__global__ void __launch_bounds__(kThreads) gather_sum_kernel(float* __restrict__ y, const float* __restrict__ src,
                                                              const int32_t* __restrict__ idx, uint32_t m, uint64_t total,
                                                              uint32_t dim, const float* __restrict__ add) {
  pdl_wait();  // (a dependent launch: src and idx are the output of the kernels ahead)
  pdl_launch_next();
  const uint64_t i = ((uint64_t) blockIdx.x * kThreads + threadIdx.x) * VEC;
  if (i >= total) return;
  const uint64_t t = i / dim, c = i % dim;
  Pack<VEC> s, v;
#pragma unroll
  for (int j = 0; j < VEC; j++) s.v[j] = 0.0f;
  for (uint32_t j = 0; j < m; j++) {  // the rows in j's order, from 0
    v.load(src + (uint64_t) idx[t * m + j] * dim + c);
#pragma unroll
    for (int q = 0; q < VEC; q++) s.v[q] = __fadd_rn(s.v[q], v.v[q]);
  }
  if (add) {
    v.load(add + i);
#pragma unroll
    for (int q = 0; q < VEC; q++) s.v[q] = __fadd_rn(s.v[q], v.v[q]);
  }
  s.store(y + i);
}

// bit 0: a wait ran out. one word a device (device memory: each device that loads the library has its own copy)
__device__ uint32_t g_wait_status;

// one thread polls the host's word with system-scope acquire loads, napping between looks, until it holds the value
// (with or without the poster's failure bit) or the time is up
__global__ void wait_kernel(const uint32_t* flag, uint32_t value, uint64_t limit_ns) {
  const cuda::atomic_ref<const uint32_t, cuda::thread_scope_system> word(*flag);
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    const uint32_t v = word.load(cuda::std::memory_order_acquire);
    if ((v & 0x7FFFFFFFu) == value) return;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 > limit_ns) {
      atomicOr(&g_wait_status, 1u);
      return;
    }
    __nanosleep(200);
  }
}

// ---- MX activation rounding --------------------------------------------------------------------------------------
__device__ __forceinline__ float e2m1_round(float v) {
  const float a = fabsf(v);
  const float q = a <= 0.25f ? 0.0f : a < 0.75f ? 0.5f : a <= 1.25f ? 1.0f : a < 1.75f ? 1.5f
                : a <= 2.5f ? 2.0f : a < 3.5f ? 3.0f : a <= 5.0f ? 4.0f : 6.0f;
  return copysignf(q, v);
}
__device__ __forceinline__ uint32_t e2m1_code(float q) {
  const float a = fabsf(q);
  const uint32_t i = a == 0.0f ? 0 : a == 0.5f ? 1 : a == 1.0f ? 2 : a == 1.5f ? 3 : a == 2.0f ? 4 : a == 3.0f ? 5 : a == 4.0f ? 6 : 7;
  return (__float_as_uint(q) >> 31) << 3 | i;
}
__device__ __forceinline__ float e4m3_round(float x) {
  const float a = fabsf(x);
  float q;
  if (a < 0.015625f) {
    q = mul_rn(rintf(__fdiv_rn(a, 0.001953125f)), 0.001953125f);
  } else {
    int e;
    frexpf(a, &e);
    const float step = ldexpf(1.0f, e - 4);
    q = mul_rn(rintf(__fdiv_rn(a, step)), step);
  }
  return copysignf(q, x);
}
__device__ __forceinline__ uint32_t e4m3_code(float q) {
  const uint32_t sign = __float_as_uint(q) >> 31 << 7;
  const float a = fabsf(q);
  if (a < 0.015625f) return sign | (uint32_t) mul_rn(a, 512.0f);
  int e;
  const float m = frexpf(a, &e);
  return sign | (uint32_t) (e + 6) << 3 | (uint32_t) mul_rn(__fsub_rn(mul_rn(m, 2.0f), 1.0f), 8.0f);
}
__device__ __forceinline__ float warp_amax(float m) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o, kWarp));
  return m;
}

// a warp a block (at most 32 values, a lane a value)
__global__ void __launch_bounds__(kThreads) fp4_kernel(float* x, uint64_t blocks, uint32_t block, bool e4m3_scale,
                                                       uint8_t* packed, uint32_t dim) {
  const uint64_t b = (uint64_t) blockIdx.x * (kThreads / kWarp) + threadIdx.x / kWarp;
  if (b >= blocks) return;
  const uint32_t lane = threadIdx.x % kWarp;
  float* v = x + b * block;
  const bool mine = lane < block;
  const float val = mine ? v[lane] : 0.0f;
  const float amax = warp_amax(fabsf(val));
  float s;
  if (e4m3_scale)
    s = e4m3_round(__fdiv_rn(fmaxf(amax, 6.0f * 0.001953125f), 6.0f));
  else
    s = exp2f(ceilf(log2f(__fdiv_rn(fmaxf(amax, 6.0f * 1.1754943508222875e-38f), 6.0f))));
  const float q = e2m1_round(fminf(fmaxf(__fdiv_rn(val, s), -6.0f), 6.0f));
  if (mine) v[lane] = mul_rn(q, s);
  if (!packed) return;
  const uint32_t code = e2m1_code(q);
  const uint32_t pair = __shfl_xor_sync(0xFFFFFFFFu, code, 1, kWarp);
  const uint64_t i = b * block + lane;
  uint8_t* row = packed + i / dim * (dim / 2 + dim / block);
  const uint32_t j = (uint32_t) (i % dim);
  if (mine && lane % 2 == 0) row[j / 2] = (uint8_t) (code | pair << 4);
  if (lane == 0)
    row[dim / 2 + j / block] = (uint8_t) (e4m3_scale ? (s > 448.0f ? 0x7Fu : e4m3_code(s)) : (uint32_t) (ilogbf(s) + 127));
}

// MXFP4 rows for the W4A4 product (32-value blocks, E8M0 scales, packed output): eight lanes a block, four values a
// lane - one 16-byte load, two shuffles for the block's largest magnitude, the rounded values back as one 16-byte
// store and the lane's four codes as one 2-byte store. The same operations a value as fp4_kernel (a power-of-two scale
// divides exactly, so the quotient is a product with its reciprocal), hence the same bits.
__global__ void __launch_bounds__(kThreads) mxfp4_rows_kernel(float* x, uint64_t blocks, uint8_t* packed, uint32_t dim) {
  const uint64_t t = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  const uint64_t b = t / 8;
  const uint32_t part = (uint32_t) (t % 8);
  const bool live = b < blocks;  // (eight lanes are live or not together; the shuffles want every lane)
  float4* at = (float4*) (x + (live ? b : 0) * 32) + part;
  const float4 v = live ? *at : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o, kWarp));
  const float s = exp2f(ceilf(log2f(__fdiv_rn(fmaxf(amax, 6.0f * 1.1754943508222875e-38f), 6.0f))));
  const float r = __fdiv_rn(1.0f, s);
  const float in[4] = {v.x, v.y, v.z, v.w};
  float q[4];
  uint32_t codes = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    q[i] = e2m1_round(fminf(fmaxf(mul_rn(in[i], r), -6.0f), 6.0f));
    codes |= e2m1_code(q[i]) << (4 * i);
  }
  if (!live) return;
  *at = make_float4(mul_rn(q[0], s), mul_rn(q[1], s), mul_rn(q[2], s), mul_rn(q[3], s));
  const uint64_t row = b * 32 / dim;
  const uint32_t j = (uint32_t) (b * 32 - row * dim);  // the block's first column
  uint8_t* out = packed + row * (dim / 2 + dim / 32);
  *(uint16_t*) (out + j / 2 + 2 * part) = (uint16_t) codes;
  if (part == 0) out[dim / 2 + j / 32] = (uint8_t) (ilogbf(s) + 127);
}

__global__ void __launch_bounds__(kThreads) fp8_kernel(float* x, uint64_t blocks, uint8_t* packed, uint32_t dim) {
  const uint64_t b = (uint64_t) blockIdx.x * (kThreads / kWarp) + threadIdx.x / kWarp;
  if (b >= blocks) return;
  const uint64_t i = b * 32 + threadIdx.x % kWarp;
  const float val = x[i];
  const float amax = warp_amax(fabsf(val));
  const float s = exp2f(ceilf(log2f(__fdiv_rn(fmaxf(amax, 1e-4f), 448.0f))));
  const float q = e4m3_round(fminf(fmaxf(__fdiv_rn(val, s), -448.0f), 448.0f));
  x[i] = mul_rn(q, s);
  if (!packed) return;
  uint8_t* row = packed + i / dim * (dim + dim / 32);
  const uint32_t j = (uint32_t) (i % dim);
  row[j] = (uint8_t) e4m3_code(q);
  if (j % 32 == 0) row[dim + j / 32] = (uint8_t) (ilogbf(s) + 127);
}

// mm_x16_attn: a warp a 32-value block of a token's row, a lane a value - each head's last rope_dim values rotated back
// by the token's position (a pair's lanes trade values), the block rounded to E4M3 under its power-of-two scale, then
// to f16 in the tiled layout; the tile's rows past the last token zero (kernels/mm.hip:105-135 in the reference)
__global__ void __launch_bounds__(kThreads) x16_attn_kernel(const float* __restrict__ x, uint32_t xs, uint32_t n, uint32_t n16,
                                                            uint32_t cols, uint32_t head_dim, uint32_t rope_dim,
                                                            const float* __restrict__ freqs, const int32_t* __restrict__ pos,
                                                            __half* __restrict__ x16, int32_t* overflow) {
  const uint64_t blk = (uint64_t) blockIdx.x * (kThreads / kWarp) + threadIdx.x / kWarp;
  const uint32_t lane = threadIdx.x % kWarp, per_row = cols / 32;
  const uint32_t t = (uint32_t) (blk / per_row), c = (uint32_t) (blk % per_row) * 32 + lane;
  if (t >= n16) return;  // (the whole warp: a block is one token's)
  float v = 0.0f;
  if (t < n) {
    v = x[(uint64_t) t * xs + c];
    const uint32_t d = c % head_dim, r0 = head_dim - rope_dim;
    if (d >= r0) {  // the whole block lies in the rotated part (r0 is a multiple of 32)
      const float other = __shfl_xor_sync(0xFFFFFFFFu, v, 1, kWarp);
      const float ang = mul_rn((float) pos[t], freqs[(d - r0) / 2]);
      const float cs = cosf(ang), sn = -sinf(ang);
      const float a = lane & 1 ? other : v, b = lane & 1 ? v : other;
      v = lane & 1 ? __fadd_rn(mul_rn(a, sn), mul_rn(b, cs)) : __fsub_rn(mul_rn(a, cs), mul_rn(b, sn));
    }
    const float amax = warp_amax(fabsf(v));
    const float s = exp2f(ceilf(log2f(__fdiv_rn(fmaxf(amax, 1e-4f), 448.0f))));
    v = mul_rn(e4m3_round(fminf(fmaxf(__fdiv_rn(v, s), -448.0f), 448.0f)), s);
  }
  if (!(fabsf(v) <= 65504.0f)) atomicOr(overflow, 1);
  x16[mm_x16_at(t, c, cols)] = __float2half_rn(v);
}

uint32_t g_wait_limit_ms = 2000;

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" bool ops_router_scored(const float* logits, const float* bias, uint32_t n_exp, uint32_t k, float scale,
                                  OpsScore score, uint32_t n_tok, int32_t* idx, float* w, void* stream) {
  if (!logits || !bias || !idx || !w || !n_exp || n_exp > OPS_MAX_EXPERTS || !k || k > OPS_MAX_TOPK || k > n_exp || !n_tok)
    return false;
  if (score == OPS_SCORE_SIGMOID) return launch_router<route::kSigmoid>(logits, bias, n_exp, k, scale, n_tok, idx, w, stream_of(stream));
  if (score == OPS_SCORE_SQRT_SOFTPLUS)
    return launch_router<route::kSqrtSoftplus>(logits, bias, n_exp, k, scale, n_tok, idx, w, stream_of(stream));
  return false;
}

extern "C" bool ops_router(const float* logits, const float* bias, uint32_t n_exp, uint32_t k, float scale,
                           uint32_t n_tok, int32_t* idx, float* w, void* stream) {
  return ops_router_scored(logits, bias, n_exp, k, scale, OPS_SCORE_SQRT_SOFTPLUS, n_tok, idx, w, stream);
}

template <bool LANE>
static bool swiglu_rows(const float* g, const float* u, uint32_t n, float lim, const float* scale, uint32_t n_tok, float* h,
                        cudaStream_t s) {
  const uint64_t total = (uint64_t) n * n_tok;
  if (words16(n, {g, u, h}))
    swiglu_kernel<LANE, 4><<<blocks_for(total / 4, kThreads), kThreads, 0, s>>>(g, u, n, lim, scale, total, h);
  else
    swiglu_kernel<LANE, 1><<<blocks_for(total, kThreads), kThreads, 0, s>>>(g, u, n, lim, scale, total, h);
  return launched();
}

extern "C" bool ops_swiglu_lane(const float* g, const float* u, uint32_t n, float lim, const float* scale, uint32_t n_tok,
                                float* h, void* stream) {
  if (!g || !u || !h || !n || !n_tok || !scale) return false;
  return swiglu_rows<true>(g, u, n, lim, scale, n_tok, h, stream_of(stream));
}

extern "C" bool ops_swiglu(const float* g, const float* u, uint32_t n, float lim, const float* scale, uint32_t n_tok,
                           float* h, void* stream) {
  if (!g || !u || !h || !n || !n_tok) return false;
  return swiglu_rows<false>(g, u, n, lim, scale, n_tok, h, stream_of(stream));
}

template <bool SCATTER>
static bool move_rows(float* dst, const float* src, const int32_t* idx, uint32_t n, uint32_t len, cudaStream_t s) {
  const uint64_t total = (uint64_t) n * len;
  if (words16(len, {dst, src}))
    rows_kernel<SCATTER, 4><<<blocks_for(total / 4, kThreads), kThreads, 0, s>>>(dst, src, idx, total, len);
  else
    rows_kernel<SCATTER, 1><<<blocks_for(total, kThreads), kThreads, 0, s>>>(dst, src, idx, total, len);
  return launched();
}

extern "C" bool ops_gather_rows(float* dst, const float* src, const int32_t* idx, uint32_t n, uint32_t len, void* stream) {
  if (!dst || !src || !idx || !n || !len) return false;
  return move_rows<false>(dst, src, idx, n, len, stream_of(stream));
}

static bool gather_sum(float* y, const float* src, const int32_t* idx, uint32_t m, uint32_t n, uint32_t dim, const float* add,
                       cudaStream_t s) {
  const uint64_t total = (uint64_t) n * dim;
  if (words16(dim, {y, src, add}))
    return launch_dependent(gather_sum_kernel<4>, dim3(blocks_for(total / 4, kThreads)), dim3(kThreads), 0, s, y, src, idx, m, total,
                            dim, add) == cudaSuccess;
  return launch_dependent(gather_sum_kernel<1>, dim3(blocks_for(total, kThreads)), dim3(kThreads), 0, s, y, src, idx, m, total, dim,
                          add) == cudaSuccess;
}

extern "C" bool ops_gather_sum(float* y, const float* src, const int32_t* idx, uint32_t m, uint32_t n, uint32_t dim,
                               void* stream) {
  if (!y || !src || !idx || !m || !n || !dim) return false;
  return gather_sum(y, src, idx, m, n, dim, nullptr, stream_of(stream));
}

extern "C" bool ops_gather_sum_add(float* y, const float* src, const int32_t* idx, uint32_t m, uint32_t n, uint32_t dim,
                                   const float* add, void* stream) {
  if (!y || !src || !idx || !m || !n || !dim || !add) return false;
  return gather_sum(y, src, idx, m, n, dim, add, stream_of(stream));
}

extern "C" bool ops_copy_rows(float* dst, const float* src, const int32_t* idx, uint32_t n, uint32_t len, void* stream) {
  if (!dst || !src || !idx || !n || !len) return false;
  return move_rows<true>(dst, src, idx, n, len, stream_of(stream));
}

extern "C" void ops_wait_set_limit_ms(uint32_t ms) { g_wait_limit_ms = ms ? ms : 1; }
extern "C" uint32_t ops_wait_limit_ms(void) { return g_wait_limit_ms; }

extern "C" bool ops_wait(const uint32_t* flag, uint32_t value, void* stream) {
  if (!flag) return false;
  wait_kernel<<<1, 1, 0, stream_of(stream)>>>(flag, value, (uint64_t) g_wait_limit_ms * 1000000ull);
  return launched();
}

extern "C" uint32_t ops_wait_status(void) {
  uint32_t v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_wait_status, sizeof v) != cudaSuccess) return 0x80000000u;
  cudaMemcpyToSymbol(g_wait_status, &zero, sizeof zero);
  return v;
}

extern "C" bool ops_fp4_round(float* x, uint64_t n, uint32_t block, bool e4m3_scale, void* packed, uint32_t dim,
                              void* stream) {
  if (!x || !n || !block || n % block || block > 32) return false;
  if (packed && (!dim || dim % block || dim % 4 || n % dim || block != (e4m3_scale ? 16u : 32u))) return false;
  if (packed && !e4m3_scale && ((uintptr_t) x & 15u) == 0 && ((uintptr_t) packed & 1u) == 0 && dim % 64 == 0) {
    // (whole rows of an even number of blocks: every block's codes start on 2 bytes)
    mxfp4_rows_kernel<<<blocks_for(n / 32 * 8, kThreads), kThreads, 0, stream_of(stream)>>>(x, n / 32, (uint8_t*) packed, dim);
    return launched();
  }
  fp4_kernel<<<blocks_for(n / block, kThreads / kWarp), kThreads, 0, stream_of(stream)>>>(x, n / block, block, e4m3_scale,
                                                                                       (uint8_t*) packed, dim);
  return launched();
}

extern "C" bool mm_x16_attn(const float* x, uint32_t xs, uint32_t n, uint32_t cols, uint32_t head_dim, uint32_t rope_dim,
                            const float* freqs, const int32_t* pos, void* x16, int32_t* overflow, void* stream) {
  if (!x || !x16 || !overflow || !n || n > MM_MAX_TOKENS || !cols || cols % MM_TILE || (n > 1 && xs < cols) || !head_dim ||
      cols % head_dim || head_dim % 32 || rope_dim > head_dim || rope_dim % 2 || (head_dim - rope_dim) % 32 ||
      (rope_dim && (!freqs || !pos)))
    return false;
  const uint32_t n16 = (n + MM_TILE - 1) / MM_TILE * MM_TILE;
  x16_attn_kernel<<<blocks_for((uint64_t) n16 * (cols / 32), kThreads / kWarp), kThreads, 0, stream_of(stream)>>>(
      x, xs, n, n16, cols, head_dim, rope_dim, freqs, pos, (__half*) x16, overflow);
  return launched();
}

extern "C" bool ops_fp8_round(float* x, uint64_t n, void* packed, uint32_t dim, void* stream) {
  if (!x || !n || n % 32 || (packed && (!dim || dim % 32 || dim % 4 || n % dim))) return false;
  fp8_kernel<<<blocks_for(n / 32, kThreads / kWarp), kThreads, 0, stream_of(stream)>>>(x, n / 32, (uint8_t*) packed, dim);
  return launched();
}
