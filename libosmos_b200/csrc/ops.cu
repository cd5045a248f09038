// The small steps around the expert FFN (include/osmos_b200/ops.h): routers, activations, gathers, the bounded
// host-flag wait and the MX activation rounding.
#include <cuda/atomic>

#include "decode.cuh"
#include "osmos_b200/mm.h"
#include "osmos_b200/ops.h"
#include "topk.cuh"

namespace osmos {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float sigmoidf(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float siluf(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float softplusf(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// a block a token: every expert's score and key through shared memory, then the first warp picks
template <int SCORE>
__global__ void __launch_bounds__(kThreads) router_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                          uint32_t n_exp, uint32_t k, float scale,
                                                          int32_t* __restrict__ idx, float* __restrict__ w) {
  __shared__ float score[OPS_MAX_EXPERTS], key[OPS_MAX_EXPERTS];
  const uint32_t t = blockIdx.x;
  for (uint32_t e = threadIdx.x; e < n_exp; e += kThreads) {
    const float l = logits[(uint64_t) t * n_exp + e];
    score[e] = SCORE == OPS_SCORE_SIGMOID ? sigmoidf(l) : sqrtf(softplusf(l));
    key[e] = order_key(__fadd_rn(score[e], bias[e]));
  }
  __syncthreads();
  if (threadIdx.x >= kWarp) return;
  const uint32_t lane = threadIdx.x;
  constexpr int kMine = OPS_MAX_EXPERTS / kWarp;
  float mine[kMine];
#pragma unroll
  for (int r = 0; r < kMine; r++) mine[r] = lane + 32u * r < n_exp ? key[lane + 32u * r] : 0.0f;
  uint32_t taken = 0;
  int32_t pick[OPS_MAX_TOPK];
  for (uint32_t s = 0; s < k; s++) {
    float best;
    pick[s] = warp_pick<kMine>(mine, n_exp, taken, best);
  }
  if (lane) return;
  float wt[OPS_MAX_TOPK], sum = 0.0f;
  for (uint32_t s = 0; s < k; s++) {
    wt[s] = (uint32_t) pick[s] < n_exp ? score[pick[s]] : 0.0f;
    sum = __fadd_rn(sum, wt[s]);
  }
  for (uint32_t s = 0; s < k; s++) {
    idx[t * k + s] = pick[s];
    w[t * k + s] = mul_rn(__fdiv_rn(wt[s], __fadd_rn(sum, 1e-20f)), scale);
  }
}

template <bool LANE>
__global__ void swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u, uint32_t n, float lim,
                              const float* __restrict__ scale, uint64_t total, float* __restrict__ h) {
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  if constexpr (LANE) {
    h[i] = lane_swiglu(g[i], u[i], lim, scale[i / n]);
  } else {
    const float gv = fminf(g[i], lim), uv = fminf(fmaxf(u[i], -lim), lim);
    const float v = mul_rn(siluf(gv), uv);
    h[i] = scale ? mul_rn(v, scale[i / n]) : v;
  }
}

__global__ void gather_rows_kernel(float* __restrict__ dst, const float* __restrict__ src, const int32_t* __restrict__ idx,
                                   uint64_t total, uint32_t len) {
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i < total) dst[i] = src[(uint64_t) idx[i / len] * len + i % len];
}

__global__ void gather_sum_kernel(float* __restrict__ y, const float* __restrict__ src, const int32_t* __restrict__ idx,
                                  uint32_t m, uint64_t total, uint32_t dim, const float* __restrict__ add) {
  pdl_wait();  // (a dependent launch: src and idx are the output of the kernels ahead)
  pdl_launch_next();
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  const uint64_t t = i / dim, c = i % dim;
  float s = 0.0f;
  for (uint32_t j = 0; j < m; j++) s = __fadd_rn(s, src[(uint64_t) idx[t * m + j] * dim + c]);
  y[i] = add ? __fadd_rn(s, add[i]) : s;
}

__global__ void copy_rows_kernel(float* __restrict__ dst, const float* __restrict__ src, const int32_t* __restrict__ idx,
                                 uint64_t total, uint32_t len) {
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  const uint64_t at = (uint64_t) idx[i / len] * len + i % len;
  dst[at] = src[at];
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
  if (score == OPS_SCORE_SIGMOID)
    router_kernel<OPS_SCORE_SIGMOID><<<n_tok, kThreads, 0, stream_of(stream)>>>(logits, bias, n_exp, k, scale, idx, w);
  else if (score == OPS_SCORE_SQRT_SOFTPLUS)
    router_kernel<OPS_SCORE_SQRT_SOFTPLUS><<<n_tok, kThreads, 0, stream_of(stream)>>>(logits, bias, n_exp, k, scale, idx, w);
  else
    return false;
  return launched();
}

extern "C" bool ops_router(const float* logits, const float* bias, uint32_t n_exp, uint32_t k, float scale,
                           uint32_t n_tok, int32_t* idx, float* w, void* stream) {
  return ops_router_scored(logits, bias, n_exp, k, scale, OPS_SCORE_SQRT_SOFTPLUS, n_tok, idx, w, stream);
}

extern "C" bool ops_swiglu_lane(const float* g, const float* u, uint32_t n, float lim, const float* scale, uint32_t n_tok,
                                float* h, void* stream) {
  if (!g || !u || !h || !n || !n_tok || !scale) return false;
  const uint64_t total = (uint64_t) n * n_tok;
  swiglu_kernel<true><<<blocks_for(total, kThreads), kThreads, 0, stream_of(stream)>>>(g, u, n, lim, scale, total, h);
  return launched();
}

extern "C" bool ops_swiglu(const float* g, const float* u, uint32_t n, float lim, const float* scale, uint32_t n_tok,
                           float* h, void* stream) {
  if (!g || !u || !h || !n || !n_tok) return false;
  const uint64_t total = (uint64_t) n * n_tok;
  swiglu_kernel<false><<<blocks_for(total, kThreads), kThreads, 0, stream_of(stream)>>>(g, u, n, lim, scale, total, h);
  return launched();
}

extern "C" bool ops_gather_rows(float* dst, const float* src, const int32_t* idx, uint32_t n, uint32_t len, void* stream) {
  if (!dst || !src || !idx || !n || !len) return false;
  const uint64_t total = (uint64_t) n * len;
  gather_rows_kernel<<<blocks_for(total, kThreads), kThreads, 0, stream_of(stream)>>>(dst, src, idx, total, len);
  return launched();
}

extern "C" bool ops_gather_sum(float* y, const float* src, const int32_t* idx, uint32_t m, uint32_t n, uint32_t dim,
                               void* stream) {
  if (!y || !src || !idx || !m || !n || !dim) return false;
  const uint64_t total = (uint64_t) n * dim;
  return launch_dependent(gather_sum_kernel, dim3(blocks_for(total, kThreads)), dim3(kThreads), 0, stream_of(stream), y, src, idx, m,
                          total, dim, (const float*) nullptr) == cudaSuccess;
}

extern "C" bool ops_gather_sum_add(float* y, const float* src, const int32_t* idx, uint32_t m, uint32_t n, uint32_t dim,
                                   const float* add, void* stream) {
  if (!y || !src || !idx || !m || !n || !dim || !add) return false;
  const uint64_t total = (uint64_t) n * dim;
  return launch_dependent(gather_sum_kernel, dim3(blocks_for(total, kThreads)), dim3(kThreads), 0, stream_of(stream), y, src, idx, m,
                          total, dim, add) == cudaSuccess;
}

extern "C" bool ops_copy_rows(float* dst, const float* src, const int32_t* idx, uint32_t n, uint32_t len, void* stream) {
  if (!dst || !src || !idx || !n || !len) return false;
  const uint64_t total = (uint64_t) n * len;
  copy_rows_kernel<<<blocks_for(total, kThreads), kThreads, 0, stream_of(stream)>>>(dst, src, idx, total, len);
  return launched();
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
