// NVFP4's own matvec for a few tokens (mv_fp4, mv_fp4_tok in include/osmos_b200/mv.h): the order of sums of the
// reference's kernels/mv_fp4.hip, not mv_run's.
//
// A row's 64-value blocks (36 bytes: four UE4M3 scales, then 32 bytes of E2M1 - sub-block s's value j in the low
// nibble of byte 4 + 8 s + j, value j + 8 in its high nibble) go to G lanes, lane l taking blocks l, l + G, ...; a
// block adds its four sub-blocks in turn (part over the 8 byte pairs, then acc = fmaf(d, part, acc) with d the scale
// halved and the E2M1 values doubled, every product exact); the G lanes meet in the xor tree. One kernel serves the
// dense entry (G 32, the tensor's scale on the sum) and the grouped one (G 8, 16 or 32 by the row's length).
#include "decode.cuh"
#include "osmos_b200/mv.h"

namespace osmos {
namespace {

constexpr int kWarps = 8, kThreads = kWarps * kWarp;
constexpr int kBlockValues = 64, kBlockWords = 9;

struct Fp4Args {
  const uint8_t* w;          // dense
  const uint8_t* const* wt;  // grouped
  const int32_t *cnt, *xrow;
  const float* x;
  float* y;
  uint32_t rows, cols, xs, ys, n_tok;
  float scale;
  int use_scale;
};

// the sixteen doubled E2M1 values, a copy in shared memory: a warp's lanes look up different codes, which constant
// memory would serve one address at a time
__device__ __forceinline__ void stage_values(float* tab) {
  if (threadIdx.x < 16) tab[threadIdx.x] = (float) osmos_e2m1_doubled[threadIdx.x];
  __syncthreads();
}

// rows of matrix w over NT tokens of x, G lanes a row
template <int G, int NT>
__device__ __forceinline__ void fp4_rows(const uint8_t* w, uint32_t rows, uint32_t cols, const float* x, uint32_t xs,
                                         float* y, uint32_t ys, float scale, int use_scale, const float* tab) {
  const uint32_t lane = threadIdx.x % kWarp, sub = lane % G;
  const uint32_t r = (blockIdx.x * kWarps + threadIdx.x / kWarp) * (kWarp / G) + lane / G;
  const uint32_t nb = cols / kBlockValues;
  const bool live = r < rows;
  float acc[NT];
#pragma unroll
  for (int t = 0; t < NT; t++) acc[t] = 0.0f;
  for (uint32_t b = sub; live && b < nb; b += G) {
    const uint32_t* p = (const uint32_t*) (w + ((uint64_t) r * nb + b) * (kBlockWords * 4));
    uint32_t q[kBlockWords];
#pragma unroll
    for (int k = 0; k < kBlockWords; k++) q[k] = __ldg(p + k);
#pragma unroll
    for (int s = 0; s < 4; s++) {
      const float d = mul_rn(ue4m3_value((q[0] >> (8 * s)) & 0xFFu), 0.5f);
      const uint32_t lo = q[1 + 2 * s], hi = q[2 + 2 * s];
      float part[NT];
#pragma unroll
      for (int t = 0; t < NT; t++) part[t] = 0.0f;
#pragma unroll
      for (int half = 0; half < 2; half++) {
        float xa[NT][4], xc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; t++) {
          const float* xp = x + (uint64_t) t * xs + (uint64_t) b * kBlockValues + 16 * s + 4 * half;
          const float4 va = __ldg((const float4*) xp), vc = __ldg((const float4*) (xp + 8));
          xa[t][0] = va.x, xa[t][1] = va.y, xa[t][2] = va.z, xa[t][3] = va.w;
          xc[t][0] = vc.x, xc[t][1] = vc.y, xc[t][2] = vc.z, xc[t][3] = vc.w;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const uint32_t byte = ((half ? hi : lo) >> (8 * j)) & 0xFFu;
          const float a = tab[byte & 0xF], c = tab[byte >> 4];
#pragma unroll
          for (int t = 0; t < NT; t++) part[t] = __fmaf_rn(a, xa[t][j], __fmaf_rn(c, xc[t][j], part[t]));
        }
      }
#pragma unroll
      for (int t = 0; t < NT; t++) acc[t] = __fmaf_rn(d, part[t], acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < NT; t++) {
    float v = acc[t];
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, o, kWarp));
    if (sub == 0 && live) y[(uint64_t) t * ys + r] = use_scale ? mul_rn(v, scale) : v;
  }
}

template <int NT>
__global__ void __launch_bounds__(kThreads) fp4_dense_kernel(const Fp4Args a) {
  __shared__ float tab[16];
  stage_values(tab);
  fp4_rows<kWarp, NT>(a.w, a.rows, a.cols, a.x, a.xs, a.y, a.ys, a.scale, a.use_scale, tab);
}

template <int G>
__global__ void __launch_bounds__(kThreads) fp4_tok_kernel(const Fp4Args a) {
  __shared__ float tab[16];
  stage_values(tab);
  const uint32_t e = blockIdx.y;
  const int32_t c = a.cnt[e];
  if (c < 1 || c > 4) return;  // an entry of count 0 is skipped: nothing read or written (the whole block)
  const uint8_t* m = a.wt[e];
  const float* xe = a.x + (uint64_t) a.xrow[e] * a.xs;
  float* ye = a.y + (uint64_t) a.xrow[e] * a.ys;
  switch (c) {
    case 1: fp4_rows<G, 1>(m, a.rows, a.cols, xe, a.xs, ye, a.ys, 1.0f, 0, tab); break;
    case 2: fp4_rows<G, 2>(m, a.rows, a.cols, xe, a.xs, ye, a.ys, 1.0f, 0, tab); break;
    case 3: fp4_rows<G, 3>(m, a.rows, a.cols, xe, a.xs, ye, a.ys, 1.0f, 0, tab); break;
    default: fp4_rows<G, 4>(m, a.rows, a.cols, xe, a.xs, ye, a.ys, 1.0f, 0, tab); break;
  }
}

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" bool mv_fp4(const void* w, uint32_t rows, uint32_t cols, const float* x, uint32_t xs, uint32_t n, float* y,
                       uint32_t ys, float scale, void* stream) {
  if (!w || !x || !y || !rows || !cols || cols % kBlockValues || xs % 4 || n < 1 || n > 4) return false;
  if (((uintptr_t) x & 15u) || ((uintptr_t) w & 3u)) return false;
  Fp4Args a{};
  a.w = (const uint8_t*) w, a.x = x, a.y = y, a.rows = rows, a.cols = cols, a.xs = xs, a.ys = ys, a.n_tok = n;
  a.scale = scale, a.use_scale = 1;
  const unsigned grid = blocks_for(rows, kWarps);
  const cudaStream_t s = stream_of(stream);
  switch (n) {
    case 1: fp4_dense_kernel<1><<<grid, kThreads, 0, s>>>(a); break;
    case 2: fp4_dense_kernel<2><<<grid, kThreads, 0, s>>>(a); break;
    case 3: fp4_dense_kernel<3><<<grid, kThreads, 0, s>>>(a); break;
    default: fp4_dense_kernel<4><<<grid, kThreads, 0, s>>>(a); break;
  }
  return launched();
}

extern "C" bool mv_fp4_tok(const void* const* w, const int32_t* cnt, const int32_t* xrow, uint32_t n, uint32_t rows,
                           uint32_t cols, const float* x, uint32_t xs, float* y, uint32_t ys, void* stream) {
  if (!w || !cnt || !xrow || !x || !y || !n || n > 65535 || !rows || !cols || cols % kBlockValues || xs % 4) return false;
  if ((uintptr_t) x & 15u) return false;
  Fp4Args a{};
  a.wt = (const uint8_t* const*) w, a.cnt = cnt, a.xrow = xrow, a.x = x, a.y = y, a.rows = rows, a.cols = cols;
  a.xs = xs, a.ys = ys;
  const uint32_t nb = cols / kBlockValues;
  const cudaStream_t s = stream_of(stream);
  if (nb <= 24) fp4_tok_kernel<8><<<dim3(blocks_for(rows, kWarps * 4), n), kThreads, 0, s>>>(a);
  else if (nb <= 48) fp4_tok_kernel<16><<<dim3(blocks_for(rows, kWarps * 2), n), kThreads, 0, s>>>(a);
  else fp4_tok_kernel<32><<<dim3(blocks_for(rows, kWarps), n), kThreads, 0, s>>>(a);
  return launched();
}
