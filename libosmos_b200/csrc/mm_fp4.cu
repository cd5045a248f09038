// NVFP4 weights times NVFP4 activations (W4A4): mm_fp4_ok, mm_fp4_act, mm_fp4_quant, mm_fp4 of include/osmos_b200/mm.h,
// for the reference's kernels/mm_fp4.hip:23-104 (the activations' quantization), :149-259 and :399-445 (the product).
//
// The quantization is the reference's rule, bit for bit: every 16 values one E4M3 scale - amax / 6 / gs to nearest
// even, at most 448 - and E2M1 codes of value / (scale gs) clamped to +-6, to nearest with ties to the even index, or
// stochastically under a seed; codes two a byte in k order, the low nibble first.
//
// The product: an E2M1 value times an E4M3 scale has at most 6 significant bits and lies between 2^-10 and 2688, so it
// is exactly an f16 - on either side. The codes are expanded to the tiled f16 layout (exactly; a stream-ordered
// scratch allocation holds them) and multiplied by the f16 tensor-core product of mm_tc.cu, whose weight side decodes
// an NVFP4 block to the same exact f16 values; every product is then exact in F32 and only the F32 additions round.
// The reference's own bound for this entry is a relative error of 1e-5 against float64 sums over the quantized
// operands (tests/gpu/test_mm_fp4_gpu.hip:129-153).
#include "common.cuh"
#include "decode.cuh"
#include "fp4_tc_api.h"
#include "mm_tc_api.h"
#include "osmos_b200/mm.h"

namespace osmos {
namespace {

constexpr int kThreads = 256;
constexpr uint32_t kGroup = 16;  // values a scale

// an F32 value >= 0 (at most 448 matters) to E4M3's code, nearest even, saturating at 448 (0x7E); below 2^-6 the
// subnormal codes m 2^-9 (kernels/mm_fp4.hip:26-43: the same function of v, written on the bits instead of frexpf)
__device__ __forceinline__ uint32_t e4m3_code_of(float v) {
  const float a = fminf(v, 448.0f);
  if (!(a > 0.0f)) return 0;
  if (a < 0.015625f) {  // subnormal: a whole number of 2^-9; 8 of them are the first normal code
    const float q = rintf(a * 512.0f);
    return q >= 8.0f ? 0x08u : (uint32_t) q;
  }
  const uint32_t u = __float_as_uint(a);
  const uint32_t r = u + 0x7FFFFu + ((u >> 20) & 1u);  // 3 mantissa bits kept, ties to even; a carry raises the exponent
  const uint32_t code = (r >> 20) - (120u << 3);       // exponent bias 127 -> 7
  return code > 0x7Eu ? 0x7Eu : code;
}
// an E4M3 code's value, codes up to 0x7E (kernels/round.h:87-93)
__device__ __forceinline__ float e4m3_value_of(uint32_t c) {
  return c >> 3 ? __uint_as_float((c << 20) + (120u << 23)) : (float) c * 0.001953125f;
}
// E2M1's code of x, |x| <= 6: the nearest of 0, .5, 1, 1.5, 2, 3, 4, 6, a tie to the even index; -0 and what rounds
// to 0 have code 0 (kernels/mm_fp4.hip:46-59)
__device__ __forceinline__ uint32_t e2m1_nearest(float x) {
  const float a = fabsf(x);
  // index i's upper boundary, and whether the boundary itself still belongs to i (i even)
  const uint32_t i = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
  return i ? (x < 0.0f ? 8u : 0u) | i : 0u;
}
__device__ __forceinline__ float e2m1_magnitude(uint32_t i) {  // 0, .5, 1, 1.5, 2, 3, 4, 6
  return (float) osmos_e2m1_doubled[i & 7u] * 0.5f;
}
// a uniform in [0, 1) of (seed, element index) and the stochastic rounding up with probability (distance from the
// grid point below) / step (kernels/mm_fp4.hip:64-81)
__device__ __forceinline__ float uniform_of(uint32_t seed, uint64_t i) {
  uint32_t h = (uint32_t) i * 0x9E3779B1u ^ (uint32_t) (i >> 32) * 0x85EBCA77u ^ seed;
  h ^= h >> 16, h *= 0x85EBCA6Bu, h ^= h >> 13, h *= 0xC2B2AE35u, h ^= h >> 16;
  return (float) (h >> 8) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ uint32_t e2m1_stochastic(float x, float u) {
  const float a = fabsf(x);
  uint32_t i = 0;
  while (i < 7 && a >= e2m1_magnitude(i + 1)) i++;
  if (i < 7 && u < (a - e2m1_magnitude(i)) / (e2m1_magnitude(i + 1) - e2m1_magnitude(i))) i++;
  return i ? (x < 0.0f ? 8u : 0u) | i : 0u;
}

struct ActArgs {
  const void* x;
  const float* gs_dev;
  uint8_t *q, *sc;
  uint32_t xs, n, cols, seed;
  float gs;
};

// a thread a group of 16 values: its scale byte and its 8 bytes of codes
template <bool BF16, bool VEC>
__global__ void __launch_bounds__(kThreads) fp4_act_kernel(const ActArgs a) {
  const uint32_t groups = a.cols / kGroup;
  const uint64_t at = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (at >= (uint64_t) a.n * groups) return;
  const uint32_t t = (uint32_t) (at / groups), b = (uint32_t) (at % groups);
  const float gs = a.gs_dev ? *a.gs_dev : a.gs;
  // the stream of random numbers salted with a scale made on the device, never 0 (0 means nearest)
  const uint32_t seed = a.seed && a.gs_dev ? (a.seed ^ __float_as_uint(gs) * 0x9E3779B1u) | 1u : a.seed;
  float v[kGroup];
  const uint64_t first = (uint64_t) t * a.xs + b * kGroup;
  if constexpr (BF16) {
    const uint16_t* p = (const uint16_t*) a.x + first;
    if constexpr (VEC) {
      const uint4 lo = __ldg((const uint4*) p), hi = __ldg((const uint4*) p + 1);
      const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int j = 0; j < 8; j++) v[2 * j] = __uint_as_float(w[j] << 16), v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    } else {
#pragma unroll
      for (int j = 0; j < (int) kGroup; j++) v[j] = __uint_as_float((uint32_t) __ldg(p + j) << 16);
    }
  } else {
    const float* p = (const float*) a.x + first;
    if constexpr (VEC) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float4 f = __ldg((const float4*) p + j);
        v[4 * j] = f.x, v[4 * j + 1] = f.y, v[4 * j + 2] = f.z, v[4 * j + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < (int) kGroup; j++) v[j] = __ldg(p + j);
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < (int) kGroup; j++) amax = fmaxf(amax, fabsf(v[j]));
  const uint32_t s = e4m3_code_of(amax / 6.0f / gs);
  const float sf = mul_rn(e4m3_value_of(s), gs);
  a.sc[(uint64_t) t * groups + b] = (uint8_t) s;
  uint32_t packed[2] = {0, 0};
#pragma unroll
  for (int j = 0; j < (int) kGroup; j++) {
    const float c = sf > 0.0f ? fminf(fmaxf(v[j] / sf, -6.0f), 6.0f) : 0.0f;
    const uint32_t code = seed ? e2m1_stochastic(c, uniform_of(seed, (uint64_t) t * a.cols + b * kGroup + j)) : e2m1_nearest(c);
    packed[j / 8] |= code << (4 * (j % 8));
  }
  *(uint2*) (a.q + (uint64_t) t * (a.cols / 2) + b * 8u) = make_uint2(packed[0], packed[1]);
}

// the codes of tokens t0 .. t0 + n (of q and sc) as exact f16 values in the tiled layout, rows of cols; a thread a
// group of 16 = one row of a 16 x 16 fragment, 32 contiguous bytes; the tile's rows past the last token zero
__global__ void __launch_bounds__(kThreads) fp4_expand_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sc,
                                                              uint32_t n, uint32_t n16, uint32_t cols, __half* __restrict__ x16) {
  const uint32_t groups = cols / kGroup;
  const uint64_t at = (uint64_t) blockIdx.x * kThreads + threadIdx.x;  // in output order: tile, fragment, token in tile
  if (at >= (uint64_t) n16 * groups) return;
  const uint32_t tile = (uint32_t) (at / ((uint64_t) MM_TILE * groups)), in = (uint32_t) (at % ((uint64_t) MM_TILE * groups));
  const uint32_t b = in / MM_TILE, t = tile * MM_TILE + in % MM_TILE;
  __align__(16) __half out[kGroup];
  if (t < n) {
    const uint2 codes = __ldg((const uint2*) (q + (uint64_t) t * (cols / 2) + b * 8u));
    const float s = mul_rn(e4m3_value_of(__ldg(sc + (uint64_t) t * groups + b) & 0x7Fu), 0.5f);
#pragma unroll
    for (int j = 0; j < (int) kGroup; j++) {
      const uint32_t c = ((j < 8 ? codes.x : codes.y) >> (4 * (j % 8))) & 15u;
      out[j] = __float2half_rn(mul_rn(s, (float) osmos_e2m1_doubled[c]));  // exact: 6 significant bits at most
    }
  } else {
#pragma unroll
    for (int j = 0; j < (int) kGroup; j++) out[j] = __ushort_as_half(0);
  }
  uint4* dst = (uint4*) (x16 + mm_x16_at(t, b * kGroup, cols));
  dst[0] = ((const uint4*) out)[0], dst[1] = ((const uint4*) out)[1];
}

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" bool mm_fp4_ok(void) {
  int dev = 0, major = 0;
  return cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess &&
         major == 10;
}

extern "C" bool mm_fp4_quant(const void* x, uint32_t bf16, uint32_t xs, uint32_t n, uint32_t cols, float gs, const float* gs_dev,
                             uint32_t sr_seed, void* q, void* sc, void* stream) {
  if (!mm_fp4_ok() || !x || !q || !sc || !n || !cols || cols % 64 || (!gs_dev && !(gs > 0.0f)) || (n > 1 && xs < cols) || ((uintptr_t) q & 7u))
    return false;
  ActArgs a{x, gs_dev, (uint8_t*) q, (uint8_t*) sc, xs, n, cols, sr_seed, gs};
  const unsigned blocks = blocks_for((uint64_t) n * (cols / kGroup), kThreads);
  const cudaStream_t s = stream_of(stream);
  const uint32_t elem = bf16 ? 2u : 4u;
  const bool vec = ((uintptr_t) x & 15u) == 0 && ((uint64_t) xs * elem) % 16 == 0;
  if (bf16) {
    if (vec) fp4_act_kernel<true, true><<<blocks, kThreads, 0, s>>>(a);
    else fp4_act_kernel<true, false><<<blocks, kThreads, 0, s>>>(a);
  } else {
    if (vec) fp4_act_kernel<false, true><<<blocks, kThreads, 0, s>>>(a);
    else fp4_act_kernel<false, false><<<blocks, kThreads, 0, s>>>(a);
  }
  return launched();
}

extern "C" bool mm_fp4_act(const float* x, uint32_t xs, uint32_t n, uint32_t cols, float gs, void* q, void* sc, void* stream) {
  return mm_fp4_quant(x, 0, xs, n, cols, gs, nullptr, 0, q, sc, stream);
}

static int g_fp4_tensor = 1;  // mm_fp4_set_tensor: 0 keeps the product on the f16 tensor-core route (the tests compare the two)
static int g_fp4_route = -1;  // the route mm_fp4's last call took: 1 the block-scaled FP4 MMA, 0 the f16 product

extern "C" int mm_fp4_last_route(void) { return g_fp4_route; }

extern "C" void mm_fp4_set_tensor(int on) { g_fp4_tensor = on; }
extern "C" uint32_t mm_fp4_desc(uint32_t mx, uint32_t n, uint32_t sf_id) { return fp4_tc::instr_desc(mx != 0, n, sf_id); }

extern "C" bool mm_mxfp4(const void* w, uint32_t rows, uint32_t cols, const void* packed, uint32_t n, float scale, float* y,
                         uint32_t ys, void* stream) {
  if (!mm_fp4_ok() || !w || !packed || !y || !n || !rows || !cols || cols % 512 || rows % 128 || (n > 1 && ys < rows)) return false;
  const uint32_t stride = cols / 2 + cols / 32;  // a token's codes, then its scale bytes
  return fp4_tc::try_launch(true, w, rows, cols, packed, stride, (const uint8_t*) packed + cols / 2, stride, n, scale, y, ys, stream) > 0;
}

extern "C" bool mm_fp4(const void* w, uint32_t rows, uint32_t cols, const void* q, const void* sc, uint32_t n, float scale,
                       float* y, uint32_t ys, void* stream) {
  if (!mm_fp4_ok() || !w || !q || !sc || !y || !n || !mm_tc::shape_ok(QTYPE_NVFP4, rows, cols) || (n > 1 && ys < rows) || ((uintptr_t) q & 7u))
    return false;
  if (g_fp4_tensor)  // the block-scaled FP4 MMA when it takes the shape (whole 128-row tiles, 256-value steps)
    if (const int st = fp4_tc::try_launch(false, w, rows, cols, q, cols / 2, sc, cols / 16, n, scale, y, ys, stream)) {
      g_fp4_route = 1;
      return st > 0;
    }
  g_fp4_route = 0;
  const cudaStream_t s = stream_of(stream);
  const uint32_t most = n < MM_MAX_TOKENS ? n : MM_MAX_TOKENS, most16 = (most + MM_TILE - 1) / MM_TILE * MM_TILE;
  void* x16 = nullptr;  // the step's f16 activations: allocated and freed in stream order
  if (cudaMallocAsync(&x16, (size_t) most16 * cols * sizeof(__half), s) != cudaSuccess) return false;
  bool ok = true;
  for (uint32_t t0 = 0; ok && t0 < n; t0 += MM_MAX_TOKENS) {  // MM_MAX_TOKENS a time through the one x16
    const uint32_t c = n - t0 < MM_MAX_TOKENS ? n - t0 : MM_MAX_TOKENS, c16 = (c + MM_TILE - 1) / MM_TILE * MM_TILE;
    fp4_expand_kernel<<<blocks_for((uint64_t) c16 * (cols / kGroup), kThreads), kThreads, 0, s>>>(
        (const uint8_t*) q + (uint64_t) t0 * (cols / 2), (const uint8_t*) sc + (uint64_t) t0 * (cols / kGroup), c, c16, cols, (__half*) x16);
    ok = launched() && mm_tc::run(QTYPE_NVFP4, w, rows, cols, x16, c, y + (uint64_t) t0 * ys, ys, scale, stream);
  }
  return (cudaFreeAsync(x16, s) == cudaSuccess) && ok;
}
