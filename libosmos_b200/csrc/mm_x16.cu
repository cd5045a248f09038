// F32 activations to the tiled f16 layout the prefill matrix products read (include/osmos_b200/mm.h).
//
// One kernel serves mm_x16, mm_x16_rows and mm_x16_heads: a thread writes a run of 8 halves that is contiguous in the
// tiled layout (half a fragment's row, 16 bytes), threads in output order so that a warp's stores fill whole lines;
// its 8 values are two 16-byte loads when x allows it, single loads otherwise. The rounding is cvt.rn.f16.f32's -
// nearest even - and the overflow test is the reference's !(|v| <= 65504), which also catches NaN
// (kernels/mm.h:53-58, kernels/mm.hip:77-159).
#include "common.cuh"
#include "osmos_b200/mm.h"

namespace osmos {
namespace {

constexpr int kThreads = 256;
constexpr uint32_t kRun = 8;
constexpr float kF16Max = 65504.0f;

struct X16Args {
  const float* x;
  const int32_t* idx;  // NULL: slot s is row s
  __half* x16;
  int32_t* overflow;
  uint32_t xs, n, slots16, cols, heads, hs;  // n: live slots; slots16: slots in whole tiles
};

template <bool VEC>
__global__ void __launch_bounds__(kThreads) x16_kernel(const X16Args a) {
  const uint64_t run = (uint64_t) blockIdx.x * kThreads + threadIdx.x;  // over heads x tiled runs
  const uint64_t per_head = (uint64_t) a.slots16 * a.cols / kRun;
  if (run >= per_head * a.heads) return;
  const uint32_t h = (uint32_t) (run / per_head);
  const uint64_t o = (run - h * per_head) * kRun;  // the run's first half in the head's x16
  const uint64_t tile = (uint64_t) MM_TILE * a.cols;
  const uint32_t in = (uint32_t) (o % tile), frag = in % (MM_TILE * MM_TILE);
  const uint32_t t = (uint32_t) (o / tile) * MM_TILE + frag / MM_TILE;
  const uint32_t c = in / (MM_TILE * MM_TILE) * MM_TILE + frag % MM_TILE;
  int64_t r = -1;
  if (t < a.n) r = a.idx ? a.idx[t] : (int64_t) t;
  float v[kRun] = {};
  if (r >= 0) {
    const float* p = a.x + (uint64_t) r * a.xs + (uint64_t) h * a.hs + c;
    if constexpr (VEC) {
      const float4 lo = __ldg((const float4*) p), hi = __ldg((const float4*) p + 1);
      v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
    } else {
#pragma unroll
      for (uint32_t j = 0; j < kRun; j++) v[j] = __ldg(p + j);
    }
  }
  bool over = false;
  __align__(16) __half out[kRun];
#pragma unroll
  for (uint32_t j = 0; j < kRun; j++) over |= !(fabsf(v[j]) <= kF16Max), out[j] = __float2half_rn(v[j]);
  if (over) atomicOr(a.overflow, 1);
  __half* dst = a.x16 + (uint64_t) h * a.slots16 * a.cols + o;
  if (((uintptr_t) dst & 15u) == 0) {
    *(uint4*) dst = *(const uint4*) out;
  } else {
#pragma unroll
    for (uint32_t j = 0; j < kRun; j++) dst[j] = out[j];
  }
}

bool launch(const X16Args& a, cudaStream_t s) {
  const uint64_t runs = (uint64_t) a.slots16 * a.cols / kRun * a.heads;
  const uint64_t blocks = (runs + kThreads - 1) / kThreads;
  if (!blocks || blocks >= (1ull << 31)) return false;
  const bool vec = (uintptr_t) a.x % 16 == 0 && a.xs % 4 == 0 && a.hs % 4 == 0;
  if (vec) x16_kernel<true><<<(unsigned) blocks, kThreads, 0, s>>>(a);
  else x16_kernel<false><<<(unsigned) blocks, kThreads, 0, s>>>(a);
  return launched();
}

uint32_t whole_tiles(uint32_t n) { return (n + MM_TILE - 1) / MM_TILE * MM_TILE; }

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" bool mm_x16(const float* x, uint32_t xs, uint32_t n, uint32_t cols, void* x16, int32_t* overflow,
                       void* stream) {
  if (!x || !x16 || !overflow || !n || n > MM_MAX_TOKENS || !cols || cols % MM_TILE || (n > 1 && xs < cols)) return false;
  const X16Args a{x, nullptr, (__half*) x16, overflow, xs, n, whole_tiles(n), cols, 1, 0};
  return launch(a, stream_of(stream));
}

extern "C" bool mm_x16_rows(const float* x, uint32_t xs, const int32_t* idx, uint32_t slots, uint32_t cols, void* x16,
                            int32_t* overflow, void* stream) {
  if (!x || !idx || !x16 || !overflow || !slots || !cols || cols % MM_TILE || xs < cols || xs % 4 || (uintptr_t) x % 16)
    return false;
  const X16Args a{x, idx, (__half*) x16, overflow, xs, slots, whole_tiles(slots), cols, 1, 0};
  return launch(a, stream_of(stream));
}

extern "C" bool mm_x16_heads(const float* x, uint32_t xs, uint32_t n, uint32_t heads, uint32_t hs, uint32_t cols,
                             void* x16, int32_t* overflow, void* stream) {
  if (!x || !x16 || !overflow || !n || n > MM_MAX_TOKENS || !heads || !cols || cols % MM_TILE || hs % 4 || xs % 4 ||
      (uintptr_t) x % 16 || (uintptr_t) x16 % 16 || (heads - 1) * (uint64_t) hs + cols > xs)
    return false;
  const X16Args a{x, nullptr, (__half*) x16, overflow, xs, n, whole_tiles(n), cols, heads, hs};
  return launch(a, stream_of(stream));
}
