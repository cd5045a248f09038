// Q4_K x int8 (include/osmos_b200/mmq.h): the activation quantizer and the generic grouped matmul kernel.
//
// This file's matmul kernel is the shape-agnostic one: a block computes 16 rows x 16 tokens, stages each 256-value
// weight block and the matching activation tile in shared memory and takes the group dots with dp4a. The order of
// the F32 operations is the contract's, so it and any tensor-core kernel for the same entry point give the same bits.
#include "common.cuh"
#include "mmq_tc_api.h"
#include "osmos_b200/mmq.h"

namespace osmos {
namespace {

constexpr int kThreads = 256, kTile = 16, kParts = 4;
constexpr int kBlockValues = 256, kBlockBytes = 144, kGroups = kBlockValues / MMQ_GROUP;

// a thread a value, a group a warp's 32 lanes
__global__ void __launch_bounds__(kThreads) x8_rows_kernel(const float* __restrict__ x, uint32_t xs,
                                                           const int32_t* __restrict__ idx, uint32_t slots, uint32_t cols,
                                                           int8_t* __restrict__ x8, float* __restrict__ dx,
                                                           float* __restrict__ sx) {
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i >= (uint64_t) slots * cols) return;  // whole warps: slots * cols is a multiple of 32
  const uint32_t s = (uint32_t) (i / cols), c = (uint32_t) (i % cols);
  const int32_t r = idx[s];
  const float v = r >= 0 ? x[(uint64_t) r * xs + c] : 0.0f;
  float a = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o, kWarp));
  const float d = __fdiv_rn(a, 127.0f);
  const int q = a == 0.0f ? 0 : (int) fminf(fmaxf(rintf(__fdiv_rn(v, d)), -127.0f), 127.0f);
  int sum = q;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o, kWarp);
  x8[mmq_x8_at(s, c, cols)] = (int8_t) q;
  if (c % MMQ_GROUP == 0) {
    const uint64_t g = mmq_dx_at(s, c / MMQ_GROUP, cols / MMQ_GROUP);
    const float dd = a == 0.0f ? 0.0f : d;
    dx[g] = dd;
    sx[g] = mul_rn(dd, (float) sum);
  }
}

constexpr int kRowPad = kBlockBytes + 4;  // a staged row's stride: 37 words, so 16 rows fall in 16 different banks

__global__ void __launch_bounds__(kThreads) q4k_kernel(const uint8_t* const* __restrict__ wt, const int32_t* __restrict__ cnt,
                                                       uint32_t cols, const int8_t* __restrict__ x8,
                                                       const float* __restrict__ dx, const float* __restrict__ sx,
                                                       const uint32_t* __restrict__ soff, float* __restrict__ ya,
                                                       const uint32_t* __restrict__ yoff, uint32_t ys) {
  __shared__ __align__(16) uint8_t wrow[kTile * kRowPad];
  __shared__ __align__(16) int xq[kGroups * kTile * MMQ_GROUP / 4];
  __shared__ float xd[kGroups * kTile], xsum[kGroups * kTile];
  const uint32_t m = blockIdx.y, n = (uint32_t) cnt[m], row0 = blockIdx.x * kTile, c0 = blockIdx.z * kTile;
  if (c0 >= n) return;
  const int r = threadIdx.x % kTile, c = threadIdx.x / kTile;
  const uint32_t nb = cols / kBlockValues, groups = cols / MMQ_GROUP;
  const uint64_t row_bytes = (uint64_t) nb * kBlockBytes;
  const uint8_t* w = wt[m] + (uint64_t) row0 * row_bytes;
  const uint32_t s0 = soff[m] + c0;  // this block's first slot: a multiple of 16, so one tile of the layouts
  float part[kParts] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (uint32_t b = 0; b < nb; b++) {
    __syncthreads();
    for (int i = threadIdx.x; i < kTile * (kBlockBytes / 4); i += kThreads) {
      const int rr = i / (kBlockBytes / 4), k = i % (kBlockBytes / 4);
      *(uint32_t*) (wrow + rr * kRowPad + 4 * k) = *(const uint32_t*) (w + rr * row_bytes + (uint64_t) b * kBlockBytes + 4 * k);
    }
    const int4* xsrc = (const int4*) (x8 + mmq_x8_at(s0, b * kBlockValues, cols));
    for (int i = threadIdx.x; i < kGroups * kTile * MMQ_GROUP / 16; i += kThreads) ((int4*) xq)[i] = xsrc[i];
    if (threadIdx.x < kGroups * kTile) {
      const uint64_t at = mmq_dx_at(s0, b * kGroups, groups) + threadIdx.x;
      xd[threadIdx.x] = dx[at], xsum[threadIdx.x] = sx[at];
    }
    __syncthreads();
    const uint8_t* blk = wrow + r * kRowPad;
    const float d = half_value(blk[0] | blk[1] << 8), dmin = half_value(blk[2] | blk[3] << 8);
    const uint8_t* sc8 = blk + 4;
    float acc = part[b % kParts];
#pragma unroll
    for (int g = 0; g < kGroups; g++) {
      const int sc = g < 4 ? sc8[g] & 0x3F : (sc8[g + 4] & 0x0F) | ((sc8[g - 4] >> 6) << 4);
      const int mn = g < 4 ? sc8[g + 4] & 0x3F : (sc8[g + 4] >> 4) | ((sc8[g] >> 6) << 4);
      const float dsc = mul_rn(d, (float) sc), dm = mul_rn(dmin, (float) mn);
      const uint32_t* qw = (const uint32_t*) (blk + 16 + (g / 2) * 32);
      const int* xw = xq + (g * kTile + c) * (MMQ_GROUP / 4);
      int isum = 0;
#pragma unroll
      for (int k = 0; k < 8; k++) isum = __dp4a((int) ((qw[k] >> (4 * (g % 2))) & 0x0F0F0F0Fu), xw[k], isum);
      const float v = mul_rn(dsc, xd[g * kTile + c]);
      acc = __fmaf_rn(v, (float) isum, acc);
      acc = __fmaf_rn(dm, -xsum[g * kTile + c], acc);
    }
    // (b % kParts is not a compile-time index: four selects keep the partials in registers)
    part[0] = b % kParts == 0 ? acc : part[0], part[1] = b % kParts == 1 ? acc : part[1];
    part[2] = b % kParts == 2 ? acc : part[2], part[3] = b % kParts == 3 ? acc : part[3];
  }
  const uint32_t t = c0 + c;
  if (t < n) {
    float s = part[0];
    s = __fadd_rn(s, part[1]), s = __fadd_rn(s, part[2]), s = __fadd_rn(s, part[3]);
    ya[yoff[m] + (uint64_t) t * ys + row0 + r] = s;
  }
}

bool g_use_tensor = true;

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" void mmq_set_tensor(int on) { g_use_tensor = on != 0; }
extern "C" uint32_t mmq_status(void) { return mmq_tc::read_status(); }

extern "C" bool mmq_known(uint32_t type) { return type == QTYPE_Q4_K; }

extern "C" bool mmq_x8_rows(const float* x, uint32_t xs, const int32_t* idx, uint32_t slots, uint32_t cols, int8_t* x8,
                            float* dx, float* sx, void* stream) {
  if (!x || !idx || !x8 || !dx || !sx || !slots || !cols || cols % MMQ_GROUP || xs < cols) return false;
  const uint64_t work = (uint64_t) slots * cols;
  x8_rows_kernel<<<blocks_for(work, kThreads), kThreads, 0, stream_of(stream)>>>(x, xs, idx, slots, cols, x8, dx, sx);
  return launched();
}

extern "C" bool mmq_group(uint32_t type, const void* const* w, const int32_t* cnt, uint32_t n_mat, uint32_t max_cnt,
                          uint32_t rows, uint32_t cols, const int8_t* x8, const float* dx, const float* sx,
                          const uint32_t* soff, float* y, const uint32_t* yoff, uint32_t ys, void* stream) {
  if (!mmq_known(type) || !w || !cnt || !x8 || !dx || !sx || !soff || !y || !yoff || !n_mat || !max_cnt || !rows ||
      rows % kTile || !cols || cols % kBlockValues || ys < rows)
    return false;
  if (g_use_tensor)
    if (const int st = mmq_tc::try_launch(w, cnt, n_mat, max_cnt, rows, cols, x8, dx, sx, soff, y, yoff, ys, stream)) return st > 0;
  const dim3 grid(rows / kTile, n_mat, (max_cnt + kTile - 1) / kTile);
  q4k_kernel<<<grid, kThreads, 0, stream_of(stream)>>>((const uint8_t* const*) w, cnt, cols, x8, dx, sx, soff, y, yoff, ys);
  return launched();
}
