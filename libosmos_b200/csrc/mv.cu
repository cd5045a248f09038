// The F32-activation matvec family (include/osmos_b200/mv.h): one kernel serves the dense, grouped and
// grouped-by-token entry points. A warp owns kRows rows of one matrix; lane l decodes chunks l, l + 32, ... of each
// row and runs one fmaf chain per (row, token); the xor tree finishes the row. kRows rows share every x chunk a lane
// loads, so x traffic from L1 is 1 / kRows of the naive count.
#include "decode.cuh"
#include "dispatch.cuh"
#include "mv_staged_api.h"
#include "osmos_b200/mv.h"

namespace osmos {
namespace {

constexpr int kWarps = 8, kThreads = kWarps * kWarp;
constexpr int kRows = 2;  // rows a warp sums at once

enum Mode : int { kDense = 0, kGroup = 1, kGroupTok = 2 };

struct MvArgs {
  const uint8_t* w;          // kDense: the matrix
  const uint8_t* const* wt;  // grouped: the matrices' table
  const int32_t* cnt;        // kGroupTok
  const int32_t* xrow;       // kGroupTok
  const float* x;
  float* y;
  uint32_t rows, cols, xs, ys, n_tok, x_mat, x_div;
};

template <uint32_t T, int NT, int MODE>
__global__ void __launch_bounds__(kThreads) mv_kernel(const MvArgs a) {
  __shared__ __align__(16) uint8_t tables[grid_smem_bytes<T>() > 0 ? grid_smem_bytes<T>() : 16];
  const Grids g = stage_grids<T>(tables);
  const int lane = threadIdx.x % kWarp;
  const uint32_t row0 = (blockIdx.x * kWarps + threadIdx.x / kWarp) * kRows;
  if (row0 >= a.rows) return;  // the whole warp

  // this block's matrix, its first token's x and y, and how many of the NT token slots are live
  const uint8_t* w;
  const float* x;
  float* y;
  uint32_t live;
  if constexpr (MODE == kDense) {
    const uint32_t t0 = blockIdx.y * NT;
    w = a.w, x = a.x + (uint64_t) t0 * a.xs, y = a.y + (uint64_t) t0 * a.ys;
    live = a.n_tok - t0 < (uint32_t) NT ? a.n_tok - t0 : (uint32_t) NT;
  } else if constexpr (MODE == kGroup) {
    const uint32_t m = blockIdx.y;
    w = a.wt[m], x = a.x + (uint64_t) (m / a.x_div) * a.x_mat, y = a.y + (uint64_t) m * a.rows, live = 1;
  } else {
    const uint32_t m = blockIdx.y;
    const int32_t c = a.cnt[m];
    if (c <= 0) return;  // an entry past a table's live ones: nothing read, nothing written
    const uint64_t r0 = (uint64_t) a.xrow[m];
    w = a.wt[m], x = a.x + r0 * a.xs, y = a.y + r0 * a.ys, live = (uint32_t) c < (uint32_t) NT ? (uint32_t) c : (uint32_t) NT;
  }

  constexpr int kPer = Fmt<T>::chunks;  // chunks a block
  const uint64_t row_bytes = (uint64_t) (a.cols / Fmt<T>::values) * Fmt<T>::bytes;
  const uint8_t* base[kRows];
#pragma unroll
  for (int q = 0; q < kRows; q++) base[q] = w + (uint64_t) (row0 + q < a.rows ? row0 + q : row0) * row_bytes;
  // a token slot past the live ones repeats the last live token: summed, never stored, nothing past it read
  const float* xt[NT];
#pragma unroll
  for (int t = 0; t < NT; t++) xt[t] = x + (uint64_t) ((uint32_t) t < live ? t : live - 1) * a.xs;

  float acc[kRows][NT];
#pragma unroll
  for (int q = 0; q < kRows; q++)
#pragma unroll
    for (int t = 0; t < NT; t++) acc[q][t] = 0.0f;

  const uint32_t chunks = a.cols / kChunk;
  for (uint32_t c = lane; c < chunks; c += kWarp) {
    float v[kRows][kChunk];
#pragma unroll
    for (int q = 0; q < kRows; q++) decode8<T>(base[q] + (uint64_t) (c / kPer) * Fmt<T>::bytes, (int) (c % kPer), v[q], g);
#pragma unroll
    for (int t = 0; t < NT; t++) {
      const float4* xp = (const float4*) (xt[t] + (uint64_t) c * kChunk);
      const float4 lo = __ldg(xp), hi = __ldg(xp + 1);
#pragma unroll
      for (int q = 0; q < kRows; q++) {
        float s = acc[q][t];
        s = __fmaf_rn(v[q][0], lo.x, s), s = __fmaf_rn(v[q][1], lo.y, s);
        s = __fmaf_rn(v[q][2], lo.z, s), s = __fmaf_rn(v[q][3], lo.w, s);
        s = __fmaf_rn(v[q][4], hi.x, s), s = __fmaf_rn(v[q][5], hi.y, s);
        s = __fmaf_rn(v[q][6], hi.z, s), s = __fmaf_rn(v[q][7], hi.w, s);
        acc[q][t] = s;
      }
    }
  }
#pragma unroll
  for (int q = 0; q < kRows; q++)
#pragma unroll
    for (int t = 0; t < NT; t++) {
      const float s = xor_tree<kWarp>(acc[q][t]);
      if (lane == 0 && row0 + q < a.rows && (uint32_t) t < live) y[(uint64_t) t * a.ys + row0 + q] = s;
    }
}

template <uint32_t T, int NT, int MODE>
bool launch(const MvArgs& a, uint32_t grid_y, cudaStream_t s) {
  const dim3 grid(blocks_for(a.rows, kWarps * kRows), grid_y);
  mv_kernel<T, NT, MODE><<<grid, kThreads, 0, s>>>(a);
  return launched();
}

// token slots a launch carries: the smallest of 1, 2, 4, 8 that holds `n` (a slot past the live ones costs work,
// never a bit)
template <uint32_t T, int MODE>
bool by_tokens(const MvArgs& a, uint32_t n, uint32_t grid_y, cudaStream_t s) {
  if (n <= 1) return launch<T, 1, MODE>(a, grid_y, s);
  if (n <= 2) return launch<T, 2, MODE>(a, grid_y, s);
  if (n <= 4) return launch<T, 4, MODE>(a, grid_y, s);
  return launch<T, 8, MODE>(a, grid_y, s);
}

template <uint32_t T> bool shape_ok(uint32_t cols) { return cols && cols % Fmt<T>::values == 0 && cols % kChunk == 0; }

bool g_use_staged = true;  // mv_set_staged: the tests run both kernels and compare their bits

template <uint32_t T>
bool strided(const void* w, uint32_t rows, uint32_t cols, const float* x, uint32_t xs, uint32_t n_tok, float* y,
             uint32_t ys, cudaStream_t s) {
  if (!shape_ok<T>(cols) || !rows || !n_tok) return false;
  if ((n_tok > 1 && (xs < cols || ys < rows)) || xs % kChunk) return false;
  if (g_use_staged && n_tok <= MV_MAX_TOKENS) {  // the staged kernel when it takes the shape: the same bits
    const mvs::Request r{w, x, y, rows, cols, xs, ys, n_tok};
    if (const int st = mvs::try_launch(T, r, s)) return st > 0;
    // long rows: as many tokens a pass as the staged kernel holds x for (a token's sums do not depend on its batch),
    // a pass it still does not take on the generic kernel
    const uint32_t fit = mvs::max_tokens(T, cols);
    if (fit && fit < n_tok) {
      for (uint32_t t = 0; t < n_tok; t += fit) {
        const uint32_t c = n_tok - t < fit ? n_tok - t : fit;
        const mvs::Request part{w, x + (uint64_t) t * xs, y + (uint64_t) t * ys, rows, cols, xs, ys, c};
        const int st = mvs::try_launch(T, part, s);
        if (st < 0) return false;
        if (st == 0) {
          MvArgs a{};
          a.w = (const uint8_t*) w, a.x = part.x, a.y = part.y, a.rows = rows, a.cols = cols, a.xs = xs, a.ys = ys, a.n_tok = c;
          if (!by_tokens<T, kDense>(a, c, 1, s)) return false;
        }
      }
      return true;
    }
  }
  MvArgs a{};
  a.w = (const uint8_t*) w, a.x = x, a.y = y, a.rows = rows, a.cols = cols, a.xs = xs, a.ys = ys, a.n_tok = n_tok;
  if (n_tok > MV_MAX_TOKENS) return launch<T, 8, kDense>(a, (n_tok + 7) / 8, s);  // a prompt's: tiles of 8 tokens
  return by_tokens<T, kDense>(a, n_tok, 1, s);
}

template <uint32_t T>
bool group(const void* const* w, uint32_t n, uint32_t rows, uint32_t cols, const float* x, uint32_t x_mat,
           uint32_t x_div, float* y, cudaStream_t s) {
  if (!shape_ok<T>(cols) || x_mat % kChunk || !x_div) return false;
  if (g_use_staged) {  // the staged kernel when it takes the shape: the same bits
    mvs::Request r{nullptr, x, y, rows, cols, cols, rows, 1};
    r.wt = w, r.n_entries = n, r.x_mat = x_mat, r.x_div = x_div;
    if (const int st = mvs::try_launch(T, r, s)) return st > 0;
  }
  MvArgs a{};
  a.wt = (const uint8_t* const*) w, a.x = x, a.y = y, a.rows = rows, a.cols = cols, a.xs = cols, a.ys = rows;
  a.n_tok = 1, a.x_mat = x_mat, a.x_div = x_div;
  return launch<T, 1, kGroup>(a, n, s);
}

template <uint32_t T>
bool group_tok(const void* const* w, const int32_t* cnt, const int32_t* xrow, uint32_t n, uint32_t max_cnt,
               uint32_t rows, uint32_t cols, const float* x, uint32_t xs, float* y, uint32_t ys, cudaStream_t s) {
  if (!shape_ok<T>(cols) || xs < cols || xs % kChunk) return false;
  if (g_use_staged) {  // the staged kernel when it takes the shape: the same bits
    mvs::Request r{nullptr, x, y, rows, cols, xs, ys, max_cnt};
    r.wt = w, r.n_entries = n, r.cnt = cnt, r.xrow = xrow;
    if (const int st = mvs::try_launch(T, r, s)) return st > 0;
  }
  MvArgs a{};
  a.wt = (const uint8_t* const*) w, a.cnt = cnt, a.xrow = xrow, a.x = x, a.y = y;
  a.rows = rows, a.cols = cols, a.xs = xs, a.ys = ys, a.n_tok = max_cnt;
  return by_tokens<T, kGroupTok>(a, max_cnt, n, s);
}

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" bool mv_strided(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const float* x, uint32_t xs,
                           uint32_t n_tok, float* y, uint32_t ys, void* stream) {
  if (!w || !x || !y) return false;
#define CASE(T) return strided<T>(w, rows, cols, x, xs, n_tok, y, ys, stream_of(stream));
  OSMOS_SWITCH_WEIGHTS(type, CASE, return false)
#undef CASE
}

extern "C" void mv_set_staged(int on) { g_use_staged = on != 0; }
extern "C" uint32_t mv_status(void) { return mvs::read_status(); }

extern "C" bool mv_run(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const float* x, uint32_t n_tok,
                       float* y, void* stream) {
  if (n_tok > MV_MAX_TOKENS) return false;  // the decode's: a step and its drafts
  return mv_strided(type, w, rows, cols, x, cols, n_tok, y, rows, stream);
}

extern "C" bool mv_group(uint32_t type, const void* const* w, uint32_t n, uint32_t rows, uint32_t cols, const float* x,
                         uint32_t x_mat, uint32_t x_div, float* y, void* stream) {
  if (!w || !x || !y || !n || n > MV_MAX_GROUP || !rows) return false;
#define CASE(T) return group<T>(w, n, rows, cols, x, x_mat, x_div, y, stream_of(stream));
  OSMOS_SWITCH_WEIGHTS(type, CASE, return false)
#undef CASE
}

extern "C" bool mv_group_tok(uint32_t type, const void* const* w, const int32_t* cnt, const int32_t* xrow, uint32_t n,
                             uint32_t max_cnt, uint32_t rows, uint32_t cols, const float* x, uint32_t xs, float* y,
                             uint32_t ys, void* stream) {
  if (!w || !cnt || !xrow || !x || !y || !n || n > MV_MAX_GROUP || !rows || !max_cnt || max_cnt > MV_MAX_TOKENS)
    return false;
#define CASE(T) return group_tok<T>(w, cnt, xrow, n, max_cnt, rows, cols, x, xs, y, ys, stream_of(stream));
  OSMOS_SWITCH_QUANT(type, CASE, return false)
#undef CASE
}
