// The int8 lane (include/osmos_b200/q8.h): activation rounding and the grouped expert matvecs over int8 inputs,
// with the gate + up + activation fusion. One kernel template serves q8_group_tok, q8_gate_up and q8_run.
//
// Thread mapping of this generic kernel: a lane of the contract is a thread; a warp holds 32 / L rows. It takes any
// shape the entry points accept. The order of every floating-point operation is fixed by the contract, so any other
// kernel for the same entry points must (and is tested to) give the same bits.
#include "decode.cuh"
#include "dispatch.cuh"
#include "lane_plain_api.h"
#include "lane_ring_api.h"
#include "lane_rows_api.h"
#include "lane_staged_api.h"
#include "osmos_b200/mv.h"
#include "osmos_b200/q8.h"
#include "q8_api.h"
#include "q8_round.cuh"

namespace osmos {
namespace {

constexpr int kWarps = 8, kThreads = kWarps * kWarp;
constexpr uint32_t kLongCols = 4096;  // rows this long or longer split over 32 lanes, shorter over 16

struct LaneArgs {
  const uint8_t* w_dense;       // q8_run: the matrix (tables NULL)
  const uint8_t* const* wg;     // the entries' matrices (gate, or the only one)
  const uint8_t* const* wu;     // FUSED: the entries' up matrices
  const int32_t *cnt, *xrow, *xin, *win;
  const int8_t* q;
  const float* d;
  const float* scale;
  float lim;
  float* out;
  uint32_t rows, cols, out_stride, n_tok;
};

template <uint32_t T, int NT, bool FUSED, bool DENSE>
__global__ void __launch_bounds__(kThreads) lane_kernel(const LaneArgs a) {
  __shared__ __align__(16) uint8_t tables[grid_smem_bytes<T>() > 0 ? grid_smem_bytes<T>() : 16];
  const Grids g = stage_grids<T>(tables);
  const int lane = threadIdx.x % kWarp;
  const int L = a.cols >= kLongCols ? 32 : 16, ll = lane % L;
  const uint32_t row = (blockIdx.x * kWarps + threadIdx.x / kWarp) * (uint32_t) (kWarp / L) + (uint32_t) (lane / L);
  const uint32_t nblk = a.cols / 32;

  const uint8_t *wg, *wu = nullptr;
  uint32_t r0, live;
  if constexpr (DENSE) {
    r0 = blockIdx.y * NT;
    live = a.n_tok - r0 < (uint32_t) NT ? a.n_tok - r0 : (uint32_t) NT;
    wg = a.w_dense;
  } else {
    const uint32_t m = blockIdx.y;
    const int32_t c = a.cnt[m];
    if (c <= 0) return;
    r0 = (uint32_t) a.xrow[m], live = (uint32_t) c < (uint32_t) NT ? (uint32_t) c : (uint32_t) NT;
    wg = a.wg[m];
    if constexpr (FUSED) wu = a.wu[m];
  }
  const uint64_t off = (uint64_t) (row < a.rows ? row : 0) * (uint64_t) (a.cols / Fmt<T>::values) * Fmt<T>::bytes;
  wg += off;
  if constexpr (FUSED) wu += off;

  // the input row of each token slot (a slot past the live ones is skipped: nothing of it is read)
  uint64_t xr[NT];
#pragma unroll
  for (int t = 0; t < NT; t++) {
    const uint32_t r = r0 + ((uint32_t) t < live ? (uint32_t) t : live - 1);
    xr[t] = a.xin ? (uint64_t) (uint32_t) a.xin[r] : r;
  }
  float ag[NT], au[NT];
#pragma unroll
  for (int t = 0; t < NT; t++) ag[t] = au[t] = 0.0f;

  constexpr int kSubs = Fmt<T>::subs;
  for (uint32_t s = ll; s < nblk; s += L) {
    LaneCodes cg, cu;
    const uint64_t at = (uint64_t) (s / kSubs) * Fmt<T>::bytes;
    lane_codes<T>(wg + at, (int) (s % kSubs), cg, g);
    if constexpr (FUSED) lane_codes<T>(wu + at, (int) (s % kSubs), cu, g);
#pragma unroll
    for (int t = 0; t < NT; t++) {
      if ((uint32_t) t < live) {
        const int4* xp = (const int4*) (a.q + xr[t] * a.cols + (uint64_t) s * 32);
        const int4 lo = __ldg(xp), hi = __ldg(xp + 1);
        const int x[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const float dx = __ldg(a.d + xr[t] * nblk + s);
        ag[t] = __fmaf_rn(dx, lane_block_sum<T>(cg, x), ag[t]);
        if constexpr (FUSED) au[t] = __fmaf_rn(dx, lane_block_sum<T>(cu, x), au[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < NT; t++) {
    float vg = ag[t], vu = au[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      if (o < L) {
        vg = __fadd_rn(vg, __shfl_xor_sync(0xFFFFFFFFu, vg, o, kWarp));
        if constexpr (FUSED) vu = __fadd_rn(vu, __shfl_xor_sync(0xFFFFFFFFu, vu, o, kWarp));
      }
    if (ll == 0 && row < a.rows && (uint32_t) t < live) {
      const uint64_t r = r0 + (uint32_t) t;
      if constexpr (FUSED)
        a.out[r * a.out_stride + row] = lane_swiglu(vg, vu, a.lim, a.scale[a.win ? a.win[r] : r]);
      else
        a.out[r * a.out_stride + row] = vg;
    }
  }
}

template <uint32_t T, int NT, bool FUSED, bool DENSE>
bool launch(const LaneArgs& a, uint32_t grid_y, cudaStream_t s) {
  const uint32_t per_block = kWarps * (kWarp / (a.cols >= kLongCols ? 32 : 16));
  lane_kernel<T, NT, FUSED, DENSE><<<dim3(blocks_for(a.rows, per_block), grid_y), kThreads, 0, s>>>(a);
  return launched();
}

template <uint32_t T, bool FUSED, bool DENSE>
bool by_tokens(const LaneArgs& a, uint32_t n, uint32_t grid_y, cudaStream_t s) {
  if (n <= 1) return launch<T, 1, FUSED, DENSE>(a, grid_y, s);
  if (n <= 2) return launch<T, 2, FUSED, DENSE>(a, grid_y, s);
  if (n <= 4) return launch<T, 4, FUSED, DENSE>(a, grid_y, s);
  return launch<T, 8, FUSED, DENSE>(a, grid_y, s);
}

// four lanes a block of 32 values, eight values a lane (q8_round.cuh)
template <bool GGML>
__global__ void __launch_bounds__(kThreads) round_kernel(const float* __restrict__ x, uint32_t rows, uint32_t cols,
                                                         uint32_t xs, int8_t* __restrict__ q, float* __restrict__ d) {
  pdl_wait();  // (a dependent launch: x is usually the output of the kernel ahead)
  pdl_launch_next();
  const uint32_t per = cols / 8;  // lanes a row
  const uint64_t total = (uint64_t) rows * per, i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  const bool live = i < total;  // (a block of four lanes is live or not as a whole; the warp's shuffles want every lane)
  const uint64_t at = live ? i : 0;
  const uint32_t r = (uint32_t) (at / per), c = (uint32_t) (at % per);
  float v[8], scale;
  load8(x + (uint64_t) r * xs + (uint64_t) c * 8, v);
  const uint2 codes = round_block8<GGML>(v, &scale);
  if (!live) return;
  int8_t* out = q + (uint64_t) r * cols + (uint64_t) c * 8;
  if (((uintptr_t) out & 7u) == 0) {
    *(uint2*) out = codes;
  } else {
#pragma unroll
    for (int j = 0; j < 8; j++) out[j] = (int8_t) ((j < 4 ? codes.x >> (8 * j) : codes.y >> (8 * (j - 4))) & 0xFF);
  }
  if (c % 4 == 0) d[(uint64_t) r * (cols / 32) + c / 4] = scale;
}

template <bool GGML>
bool round_rows(const float* x, uint32_t rows, uint32_t cols, uint32_t xs, int8_t* q, float* d, cudaStream_t s) {
  if (!x || !q || !d || !rows || !cols || cols % 32 || xs < cols) return false;
  const uint64_t lanes = (uint64_t) rows * (cols / 8);
  return launch_dependent(round_kernel<GGML>, dim3(blocks_for(lanes, kThreads)), dim3(kThreads), 0, s, x, rows, cols, xs, q, d) ==
         cudaSuccess;
}

int g_use_staged = 1;  // q8_set_staged: the tests run every kernel and compare their bits (0 generic only, 2 no ring)

// the grouped entry points' warp-ring kernel when it takes the type and shape: 1 queued, 0 not taken, -1 refused
int ring_first(uint32_t type, const LaneArgs& a, bool fused, uint32_t n_entries, uint32_t max_cnt, void* stream) {
  if (g_use_staged != 1) return 0;
  ring::Request r{};
  r.fused = fused, r.wg = (const void* const*) a.wg, r.wu = (const void* const*) a.wu, r.cnt = a.cnt, r.xrow = a.xrow;
  r.xin = a.xin, r.win = a.win, r.q = a.q, r.d = a.d, r.scale = a.scale, r.lim = a.lim, r.out = a.out, r.rows = a.rows;
  r.cols = a.cols, r.out_stride = a.out_stride, r.n_entries = n_entries, r.max_cnt = max_cnt;
  return ring::try_launch(type, r, stream);
}

// the staged kernel when it takes the shape: 1 queued, 0 not taken, -1 refused
int staged_first(uint32_t type, const LaneArgs& a, bool fused, bool dense, uint32_t n_entries, uint32_t max_cnt, void* stream) {
  if (!g_use_staged) return 0;
  staged::Request r{};
  r.fused = fused, r.dense = dense, r.w_dense = a.w_dense, r.wg = (const void* const*) a.wg, r.wu = (const void* const*) a.wu;
  r.cnt = a.cnt, r.xrow = a.xrow, r.xin = a.xin, r.win = a.win, r.q = a.q, r.d = a.d, r.scale = a.scale, r.lim = a.lim;
  r.out = a.out, r.rows = a.rows, r.cols = a.cols, r.out_stride = a.out_stride, r.n_entries = n_entries;
  r.max_cnt = max_cnt, r.n_tok = a.n_tok;
  return staged::try_launch(type, r, stream);
}

}  // namespace

bool q8_gate_up_ep(uint32_t type, const void* const* wg, const void* const* wu, const int32_t* cnt, const int32_t* xrow,
                   const int32_t* xin, const int32_t* win, uint32_t n, uint32_t max_cnt, uint32_t rows, uint32_t cols,
                   const int8_t* q, const float* d, const float* scale, float lim, float* h, uint32_t hs, const LaneEp& ep,
                   bool dry, cudaStream_t s) {
  if (!n || n > MV_MAX_GROUP || !rows || !max_cnt || max_cnt > MV_MAX_TOKENS || !cols || cols % 256 || hs < rows) return false;
  if (!dry && (!wg || !wu || !cnt || !xrow || !q || !d || !h || !scale)) return false;
  if (!qtype_row(type) || !(qtype_row(type)->paths & QTYPE_PATH_Q8)) return false;
  ring::Request r{};
  r.fused = true, r.wg = wg, r.wu = wu, r.cnt = cnt, r.xrow = xrow, r.xin = xin, r.win = win, r.q = q, r.d = d;
  r.scale = scale, r.lim = lim, r.out = h, r.rows = rows, r.cols = cols, r.out_stride = hs, r.n_entries = n;
  r.max_cnt = max_cnt, r.ep = ep, r.dry = dry;
  return ring::try_launch(type, r, s) > 0;
}

bool q8_group_tok_ep(uint32_t type, const void* const* w, const int32_t* cnt, const int32_t* xrow, const int32_t* xin,
                     uint32_t n, uint32_t max_cnt, uint32_t rows, uint32_t cols, const int8_t* q, const float* d, float* y,
                     uint32_t ys, const LaneEp& ep, bool dry, cudaStream_t s) {
  if (!n || n > MV_MAX_GROUP || !rows || !max_cnt || max_cnt > MV_MAX_TOKENS || !cols || cols % 256) return false;
  if (!dry && (!w || !cnt || !xrow || !q || !d || (!y && !ep.out_rows))) return false;
  if (!qtype_row(type) || !(qtype_row(type)->paths & QTYPE_PATH_Q8)) return false;
  rows::Request rr{w, cnt, xrow, xin, q, d, y, rows, cols, ys, n, max_cnt, ep, dry};
  if (const int st = rows::try_launch(type, rr, s)) return st > 0;
  ring::Request r{};
  r.fused = false, r.wg = w, r.cnt = cnt, r.xrow = xrow, r.xin = xin, r.q = q, r.d = d, r.out = y, r.rows = rows;
  r.cols = cols, r.out_stride = ys, r.n_entries = n, r.max_cnt = max_cnt, r.ep = ep, r.dry = dry;
  return ring::try_launch(type, r, s) > 0;
}

}  // namespace osmos

using namespace osmos;

extern "C" bool q8_known(uint32_t type) { return qtype_row(type) && (qtype_row(type)->paths & QTYPE_PATH_Q8); }
extern "C" void q8_set_staged(int on) { g_use_staged = on; }
extern "C" uint32_t q8_status(void) { return staged::read_status() | plain::read_status() | ring::read_status() | rows::read_status(); }

extern "C" bool q8_round(const float* x, uint32_t rows, uint32_t cols, uint32_t xs, int8_t* q, float* d, void* stream) {
  return round_rows<false>(x, rows, cols, xs, q, d, stream_of(stream));
}

extern "C" bool q8_0_round(const float* x, uint32_t rows, uint32_t cols, uint32_t xs, int8_t* q, float* d,
                           void* stream) {
  return round_rows<true>(x, rows, cols, xs, q, d, stream_of(stream));
}

extern "C" bool q8_group_tok(uint32_t type, const void* const* w, const int32_t* cnt, const int32_t* xrow,
                             const int32_t* xin, uint32_t n, uint32_t max_cnt, uint32_t rows, uint32_t cols,
                             const int8_t* q, const float* d, float* y, uint32_t ys, void* stream) {
  if (!w || !cnt || !xrow || !q || !d || !y || !n || n > MV_MAX_GROUP || !rows || !max_cnt ||
      max_cnt > MV_MAX_TOKENS || !cols || cols % 256)
    return false;
  LaneArgs a{};
  a.wg = (const uint8_t* const*) w, a.cnt = cnt, a.xrow = xrow, a.xin = xin, a.q = q, a.d = d, a.out = y;
  a.rows = rows, a.cols = cols, a.out_stride = ys;
  if (qtype_row(type) && (qtype_row(type)->paths & QTYPE_PATH_Q8)) {
    if (g_use_staged == 1) {  // 512-column matrices: a thread a row
      const rows::Request r{w, cnt, xrow, xin, q, d, y, rows, cols, ys, n, max_cnt, LaneEp{}, false};
      if (const int st = rows::try_launch(type, r, stream)) return st > 0;
    }
    if (const int st = ring_first(type, a, false, n, max_cnt, stream)) return st > 0;
    if (const int st = staged_first(type, a, false, false, n, max_cnt, stream)) return st > 0;
  }
#define CASE(T) return by_tokens<T, false, false>(a, max_cnt, n, stream_of(stream));
  OSMOS_SWITCH_LANE(type, CASE, return false)
#undef CASE
}

extern "C" bool q8_gate_up(uint32_t type, const void* const* wg, const void* const* wu, const int32_t* cnt,
                           const int32_t* xrow, const int32_t* xin, const int32_t* win, uint32_t n, uint32_t max_cnt,
                           uint32_t rows, uint32_t cols, const int8_t* q, const float* d, const float* scale, float lim,
                           float* h, uint32_t hs, void* stream) {
  if (!wg || !wu || !cnt || !xrow || !q || !d || !h || !n || n > MV_MAX_GROUP || !rows || !max_cnt ||
      max_cnt > MV_MAX_TOKENS || !cols || cols % 256 || !scale || hs < rows)
    return false;
  LaneArgs a{};
  a.wg = (const uint8_t* const*) wg, a.wu = (const uint8_t* const*) wu, a.cnt = cnt, a.xrow = xrow, a.xin = xin;
  a.win = win, a.q = q, a.d = d, a.scale = scale, a.lim = lim, a.out = h, a.rows = rows, a.cols = cols, a.out_stride = hs;
  if (qtype_row(type) && (qtype_row(type)->paths & QTYPE_PATH_Q8)) {
    if (const int st = ring_first(type, a, true, n, max_cnt, stream)) return st > 0;
    if (const int st = staged_first(type, a, true, false, n, max_cnt, stream)) return st > 0;
  }
#define CASE(T) return by_tokens<T, true, false>(a, max_cnt, n, stream_of(stream));
  OSMOS_SWITCH_LANE(type, CASE, return false)
#undef CASE
}

extern "C" bool q8_run(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const int8_t* q, const float* d,
                       uint32_t n_tok, float* y, uint32_t ys, void* stream) {
  const OsmosQTypeInfo* t = qtype_row(type);
  if (!t || !w || !q || !d || !y || !rows || !n_tok || !cols || cols % t->values || cols % 32 || (n_tok > 1 && ys < rows))
    return false;
  LaneArgs a{};
  a.w_dense = (const uint8_t*) w, a.q = q, a.d = d, a.out = y, a.rows = rows, a.cols = cols, a.out_stride = ys;
  a.n_tok = n_tok;
  if (g_use_staged) {  // the plain blocks' own kernel (Q4_0, Q8_0; one or two tokens)
    const plain::Request r{w, q, d, y, rows, cols, ys, n_tok};
    if (const int st = plain::try_launch(type, r, stream)) return st > 0;
  }
  if (t->paths & (QTYPE_PATH_Q8 | QTYPE_PATH_Q8_EXT))
    if (const int st = staged_first(type, a, false, true, 1, n_tok, stream)) return st > 0;
#define CASE(T)                                                                                        \
  return n_tok > 8 ? launch<T, 8, false, true>(a, (n_tok + 7) / 8, stream_of(stream))                  \
                   : by_tokens<T, false, true>(a, n_tok, 1, stream_of(stream));
  OSMOS_SWITCH_LANE_EXT(type, CASE, return false)
#undef CASE
}
