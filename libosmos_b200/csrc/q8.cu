// The int8 lane (include/osmos_b200/q8.h): activation rounding and the grouped expert matvecs over int8 inputs,
// with the gate + up + activation fusion. One kernel template serves q8_group_tok, q8_gate_up and q8_run.
//
// This generic kernel takes any shape the entry points accept. A block owns one entry (or one group of a dense call's
// tokens) and a run of its rows: the entry's tokens - their int8 rows and block scales - are brought into shared
// memory once, NT at a time, and every row of the run reads them from there; a thread is a lane of the contract, a
// warp holds 32 / L rows at a time and walks the run. The order of every floating-point operation is fixed by the
// contract (a lane's blocks in ascending order, the xor tree, the activation), so any other kernel for the same
// entry points must (and is tested to) give the same bits.
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
constexpr uint32_t kTokenSmem = 160u * 1024u;  // the most shared memory a block's tokens may take

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
  uint32_t max_cnt;   // the grouped forms: the most tokens an entry has
  uint32_t run_rows;  // rows a block walks (a multiple of the rows its warps hold at once)
};

template <uint32_t T, int NT, bool FUSED, bool DENSE>
__global__ void __launch_bounds__(kThreads) lane_kernel(const LaneArgs a) {
  extern __shared__ __align__(16) uint8_t tokens[];  // NT int8 rows, then their NT rows of block scales
  __shared__ __align__(16) uint8_t tables[grid_smem_bytes<T>() > 0 ? grid_smem_bytes<T>() : 16];
  __shared__ uint32_t s_src[NT];  // where each staged token's row lies in q / d
  const Grids g = stage_grids<T>(tables);
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t L = a.cols >= kLongCols ? 32u : 16u, sub = lane % L, at_once = kWarp / L;
  const uint32_t nblk = a.cols / 32, pieces = a.cols / 16;
  const int4* const xq = (const int4*) tokens;
  const float* const xd = (const float*) (tokens + (size_t) NT * a.cols);

  // whose tokens: `count` rows of the inputs from `first`, and the matrices they meet
  uint32_t first, count;
  const uint8_t *wg, *wu = nullptr;
  if constexpr (DENSE) {
    first = blockIdx.y * NT, count = a.n_tok - first < (uint32_t) NT ? a.n_tok - first : (uint32_t) NT;
    wg = a.w_dense;
  } else {
    const uint32_t m = blockIdx.y;
    const int32_t c = a.cnt[m];
    if (c <= 0) return;
    first = (uint32_t) a.xrow[m], count = (uint32_t) c < a.max_cnt ? (uint32_t) c : a.max_cnt;
    wg = a.wg[m];
    if constexpr (FUSED) wu = a.wu[m];
  }
  const uint64_t row_bytes = (uint64_t) (a.cols / Fmt<T>::values) * Fmt<T>::bytes;
  const uint32_t run0 = blockIdx.x * a.run_rows, run1 = run0 + a.run_rows < a.rows ? run0 + a.run_rows : a.rows;
  constexpr int kSubs = Fmt<T>::subs;

  for (uint32_t t0 = 0; t0 < count; t0 += NT) {
    const uint32_t live = count - t0 < (uint32_t) NT ? count - t0 : (uint32_t) NT;
    // ---- the group's tokens into shared memory
    if (t0) __syncthreads();  // (the rows of the group before are done with it)
    if (tid < live) s_src[tid] = a.xin ? (uint32_t) a.xin[first + t0 + tid] : first + t0 + tid;
    __syncthreads();
    for (uint32_t i = tid; i < live * pieces; i += kThreads) {
      const uint32_t t = i / pieces, c = i - t * pieces;
      ((int4*) tokens)[t * pieces + c] = __ldg((const int4*) (a.q + (uint64_t) s_src[t] * a.cols) + c);
    }
    for (uint32_t i = tid; i < live * nblk; i += kThreads) {
      const uint32_t t = i / nblk, c = i - t * nblk;
      ((float*) (tokens + (size_t) NT * a.cols))[t * nblk + c] = __ldg(a.d + (uint64_t) s_src[t] * nblk + c);
    }
    __syncthreads();
    // ---- the run's rows, 32 / L a warp at a time
    for (uint32_t base = run0 + warp * at_once; base < run1; base += kWarps * at_once) {
      const uint32_t row = base + lane / L;  // (a row past the matrix is computed from row 0 and dropped)
      const uint64_t off = (uint64_t) (row < a.rows ? row : 0) * row_bytes;
      float ag[NT], au[NT];
#pragma unroll
      for (int t = 0; t < NT; t++) ag[t] = au[t] = 0.0f;
      for (uint32_t s = sub; s < nblk; s += L) {
        LaneCodes cg, cu;
        const uint64_t at = off + (uint64_t) (s / kSubs) * Fmt<T>::bytes;
        lane_codes<T>(wg + at, (int) (s % kSubs), cg, g);
        if constexpr (FUSED) lane_codes<T>(wu + at, (int) (s % kSubs), cu, g);
#pragma unroll
        for (int t = 0; t < NT; t++) {
          if ((uint32_t) t < live) {
            const int4 lo = xq[(uint32_t) t * pieces + 2 * s], hi = xq[(uint32_t) t * pieces + 2 * s + 1];
            const int x[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const float dx = xd[(uint32_t) t * nblk + s];
            ag[t] = __fmaf_rn(dx, lane_block_sum<T>(cg, x), ag[t]);
            if constexpr (FUSED) au[t] = __fmaf_rn(dx, lane_block_sum<T>(cu, x), au[t]);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < NT; t++) {
        float vg = ag[t], vu = au[t];
        for (uint32_t o = L / 2; o > 0; o >>= 1) {
          vg = __fadd_rn(vg, __shfl_xor_sync(0xFFFFFFFFu, vg, o, kWarp));
          if constexpr (FUSED) vu = __fadd_rn(vu, __shfl_xor_sync(0xFFFFFFFFu, vu, o, kWarp));
        }
        if (sub == 0 && row < a.rows && (uint32_t) t < live) {
          const uint64_t r = first + t0 + (uint32_t) t;
          if constexpr (FUSED)
            a.out[r * a.out_stride + row] = lane_swiglu(vg, vu, a.lim, a.scale[a.win ? a.win[r] : r]);
          else
            a.out[r * a.out_stride + row] = vg;
        }
      }
    }
  }
}

// tokens a block stages at once: the fewest of 1, 2, 4, 8 that cover n, fewer where their rows would not fit
template <uint32_t T, int NT, bool FUSED, bool DENSE>
bool launch(LaneArgs a, uint32_t grid_y, cudaStream_t s) {
  const uint32_t bytes = (uint32_t) NT * (a.cols + a.cols / 32 * 4);
  if (bytes > kTokenSmem) {
    if constexpr (NT > 1) return launch<T, NT / 2, FUSED, DENSE>(a, DENSE ? (a.n_tok + NT / 2 - 1) / (NT / 2) : grid_y, s);
    return false;
  }
  // rows a block walks: as many as leave every SM about two blocks, at most eight passes of its warps
  const uint32_t at_once = kWarps * (kWarp / (a.cols >= kLongCols ? 32u : 16u));
  int sms = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return false;
  uint32_t passes = 8;
  while (passes > 1 && (uint64_t) blocks_for(a.rows, at_once * passes) * grid_y < 2u * (uint32_t) sms) passes >>= 1;
  a.run_rows = at_once * passes;
  static bool sized[64] = {};  // (one record a template instance, one flag a device)
  auto kernel = lane_kernel<T, NT, FUSED, DENSE>;
  if (!allow_dynamic_smem(kernel, (int) kTokenSmem, sized)) return false;
  kernel<<<dim3(blocks_for(a.rows, a.run_rows), grid_y), kThreads, bytes, s>>>(a);
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
  a.rows = rows, a.cols = cols, a.out_stride = ys, a.max_cnt = max_cnt;
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
  a.max_cnt = max_cnt;
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
