// Routing, expert tables, activation and combine of an MoE layer (include/osmos_b200/moe.h), and the device-built
// tables of the int8 lane (include/osmos_b200/lane.h). Everything here is built on the GPU: no host round trip
// between the router and the experts.
//
// The router is a warp a token (route.cuh). The tables are one block of 1024 threads: a thread an expert for the
// counts and the prefix sums (every sum of the block in ONE pass of shuffles, whatever their number), and the picks'
// places by the first warp walking the picks 32 at a time in pick order - lanes with the same expert find each other
// with match.any, the group's first lane reserves the group's places in the expert's running fill - which is the
// stable sort by expert without a thread ever scanning the picks before its own.
#include "moe_api.h"

#include "act.cuh"
#include "decode.cuh"
#include "osmos_b200/moe.h"
#include "route.cuh"

namespace osmos {
namespace {

constexpr int kThreads = 256;
constexpr uint32_t kMaxExperts = 1024, kMaxK = 32;

// ---- the router ----------------------------------------------------------------------------------------------------
constexpr int kRouteWarps = 4;  // tokens a block

template <int R>
__global__ void __launch_bounds__(kRouteWarps* kWarp) route_kernel(const float* __restrict__ logits, uint32_t n_tok,
                                                                   uint32_t n_exp, uint32_t k, int32_t* __restrict__ ids,
                                                                   float* __restrict__ w, int32_t* __restrict__ rows) {
  pdl_wait();  // (a dependent launch: the step before may still be reading the ids and weights this one writes)
  pdl_launch_next();
  const uint32_t t = blockIdx.x * kRouteWarps + threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
  if (t >= n_tok) return;  // (the whole warp)
  const route::Pick p = route::softmax_topk<R>(logits + (uint64_t) t * n_exp, n_exp, k, lane);
  if (lane < k) ids[t * k + lane] = (int32_t) p.id, w[t * k + lane] = p.w, rows[t * k + lane] = (int32_t) t;
}

// ---- per-expert tables ---------------------------------------------------------------------------------------------
constexpr int kTableThreads = 1024;  // a thread an expert
constexpr int kTableWarps = kTableThreads / kWarp;
constexpr int kPart = MM_TILE << (Q4X_TILE_RUNS - 1);  // an entry's most tokens (128)
constexpr uint32_t kInlinePicks = 1024;  // up to this many picks are placed by the table kernel itself

__device__ __forceinline__ int tile_run(int c) { return c <= 16 ? 0 : c <= 32 ? 1 : c <= 64 ? 2 : 3; }

// N exclusive prefix sums over the block's kTableThreads threads at once: v[i] becomes the sum of the v[i] of the
// threads before this one, total[i] the sum over all threads. One pass: a shuffle scan in each warp, the warps' sums
// through shared memory, the first N warps scanning one array each. Integers: any order gives the same result.
template <int N>
__device__ __forceinline__ void block_exclusive(int (&v)[N], int (&total)[N], int (*warp_sums)[kTableWarps]) {
  static_assert(N <= kTableWarps, "one warp scans one array of warp sums");
  const int lane = threadIdx.x % kWarp, wid = threadIdx.x / kWarp;
  int inc[N];
#pragma unroll
  for (int i = 0; i < N; i++) {
    inc[i] = v[i];
#pragma unroll
    for (int o = 1; o < kWarp; o <<= 1) {
      const int up = __shfl_up_sync(0xFFFFFFFFu, inc[i], o, kWarp);
      if (lane >= o) inc[i] += up;
    }
  }
  __syncthreads();  // the scratch free of its last use
  if (lane == kWarp - 1)
#pragma unroll
    for (int i = 0; i < N; i++) warp_sums[i][wid] = inc[i];
  __syncthreads();
  if (wid < N) {
    int s = warp_sums[wid][lane];
#pragma unroll
    for (int o = 1; o < kWarp; o <<= 1) {
      const int up = __shfl_up_sync(0xFFFFFFFFu, s, o, kWarp);
      if (lane >= o) s += up;
    }
    warp_sums[wid][lane] = s;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; i++) {
    total[i] = warp_sums[i][kWarp - 1];
    v[i] = inc[i] - v[i] + (wid ? warp_sums[i][wid - 1] : 0);
  }
}

// The picks' ranks inside their experts, in pick order, by the calling warp alone: sids[i] the pick's expert (or -1: not
// placed), fill[e] the places of expert e handed out so far (zero on entry). rank[i] = how many picks of the same expert
// come before pick i.
__device__ __forceinline__ void rank_picks(const int32_t* sids, uint32_t n, int* fill, uint16_t* rank) {
  const uint32_t lane = threadIdx.x % kWarp;
  for (uint32_t i0 = 0; i0 < n; i0 += kWarp) {
    const uint32_t i = i0 + lane;
    const int32_t id = i < n ? sids[i] : -1;
    const uint32_t same = __match_any_sync(0xFFFFFFFFu, id);
    const uint32_t first = (uint32_t) __ffs((int) same) - 1u;
    int base = 0;
    if (lane == first && id >= 0) {
      base = fill[id];
      fill[id] = base + __popc(same);
    }
    __syncwarp();
    base = __shfl_sync(0xFFFFFFFFu, base, (int) first, kWarp);
    if (id >= 0) rank[i] = (uint16_t) (base + __popc(same & ((1u << lane) - 1u)));
  }
}

__global__ void __launch_bounds__(kTableThreads) tiles_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t k,
                                                              uint32_t n_exp, uint32_t dim, uint32_t ff,
                                                              const Q4xExpertTiles t, const Q4xExpertBounds bd) {
  __shared__ int count[kMaxExperts], place0[kMaxExperts], slot0[kMaxExperts], warp_sums[2 + Q4X_TILE_RUNS][kTableWarps];
  __shared__ int32_t sids[kInlinePicks];
  __shared__ uint16_t rank[kInlinePicks];
  pdl_wait();  // (a dependent launch: ids are the router's output)
  pdl_launch_next();
  const uint32_t e = threadIdx.x;
  const bool inline_place = n <= kInlinePicks;
  count[e] = 0;
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = ids[i];
    const bool known = (uint32_t) id < n_exp;  // (an id outside the experts has no place: it is left out)
    if (known) atomicAdd(&count[id], 1);
    if (inline_place) sids[i] = known ? id : -1;
  }
  __syncthreads();
  const int c = e < n_exp ? count[e] : 0;
  const int padded = (c + MM_TILE - 1) / MM_TILE * MM_TILE, last = c % kPart;
  // the expert's first place, first slot, and first entry in each run of tile counts
  int first[2 + Q4X_TILE_RUNS], total[2 + Q4X_TILE_RUNS];
  first[0] = c, first[1] = padded;
#pragma unroll
  for (int r = 0; r < Q4X_TILE_RUNS; r++)
    first[2 + r] = (r == Q4X_TILE_RUNS - 1 ? c / kPart : 0) + (last && tile_run(last) == r);
  block_exclusive(first, total, warp_sums);
  place0[e] = first[0], slot0[e] = first[1];
  count[e] = 0;  // (the fill counters of the ranking below)
  if (e < n_exp) {
    t.off[e] = first[0], t.off[n_exp + e] = first[1], t.off[2 * n_exp + e] = c;
    for (int s = first[1] + c; s < first[1] + padded; s++) t.gidx[s] = -1, t.hidx[s] = -1;
    // the expert's tokens in parts of at most 128, each an entry of the run its tile count belongs to
    for (int done = 0; done < c; done += kPart) {
      const int m = c - done < kPart ? c - done : kPart, r = tile_run(m);
      const uint32_t en = bd.first[r] + (uint32_t) first[2 + r]++;
      const uint32_t slot = (uint32_t) (first[1] + done), place = (uint32_t) (first[0] + done);
      t.cnt[en] = m;
      t.xg[en] = slot * dim, t.xd[en] = slot * ff, t.yg[en] = place * ff, t.yd[en] = place * dim;
#pragma unroll
      for (int j = 0; j < Q4X_GROUP_TENSORS; j++)
        t.ptr[j][en] = t.tab[j] ? t.tab[j][e] : (const uint8_t*) t.base[j] + (uint64_t) e * t.bytes[j];
    }
  }
  // the tables' tails, launched to their bounds: entries of no tokens, slots of no token
#pragma unroll
  for (int r = 0; r < Q4X_TILE_RUNS; r++)
    for (uint32_t i = (uint32_t) total[2 + r] + threadIdx.x; i < bd.count[r]; i += kTableThreads) t.cnt[bd.first[r] + i] = 0;
  for (uint32_t s = (uint32_t) total[1] + threadIdx.x; s < bd.slots; s += kTableThreads) t.gidx[s] = -1, t.hidx[s] = -1;
  if (!inline_place) return;  // place_kernel's
  __syncthreads();
  if (threadIdx.x < kWarp) rank_picks(sids, n, count, rank);
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = sids[i];
    if (id < 0) continue;
    const int q = place0[id] + rank[i], s = slot0[id] + rank[i];
    t.where[i] = q, t.gidx[s] = (int32_t) (i / k), t.hidx[s] = q;
  }
}

// a block an expert: its picks in pick order, a block-wide tile of picks at a time - each pick's rank the expert's
// picks before it (in the tile: by ballots; before the tile: a running count)
template <class Put>
__device__ __forceinline__ void place_expert(const int32_t* __restrict__ ids, uint32_t n, int32_t e, int c, Put put) {
  __shared__ int warp_cnt[kThreads / kWarp];
  const int lane = threadIdx.x % kWarp, wid = threadIdx.x / kWarp;
  int done = 0;
  for (uint32_t i0 = 0; i0 < n && done < c; i0 += kThreads) {
    const uint32_t i = i0 + threadIdx.x;
    const bool f = i < n && ids[i] == e;
    const uint32_t votes = __ballot_sync(0xFFFFFFFFu, f);
    if (lane == 0) warp_cnt[wid] = __popc(votes);
    __syncthreads();
    int before = 0, tile = 0;
#pragma unroll
    for (int wdx = 0; wdx < kThreads / kWarp; wdx++) {
      before += wdx < wid ? warp_cnt[wdx] : 0;
      tile += warp_cnt[wdx];
    }
    if (f) put(i, done + before + __popc(votes & ((1u << lane) - 1u)));
    done += tile;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads) place_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t k,
                                                         uint32_t n_exp, const Q4xExpertTiles t) {
  const int32_t e = (int32_t) blockIdx.x;
  const int c = t.off[2 * n_exp + e];
  if (!c) return;
  const int p0 = t.off[e], s0 = t.off[n_exp + e];
  place_expert(ids, n, e, c, [&](uint32_t i, int rank) {
    const int q = p0 + rank;
    t.where[i] = q, t.gidx[s0 + rank] = (int32_t) (i / k), t.hidx[s0 + rank] = q;
  });
}

// ---- the int8 lane's tables (include/osmos_b200/lane.h) -----------------------------------------------------------
// a token's rows in ascending row (= ascending expert id), the picks without a row here (-1) last: k is small, one
// thread sorts by insertion
template <class Rows>
__device__ __forceinline__ void order_token(Rows row_of, uint32_t t, uint32_t k, int32_t* order) {
  int32_t r[kMaxK];
  for (uint32_t j = 0; j < k; j++) r[j] = row_of(t * k + j);
  for (uint32_t a = 1; a < k; a++)
    for (uint32_t c = a; c > 0 && (uint32_t) r[c] < (uint32_t) r[c - 1]; c--) {
      const int32_t s = r[c];
      r[c] = r[c - 1], r[c - 1] = s;
    }
  for (uint32_t j = 0; j < k; j++) order[t * k + j] = r[j];
}

// where row (token t, pick j) of the exchange goes: its home rank's receive block, row (t % tokens) * k + j
__device__ __forceinline__ float* home_row(const LaneRowHomes& h, uint32_t half, uint32_t i, uint32_t k) {
  const uint32_t t = i / k, j = i % k;
  return (float*) (h.base[t / h.tokens] + h.recv[half]) + ((uint64_t) (t % h.tokens) * k + j) * h.dim;
}

__global__ void __launch_bounds__(kTableThreads) lane_tables_kernel(const int32_t* __restrict__ ids, uint32_t n,
                                                                    uint32_t k, uint32_t n_exp, const LaneExperts ex,
                                                                    const LaneTables t, uint32_t e0, uint32_t e1,
                                                                    const LaneTablesSync sy, const LaneRowHomes homes) {
  __shared__ int count[kMaxExperts], first_row[kMaxExperts], warp_sums[2][kTableWarps];
  __shared__ int32_t sids[kInlinePicks], srow[kInlinePicks];
  __shared__ uint16_t rank[kInlinePicks];
  pdl_wait();  // (a dependent launch: ids are the router's output)
  pdl_launch_next();
  const uint32_t e = threadIdx.x;
  const bool inline_place = n <= kInlinePicks;
  count[e] = 0;
  uint32_t step = 0;
  if (sy.flags) {  // expert-parallel: the picks are the peers' - every peer's flag must have reached this step
    step = *sy.step;
    if (threadIdx.x < sy.n_ranks && !flag_wait(sy.flags + threadIdx.x, step, sy.n_ranks == 1)) atomicOr(sy.status, 1u);
    ids = (const int32_t*) ((const uint8_t*) ids + (step & 1u) * sy.half_bytes);
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = ids[i];
    const bool own = (uint32_t) id >= e0 && (uint32_t) id < e1;  // experts outside [e0, e1) are another rank's
    if (own) atomicAdd(&count[id], 1);
    if (inline_place) sids[i] = own ? id : -1;
  }
  __syncthreads();
  const int c = e < n_exp ? count[e] : 0;
  int first[2] = {c, (c + LANE_MAX_TOKENS - 1) / LANE_MAX_TOKENS}, total[2];
  const int parts = first[1];
  block_exclusive(first, total, warp_sums);
  first_row[e] = first[0];
  count[e] = 0;  // (the fill counters of the ranking below)
  if (e < n_exp) {
    t.off[e] = first[0], t.off[n_exp + e] = c;
    for (int part = 0; part < parts; part++) {
      const int en = first[1] + part, left = c - part * LANE_MAX_TOKENS;
      t.cnt[en] = left < LANE_MAX_TOKENS ? left : LANE_MAX_TOKENS;
      t.xrow[en] = first[0] + part * LANE_MAX_TOKENS;
#pragma unroll
      for (int j = 0; j < 3; j++)
        t.w[j][en] = ex.tab[j] ? ex.tab[j][e] : (const uint8_t*) ex.base[j] + (uint64_t) e * ex.bytes[j];
    }
  }
  for (uint32_t i = (uint32_t) total[1] + threadIdx.x; i < t.max_entries; i += kTableThreads) t.cnt[i] = 0;
  if (threadIdx.x == 0) t.counts[0] = total[1], t.counts[1] = total[0];
  if (!inline_place) return;  // lane_place_kernel's
  __syncthreads();
  if (threadIdx.x < kWarp) rank_picks(sids, n, count, rank);
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = sids[i];
    const int r = id < 0 ? -1 : first_row[id] + rank[i];
    srow[i] = r, t.row_of[i] = r;
    if (r < 0) continue;
    t.tok[r] = (int32_t) (i / k), t.pair[r] = (int32_t) i;
    if (homes.rows) homes.rows[r] = home_row(homes, step & 1u, i, k);
    if (homes.scale) homes.scale[r] = ((const float*) ((const uint8_t*) sy.weights + (step & 1u) * sy.weights_half))[i];
  }
  // each token's rows in order, in the same launch, a thread a pick: its place among its token's picks is the number
  // of them with a smaller row (the picks without a row, -1, compare as the largest; equal ones keep their order)
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const uint32_t first = i / k * k, mine = (uint32_t) srow[i];
    uint32_t place = 0;
    for (uint32_t j = first; j < first + k; j++) {
      const uint32_t other = (uint32_t) srow[j];
      place += other < mine || (other == mine && j < i);
    }
    t.order[first + place] = (int32_t) mine;
  }
}

__global__ void __launch_bounds__(kThreads) lane_place_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t k,
                                                              uint32_t n_exp, const LaneTables t, uint32_t e0,
                                                              uint32_t e1) {
  const int32_t e = (int32_t) blockIdx.x;
  if ((uint32_t) e < e0 || (uint32_t) e >= e1) {  // not this rank's: its picks have no row here
    for (uint32_t i = threadIdx.x; i < n; i += kThreads)
      if (ids[i] == e) t.row_of[i] = -1;
    return;
  }
  const int c = t.off[n_exp + e];
  if (!c) return;
  const int r0 = t.off[e];
  place_expert(ids, n, e, c, [&](uint32_t i, int rank) {
    t.tok[r0 + rank] = (int32_t) (i / k), t.pair[r0 + rank] = (int32_t) i, t.row_of[i] = r0 + rank;
  });
}

__global__ void lane_order_kernel(const int32_t* __restrict__ row_of, uint32_t n_tok, uint32_t k,
                                  int32_t* __restrict__ order) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tok) return;
  order_token([&](uint32_t i) { return row_of[i]; }, t, k, order);
}

// ---- activation and combine ------------------------------------------------------------------------------------
// four neighbouring values a thread where the addresses allow it (VEC 4), else one
template <int VEC>
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u, uint64_t n,
                                                          float* __restrict__ y, const Q4xX16 side) {
  const uint64_t i = ((uint64_t) blockIdx.x * kThreads + threadIdx.x) * VEC;
  if (i >= n) return;
  float gv[VEC], uv[VEC], out[VEC];
  if constexpr (VEC == 4) {
    const float4 a = *(const float4*) (g + i), b = *(const float4*) (u + i);
    gv[0] = a.x, gv[1] = a.y, gv[2] = a.z, gv[3] = a.w, uv[0] = b.x, uv[1] = b.y, uv[2] = b.z, uv[3] = b.w;
  } else {
    gv[0] = g[i], uv[0] = u[i];
  }
#pragma unroll
  for (int v = 0; v < VEC; v++) out[v] = mul_rn(siluf(gv[v]), uv[v]);
  if constexpr (VEC == 4) *(float4*) (y + i) = make_float4(out[0], out[1], out[2], out[3]);
  else y[i] = out[0];
  if (side.x16)
#pragma unroll
    for (int v = 0; v < VEC; v++)
      x16_store((__half*) side.x16, side.overflow, side.row0 + (uint32_t) ((i + v) / side.cols), (uint32_t) ((i + v) % side.cols),
                side.cols, out[v]);
}

// the activation straight into down's tiled f16 input: slot s takes row idx[s] of g and u (a pad slot, -1, zeros); a
// thread eight neighbouring columns of a slot - half a tile row, one 16-byte store
__global__ void __launch_bounds__(kThreads) swiglu_rows_kernel(const float* __restrict__ g, const float* __restrict__ u, uint32_t ff,
                                                               const int32_t* __restrict__ idx, uint32_t slots,
                                                               __half* __restrict__ x16, int32_t* overflow) {
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  const uint32_t per = ff / 8;
  if (i >= (uint64_t) slots * per) return;
  const uint32_t s = (uint32_t) (i / per), c = (uint32_t) (i % per) * 8;
  const int32_t r = idx[s];
  __align__(16) __half h[8];
  bool over = false;
  if (r >= 0) {
    const float* gp = g + (uint64_t) r * ff + c;
    const float* up = u + (uint64_t) r * ff + c;
#pragma unroll
    for (int v = 0; v < 8; v++) {
      const float o = mul_rn(siluf(gp[v]), up[v]);
      over |= !(fabsf(o) <= 65504.0f);
      h[v] = __float2half_rn(o);
    }
  } else {
#pragma unroll
    for (int v = 0; v < 8; v++) h[v] = __float2half_rn(0.0f);
  }
  if (over) atomicOr(overflow, 1);
  *(uint4*) (x16 + (uint64_t) (s / 16) * 16 * ff + (c / 16) * 256 + (s % 16) * 16 + c % 16) = *(const uint4*) h;
}

template <int VEC>
__global__ void moe_sum_kernel(const float* __restrict__ y, const int32_t* __restrict__ where, const float* __restrict__ w,
                               uint64_t total, uint32_t k, uint32_t dim, const float* __restrict__ shared,
                               const float* __restrict__ shared_logit, float* __restrict__ out) {
  const uint64_t i = ((uint64_t) blockIdx.x * kThreads + threadIdx.x) * VEC;
  if (i >= total) return;
  const uint64_t t = i / dim, c = i % dim;
  float sum[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) sum[v] = 0.0f;
  for (uint32_t j = 0; j < k; j++) {
    const float* row = y + (uint64_t) where[t * k + j] * dim + c;
    const float wj = w[t * k + j];
    if constexpr (VEC == 4) {
      const float4 v = *(const float4*) row;
      sum[0] = __fadd_rn(sum[0], mul_rn(v.x, wj)), sum[1] = __fadd_rn(sum[1], mul_rn(v.y, wj));
      sum[2] = __fadd_rn(sum[2], mul_rn(v.z, wj)), sum[3] = __fadd_rn(sum[3], mul_rn(v.w, wj));
    } else {
      sum[0] = __fadd_rn(sum[0], mul_rn(row[0], wj));
    }
  }
  const float gate = sigmoidf(shared_logit[t]);
#pragma unroll
  for (int v = 0; v < VEC; v++) out[i + v] = __fadd_rn(sum[v], mul_rn(shared[i + v], gate));
}

}  // namespace

// the lane tables with the expert-parallel step's extras (moe_api.h); sy.flags / homes.rows NULL: the plain tables
bool lane_tables_launch(const int32_t* ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t expert0, uint32_t expert1,
                        const LaneExperts* ex, const LaneTables* t, const LaneTablesSync& sy, const LaneRowHomes& homes,
                        cudaStream_t s) {
  if (!ids || !n || !k || n % k || k > kMaxK || !n_exp || n_exp > kMaxExperts || expert0 >= expert1 ||
      expert1 > n_exp || !ex || !t || !t->cnt || !t->xrow || !t->tok || !t->pair || !t->row_of || !t->order ||
      !t->off || !t->counts || t->max_entries < lane_max_entries(n, n_exp))
    return false;
  for (int j = 0; j < 3; j++)
    if ((!ex->tab[j] && (!ex->base[j] || !ex->bytes[j])) || !t->w[j]) return false;
  if ((sy.flags || homes.rows) && n > kInlinePicks) return false;  // (the exchange's step is a decode step: few picks)
  if (launch_dependent(lane_tables_kernel, dim3(1), dim3(kTableThreads), 0, s, ids, n, k, n_exp, *ex, *t, expert0, expert1,
                       sy, homes) != cudaSuccess)
    return false;
  if (n > kInlinePicks) {
    lane_place_kernel<<<n_exp, kThreads, 0, s>>>(ids, n, k, n_exp, *t, expert0, expert1);
    if (!launched()) return false;
    lane_order_kernel<<<blocks_for(n / k, 128), 128, 0, s>>>(t->row_of, n / k, k, t->order);
  }
  return launched();
}

}  // namespace osmos

using namespace osmos;

extern "C" bool q4x_route(const float* logits, uint32_t n_tok, uint32_t n_exp, uint32_t k, int32_t* ids, float* w,
                          int32_t* rows, void* stream) {
  if (!logits || !ids || !w || !rows || !n_tok || !n_exp || n_exp > kMaxExperts || !k || k > kMaxK || k > n_exp)
    return false;
  const dim3 grid(blocks_for(n_tok, kRouteWarps)), block(kRouteWarps * kWarp);
  const cudaStream_t s = stream_of(stream);
  switch (route::regs_for(n_exp)) {
    case 4: return launch_dependent(route_kernel<4>, grid, block, 0, s, logits, n_tok, n_exp, k, ids, w, rows) == cudaSuccess;
    case 8: return launch_dependent(route_kernel<8>, grid, block, 0, s, logits, n_tok, n_exp, k, ids, w, rows) == cudaSuccess;
    case 16: return launch_dependent(route_kernel<16>, grid, block, 0, s, logits, n_tok, n_exp, k, ids, w, rows) == cudaSuccess;
    default: return launch_dependent(route_kernel<32>, grid, block, 0, s, logits, n_tok, n_exp, k, ids, w, rows) == cudaSuccess;
  }
}

extern "C" void q4x_expert_bounds(uint32_t n, uint32_t n_exp, Q4xExpertBounds* b) {
  // a run r holds the entries of 2^r tiles: an expert gives one entry to the run of its last part (at most one an
  // expert, and it needs more than 16 * 2^(r-1) tokens), and all its full 128-token parts to the last run
  const uint32_t most = n < n_exp ? n : n_exp;
  uint32_t at = 0;
  for (uint32_t r = 0; r < Q4X_TILE_RUNS; r++) {
    const uint32_t need = r ? (MM_TILE << (r - 1)) + 1u : 1u;  // the fewest tokens of an entry of this run
    uint32_t cap = n / need < most ? n / need : most;
    if (r == Q4X_TILE_RUNS - 1) cap = n / need;  // (full parts: not bounded by the experts)
    b->first[r] = at, b->count[r] = cap, at += cap;
  }
  b->entries = at;
  b->slots = n + (MM_TILE - 1) * most;
}

extern "C" bool q4x_expert_tiles(const int32_t* ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t dim, uint32_t ff,
                                 const Q4xExpertTiles* t, void* stream) {
  if (!ids || !n || !k || n % k || !n_exp || n_exp > kMaxExperts || !dim || !ff || !t || !t->cnt || !t->gidx ||
      !t->hidx || !t->xg || !t->yg || !t->xd || !t->yd || !t->where || !t->off)
    return false;
  for (int j = 0; j < Q4X_GROUP_TENSORS; j++)
    if ((!t->tab[j] && (!t->base[j] || !t->bytes[j])) || !t->ptr[j]) return false;
  Q4xExpertBounds bd;
  q4x_expert_bounds(n, n_exp, &bd);
  tiles_kernel<<<1, kTableThreads, 0, stream_of(stream)>>>(ids, n, k, n_exp, dim, ff, *t, bd);
  if (!launched()) return false;
  if (n > kInlinePicks) place_kernel<<<n_exp, kThreads, 0, stream_of(stream)>>>(ids, n, k, n_exp, *t);
  return launched();
}

// ---- q4x_expert_tiles without caller scratch ----------------------------------------------------------------------
// The tables' scratch (an expert's first place, first slot and count) in a fixed device array of this library, for
// callers that must not allocate: see include/osmos_b200/moe.h. One array a device that loads the library, held until
// the process exits; every call on a device shares it.
constexpr uint32_t kStaticTilesExperts = 1024;  // the most experts the fixed scratch holds (12 KB)
static __device__ __align__(256) int32_t g_tiles_scratch[3 * kStaticTilesExperts];
constexpr int kStaticTilesDevices = 64;
static int32_t* g_tiles_scratch_at[kStaticTilesDevices];  // the array's device address, per device, once looked up

extern "C" bool q4x_expert_tiles_static(const int32_t* ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t dim,
                                        uint32_t ff, const Q4xExpertTiles* t, void* stream) {
  if (!t || !n_exp || n_exp > kStaticTilesExperts) return false;  // past the fixed scratch: refused, nothing queued
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kStaticTilesDevices) return false;
  if (!g_tiles_scratch_at[device]) {
    // host code cannot use the array's name as an address: ask the runtime where it lives on the current device
    void* at = nullptr;
    if (cudaGetSymbolAddress(&at, g_tiles_scratch) != cudaSuccess || !at) return false;
    g_tiles_scratch_at[device] = (int32_t*) at;
  }
  Q4xExpertTiles with_scratch = *t;
  with_scratch.off = g_tiles_scratch_at[device];
  return q4x_expert_tiles(ids, n, k, n_exp, dim, ff, &with_scratch, stream);
}

extern "C" bool q4x_swiglu(const float* g, const float* u, uint64_t n, float* y, const Q4xX16* side, void* stream) {
  if (!g || !u || !y || !n) return false;
  const Q4xX16 s = side ? *side : Q4xX16{nullptr, nullptr, 1, 0};
  if (n % 4 == 0 && ((uintptr_t) g | (uintptr_t) u | (uintptr_t) y) % 16 == 0)
    swiglu_kernel<4><<<blocks_for(n / 4, kThreads), kThreads, 0, stream_of(stream)>>>(g, u, n, y, s);
  else
    swiglu_kernel<1><<<blocks_for(n, kThreads), kThreads, 0, stream_of(stream)>>>(g, u, n, y, s);
  return launched();
}

extern "C" bool q4x_swiglu_rows(const float* g, const float* u, uint32_t ff, const int32_t* idx, uint32_t slots, void* x16,
                                int32_t* overflow, void* stream) {
  if (!g || !u || !idx || !x16 || !overflow || !slots || !ff || ff % MM_TILE || ((uintptr_t) x16 & 15u)) return false;
  const uint64_t work = (uint64_t) slots * (ff / 8);
  swiglu_rows_kernel<<<blocks_for(work, kThreads), kThreads, 0, stream_of(stream)>>>(g, u, ff, idx, slots, (__half*) x16, overflow);
  return launched();
}

extern "C" bool q4x_moe_sum(const float* y, const int32_t* where, const float* w, uint32_t n_tok, uint32_t k,
                            uint32_t dim, const float* shared, const float* shared_logit, float* out, void* stream) {
  if (!y || !where || !w || !shared || !shared_logit || !out || !n_tok || !k || !dim) return false;
  const uint64_t total = (uint64_t) n_tok * dim;
  const bool vec = dim % 4 == 0 && ((uintptr_t) y | (uintptr_t) shared | (uintptr_t) out) % 16 == 0;
  if (vec)
    moe_sum_kernel<4><<<blocks_for(total / 4, kThreads), kThreads, 0, stream_of(stream)>>>(y, where, w, total, k, dim,
                                                                                         shared, shared_logit, out);
  else
    moe_sum_kernel<1><<<blocks_for(total, kThreads), kThreads, 0, stream_of(stream)>>>(y, where, w, total, k, dim, shared,
                                                                                     shared_logit, out);
  return launched();
}

extern "C" uint32_t lane_max_entries(uint32_t n, uint32_t n_exp) {
  // every expert with a pick has at most one entry that is not full
  const uint32_t most = n < n_exp ? n : n_exp;
  return n / LANE_MAX_TOKENS + most;
}

extern "C" bool lane_tables(const int32_t* ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t expert0,
                            uint32_t expert1, const LaneExperts* ex, const LaneTables* t, void* stream) {
  return lane_tables_launch(ids, n, k, n_exp, expert0, expert1, ex, t, LaneTablesSync{}, LaneRowHomes{}, stream_of(stream));
}
