// Routing, expert tables, activation and combine of an MoE layer (include/osmos_b200/moe.h), and the device-built
// tables of the int8 lane (include/osmos_b200/lane.h). Everything here is built on the GPU: no host round trip
// between the router and the experts.
#include "decode.cuh"
#include "osmos_b200/lane.h"
#include "osmos_b200/moe.h"
#include "topk.cuh"

namespace osmos {
namespace {

constexpr int kThreads = 256;
constexpr uint32_t kMaxExperts = 1024, kMaxK = 32;
constexpr float kSumFloor = 6.103515625e-5f;  // 2^-14: the floor under the picked probabilities' sum

// a block's reductions by one fixed tree (thread i's partial first, then halving strides): every thread gets the
// result, and the result depends on nothing but the inputs' places
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
  scratch[threadIdx.x] = v;
  __syncthreads();
  for (int s = kThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s)
      scratch[threadIdx.x] = MAX ? fmaxf(scratch[threadIdx.x], scratch[threadIdx.x + s])
                                 : __fadd_rn(scratch[threadIdx.x], scratch[threadIdx.x + s]);
    __syncthreads();
  }
  const float r = scratch[0];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(kThreads) route_kernel(const float* __restrict__ logits, uint32_t n_exp, uint32_t k,
                                                         int32_t* __restrict__ ids, float* __restrict__ w,
                                                         int32_t* __restrict__ rows) {
  __shared__ float p[kMaxExperts], scratch[kThreads];
  pdl_wait();  // (a dependent launch: the step before may still be reading the ids and weights this one writes)
  pdl_launch_next();
  const uint32_t t = blockIdx.x;
  const float* l = logits + (uint64_t) t * n_exp;
  float m = __int_as_float(0xFF800000);
  for (uint32_t i = threadIdx.x; i < n_exp; i += kThreads) m = fmaxf(m, l[i]);
  m = block_reduce<true>(m, scratch);
  float sum = 0.0f;
  for (uint32_t i = threadIdx.x; i < n_exp; i += kThreads) {
    p[i] = expf(__fsub_rn(l[i], m));
    sum = __fadd_rn(sum, p[i]);
  }
  const float inv = __fdiv_rn(1.0f, block_reduce<false>(sum, scratch));
  for (uint32_t i = threadIdx.x; i < n_exp; i += kThreads) p[i] = mul_rn(p[i], inv);
  __syncthreads();
  if (threadIdx.x >= kWarp) return;
  const uint32_t lane = threadIdx.x;
  constexpr int kMine = kMaxExperts / kWarp;
  float mine[kMine];
#pragma unroll
  for (int r = 0; r < kMine; r++) mine[r] = lane + 32u * r < n_exp ? order_key(p[lane + 32u * r]) : 0.0f;
  uint32_t taken = 0;
  float pick[kMaxK], total = 0.0f;
  for (uint32_t j = 0; j < k; j++) {
    float best;
    const int e = warp_pick<kMine>(mine, n_exp, taken, best);
    pick[j] = best, total = __fadd_rn(total, best);
    if (!lane) ids[t * k + j] = e, rows[t * k + j] = (int32_t) t;
  }
  if (lane) return;
  const float div = fmaxf(total, kSumFloor);
  for (uint32_t j = 0; j < k; j++) w[t * k + j] = __fdiv_rn(pick[j], div);
}

// ---- per-expert tables -----------------------------------------------------------------------------------------
constexpr int kTableThreads = 1024;  // a thread an expert
constexpr int kPart = MM_TILE << (Q4X_TILE_RUNS - 1);  // an entry's most tokens (128)
constexpr uint32_t kInlinePicks = 1024;  // up to this many picks are placed by the table kernel itself

__device__ __forceinline__ int run_of(int c) { return c <= 16 ? 0 : c <= 32 ? 1 : c <= 64 ? 2 : 3; }

// exclusive prefix sums over the block's kTableThreads values (thread i's value v): returns the sum of the values
// of the threads before i; *total the sum of all. integers: any order gives the same result
__device__ __forceinline__ int block_exclusive(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x % kWarp, wid = threadIdx.x / kWarp;
  int inc = v;
#pragma unroll
  for (int o = 1; o < kWarp; o <<= 1) {
    const int up = __shfl_up_sync(0xFFFFFFFFu, inc, o, kWarp);
    if (lane >= o) inc += up;
  }
  __syncthreads();  // the scratch free of its last use
  if (lane == kWarp - 1) warp_sums[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    int s = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < kWarp; o <<= 1) {
      const int up = __shfl_up_sync(0xFFFFFFFFu, s, o, kWarp);
      if (lane >= o) s += up;
    }
    warp_sums[lane] = s;
  }
  __syncthreads();
  *total = warp_sums[kWarp - 1];
  return inc - v + (wid ? warp_sums[wid - 1] : 0);
}

// pick i's rank among the picks of its own expert before it (the stable sort's order), for few picks: every thread
// walks the picks before its own in shared memory
__device__ __forceinline__ int rank_inline(const int32_t* sids, uint32_t i) {
  const int32_t e = sids[i];
  int r = 0;
  for (uint32_t j = 0; j < i; j++) r += sids[j] == e;
  return r;
}

__global__ void __launch_bounds__(kTableThreads) tiles_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t k,
                                                              uint32_t n_exp, uint32_t dim, uint32_t ff,
                                                              const Q4xExpertTiles t, const Q4xExpertBounds bd) {
  __shared__ int count[kMaxExperts], first_place[kMaxExperts], first_slot[kMaxExperts], warp_sums[kWarp];
  __shared__ int32_t sids[kInlinePicks];
  pdl_wait();  // (a dependent launch: ids are the router's output)
  pdl_launch_next();
  const uint32_t e = threadIdx.x;
  count[e] = 0;
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = ids[i];
    atomicAdd(&count[id], 1);
    if (n <= kInlinePicks) sids[i] = id;
  }
  __syncthreads();
  const int c = e < n_exp ? count[e] : 0;
  const int slots = (c + MM_TILE - 1) / MM_TILE * MM_TILE, rem = c % kPart;
  int live_slots, dummy, live_run[Q4X_TILE_RUNS], at[Q4X_TILE_RUNS];
  const int p0 = block_exclusive(c, warp_sums, &dummy);
  const int s0 = block_exclusive(slots, warp_sums, &live_slots);
#pragma unroll
  for (int r = 0; r < Q4X_TILE_RUNS; r++) {
    const int mine = (r == Q4X_TILE_RUNS - 1 ? c / kPart : 0) + (rem && run_of(rem) == r);
    at[r] = (int) bd.first[r] + block_exclusive(mine, warp_sums, &live_run[r]);
  }
  first_place[e] = p0, first_slot[e] = s0;
  if (e < n_exp) {
    t.off[e] = p0, t.off[n_exp + e] = s0, t.off[2 * n_exp + e] = c;
    for (int s = s0 + c; s < s0 + slots; s++) t.gidx[s] = -1, t.hidx[s] = -1;
    for (int part = 0; part * kPart < c; part++) {
      const int m = c - part * kPart < kPart ? c - part * kPart : kPart, en = at[run_of(m)]++;
      const int slot = s0 + part * kPart, place = p0 + part * kPart;
      t.cnt[en] = m;
      t.xg[en] = (uint32_t) slot * dim, t.xd[en] = (uint32_t) slot * ff;
      t.yg[en] = (uint32_t) place * ff, t.yd[en] = (uint32_t) place * dim;
#pragma unroll
      for (int j = 0; j < Q4X_GROUP_TENSORS; j++)
        t.ptr[j][en] = t.tab[j] ? t.tab[j][e] : (const uint8_t*) t.base[j] + (uint64_t) e * t.bytes[j];
    }
  }
  // the tables' tails, launched to their bounds: entries of no tokens, slots of no token
#pragma unroll
  for (int r = 0; r < Q4X_TILE_RUNS; r++)
    for (uint32_t i = (uint32_t) live_run[r] + threadIdx.x; i < bd.count[r]; i += kTableThreads) t.cnt[bd.first[r] + i] = 0;
  for (uint32_t s = (uint32_t) live_slots + threadIdx.x; s < bd.slots; s += kTableThreads) t.gidx[s] = -1, t.hidx[s] = -1;
  if (n > kInlinePicks) return;  // place_kernel's
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = sids[i];
    const int q = first_place[id] + rank_inline(sids, i), s = first_slot[id] + q - first_place[id];
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
__device__ __forceinline__ void order_token(const int32_t* row_of, uint32_t t, uint32_t k, int32_t* order) {
  int32_t r[kMaxK];
  for (uint32_t j = 0; j < k; j++) r[j] = row_of[t * k + j];
  for (uint32_t a = 1; a < k; a++)
    for (uint32_t c = a; c > 0 && (uint32_t) r[c] < (uint32_t) r[c - 1]; c--) {
      const int32_t s = r[c];
      r[c] = r[c - 1], r[c - 1] = s;
    }
  for (uint32_t j = 0; j < k; j++) order[t * k + j] = r[j];
}

__global__ void __launch_bounds__(kTableThreads) lane_tables_kernel(const int32_t* __restrict__ ids, uint32_t n,
                                                                    uint32_t k, uint32_t n_exp, const LaneExperts ex,
                                                                    const LaneTables t, uint32_t e0, uint32_t e1) {
  __shared__ int count[kMaxExperts], first_row[kMaxExperts], warp_sums[kWarp];
  __shared__ int32_t sids[kInlinePicks];
  pdl_wait();  // (a dependent launch: ids are the router's output)
  pdl_launch_next();
  const uint32_t e = threadIdx.x;
  count[e] = 0;
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = ids[i];
    const bool own = (uint32_t) id >= e0 && (uint32_t) id < e1;  // experts outside [e0, e1) are another rank's
    if (own) atomicAdd(&count[id], 1);
    if (n <= kInlinePicks) sids[i] = own ? id : -1;
  }
  __syncthreads();
  const int c = e < n_exp ? count[e] : 0;
  const int ents = (c + LANE_MAX_TOKENS - 1) / LANE_MAX_TOKENS;
  int rows, live;
  const int r0 = block_exclusive(c, warp_sums, &rows);
  const int en0 = block_exclusive(ents, warp_sums, &live);
  first_row[e] = r0;
  if (e < n_exp) {
    t.off[e] = r0, t.off[n_exp + e] = c;
    for (int part = 0; part < ents; part++) {
      const int en = en0 + part;
      t.cnt[en] = c - part * LANE_MAX_TOKENS < LANE_MAX_TOKENS ? c - part * LANE_MAX_TOKENS : LANE_MAX_TOKENS;
      t.xrow[en] = r0 + part * LANE_MAX_TOKENS;
#pragma unroll
      for (int j = 0; j < 3; j++)
        t.w[j][en] = ex.tab[j] ? ex.tab[j][e] : (const uint8_t*) ex.base[j] + (uint64_t) e * ex.bytes[j];
    }
  }
  for (uint32_t i = (uint32_t) live + threadIdx.x; i < t.max_entries; i += kTableThreads) t.cnt[i] = 0;
  if (threadIdx.x == 0) t.counts[0] = live, t.counts[1] = rows;
  if (n > kInlinePicks) return;  // lane_place_kernel's
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < n; i += kTableThreads) {
    const int32_t id = sids[i];
    if (id < 0) {
      t.row_of[i] = -1;
      continue;
    }
    const int r = first_row[id] + rank_inline(sids, i);
    t.tok[r] = (int32_t) (i / k), t.pair[r] = (int32_t) i, t.row_of[i] = r;
  }
  // each token's rows in order, in the same launch (the block's own writes, after its barrier)
  __syncthreads();
  for (uint32_t tk = threadIdx.x; tk < n / k; tk += kTableThreads) order_token(t.row_of, tk, k, t.order);
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

// a token's rows in ascending expert id (rows ascend with the expert, so ascending row): its k picks' rows sorted,
// the picks without a row here (-1) last
__global__ void lane_order_kernel(const int32_t* __restrict__ row_of, uint32_t n_tok, uint32_t k,
                                  int32_t* __restrict__ order) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tok) return;
  order_token(row_of, t, k, order);
}

// ---- activation and combine ------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float siluf(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }

__device__ __forceinline__ void x16_put(const Q4xX16& side, uint64_t i, float v) {
  if (!side.x16) return;
  const uint32_t t = side.row0 + (uint32_t) (i / side.cols), c = (uint32_t) (i % side.cols);
  if (!(fabsf(v) <= 65504.0f)) atomicOr(side.overflow, 1);
  ((__half*) side.x16)[(uint64_t) (t / 16) * 16 * side.cols + (c / 16) * 256 + (t % 16) * 16 + c % 16] = __float2half_rn(v);
}

__global__ void swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u, uint64_t n, float* __restrict__ y,
                              const Q4xX16 side) {
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  y[i] = mul_rn(siluf(g[i]), u[i]);
  x16_put(side, i, y[i]);
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
}  // namespace osmos

using namespace osmos;

extern "C" bool q4x_route(const float* logits, uint32_t n_tok, uint32_t n_exp, uint32_t k, int32_t* ids, float* w,
                          int32_t* rows, void* stream) {
  if (!logits || !ids || !w || !rows || !n_tok || !n_exp || n_exp > kMaxExperts || !k || k > kMaxK || k > n_exp)
    return false;
  return launch_dependent(route_kernel, dim3(n_tok), dim3(kThreads), 0, stream_of(stream), logits, n_exp, k, ids, w, rows) ==
         cudaSuccess;
}

extern "C" void q4x_expert_bounds(uint32_t n, uint32_t n_exp, Q4xExpertBounds* b) {
  const uint32_t most = n < n_exp ? n : n_exp;
  const uint32_t cap[Q4X_TILE_RUNS] = {most, n / 17 < most ? n / 17 : most, n / 33 < most ? n / 33 : most, n / 65};
  b->entries = 0;
  for (int r = 0; r < Q4X_TILE_RUNS; r++) b->first[r] = b->entries, b->count[r] = cap[r], b->entries += cap[r];
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
  swiglu_kernel<<<blocks_for(n, kThreads), kThreads, 0, stream_of(stream)>>>(g, u, n, y, s);
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
  if (!ids || !n || !k || n % k || k > kMaxK || !n_exp || n_exp > kMaxExperts || expert0 >= expert1 ||
      expert1 > n_exp || !ex || !t || !t->cnt || !t->xrow || !t->tok || !t->pair || !t->row_of || !t->order ||
      !t->off || !t->counts || t->max_entries < lane_max_entries(n, n_exp))
    return false;
  for (int j = 0; j < 3; j++)
    if ((!ex->tab[j] && (!ex->base[j] || !ex->bytes[j])) || !t->w[j]) return false;
  const cudaStream_t s = stream_of(stream);
  if (launch_dependent(lane_tables_kernel, dim3(1), dim3(kTableThreads), 0, s, ids, n, k, n_exp, *ex, *t, expert0, expert1) !=
      cudaSuccess)
    return false;
  if (n > kInlinePicks) {
    lane_place_kernel<<<n_exp, kThreads, 0, s>>>(ids, n, k, n_exp, *t, expert0, expert1);
    if (!launched()) return false;
  }
  if (n > kInlinePicks) lane_order_kernel<<<blocks_for(n / k, 128), 128, 0, s>>>(t->row_of, n / k, k, t->order);
  return launched();
}
