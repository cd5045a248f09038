// Expert-parallel glue kernels (include/osmos_b200/ep.h): unpack of the gathered dispatch segments, the scatter of
// computed rows into the combine's send buffer, and the ordered per-token combine. Plain copies and a fixed-order sum:
// the bits are those of the single-GPU layer.
#include <cstring>

#include "common.cuh"
#include "ep_sync.cuh"
#include "moe_api.h"
#include "osmos_b200/ep.h"
#include "osmos_b200/q8.h"
#include "q8_api.h"
#include "q8_round.cuh"
#include "route.cuh"

namespace osmos {
namespace {

constexpr int kThreads = 256;

__host__ __device__ inline uint64_t up16(uint64_t v) { return (v + 15u) & ~(uint64_t) 15u; }
__host__ __device__ inline EpSegment segment_of(uint32_t tokens, uint32_t k, uint32_t dim) {
  EpSegment s;
  s.ids = 0;
  s.weights = up16((uint64_t) tokens * k * 4);
  s.q = s.weights + up16((uint64_t) tokens * k * 4);
  s.d = s.q + up16((uint64_t) tokens * dim);
  s.bytes = s.d + up16((uint64_t) tokens * (dim / 32) * 4);
  return s;
}

// a thread a 4-byte word of one of the four token-major arrays
__global__ void unpack_kernel(const uint8_t* __restrict__ gathered, uint32_t n_ranks, uint32_t tokens, uint32_t k,
                              uint32_t dim, uint32_t* __restrict__ ids, uint32_t* __restrict__ weights,
                              uint32_t* __restrict__ q, uint32_t* __restrict__ d) {
  pdl_wait();  // (a dependent launch: what this kernel reads is the output of the kernels ahead)
  pdl_launch_next();
  const EpSegment s = segment_of(tokens, k, dim);
  const uint64_t w_ids = (uint64_t) tokens * k, w_q = (uint64_t) tokens * dim / 4, w_d = (uint64_t) tokens * (dim / 32);
  const uint64_t per_rank = 2 * w_ids + w_q + w_d;
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i >= per_rank * n_ranks) return;
  const uint64_t r = i / per_rank;
  uint64_t w = i % per_rank;
  const uint8_t* seg = gathered + r * s.bytes;
  if (w < w_ids) {
    ids[r * w_ids + w] = ((const uint32_t*) (seg + s.ids))[w];
    return;
  }
  w -= w_ids;
  if (w < w_ids) {
    weights[r * w_ids + w] = ((const uint32_t*) (seg + s.weights))[w];
    return;
  }
  w -= w_ids;
  if (w < w_q) {
    q[r * w_q + w] = ((const uint32_t*) (seg + s.q))[w];
    return;
  }
  w -= w_q;
  d[r * w_d + w] = ((const uint32_t*) (seg + s.d))[w];
}

__global__ void scatter_rows_kernel(const float4* __restrict__ ye, const int32_t* __restrict__ row_of, uint32_t n_picks,
                                    uint32_t k, uint32_t tokens, uint32_t dim4, float4* __restrict__ send) {
  pdl_wait();  // (a dependent launch: what this kernel reads is the output of the kernels ahead)
  pdl_launch_next();
  const uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x;
  if (i >= (uint64_t) n_picks * dim4) return;
  const uint32_t pick = (uint32_t) (i / dim4), c = (uint32_t) (i % dim4);
  const int32_t row = row_of[pick];
  if (row < 0) return;
  const uint32_t t = pick / k, j = pick % k;
  const uint64_t slot = (uint64_t) (t / tokens) * tokens * k + (uint64_t) (t % tokens) * k + j;
  send[slot * dim4 + c] = ye[(uint64_t) row * dim4 + c];
}

// a block a home token: its picks ordered by expert id (k is small: an insertion sort by one thread), then every
// thread its columns, the rows added in that order from 0
__global__ void __launch_bounds__(kThreads) combine_kernel(const float* __restrict__ recv, const int32_t* __restrict__ ids,
                                                           uint32_t tokens, uint32_t k, uint32_t experts_per_rank,
                                                           uint32_t dim, const float* __restrict__ add,
                                                           float* __restrict__ out) {
  pdl_wait();  // (a dependent launch: what this kernel reads is the output of the kernels ahead)
  pdl_launch_next();
  __shared__ uint32_t slot[32];
  const uint32_t t = blockIdx.x;
  if (threadIdx.x == 0) {
    int32_t e[32];
    uint32_t j_of[32];
    for (uint32_t j = 0; j < k; j++) e[j] = ids[t * k + j], j_of[j] = j;
    for (uint32_t a = 1; a < k; a++)
      for (uint32_t c = a; c > 0 && e[c] < e[c - 1]; c--) {
        const int32_t se = e[c];
        const uint32_t sj = j_of[c];
        e[c] = e[c - 1], e[c - 1] = se, j_of[c] = j_of[c - 1], j_of[c - 1] = sj;
      }
    for (uint32_t j = 0; j < k; j++)
      slot[j] = ((uint32_t) e[j] / experts_per_rank) * tokens * k + t * k + j_of[j];
  }
  __syncthreads();
  for (uint32_t c = threadIdx.x; c < dim; c += kThreads) {
    float s = 0.0f;
    for (uint32_t j = 0; j < k; j++) s = __fadd_rn(s, recv[(uint64_t) slot[j] * dim + c]);
    out[(uint64_t) t * dim + c] = add ? __fadd_rn(s, add[(uint64_t) t * dim + c]) : s;
  }
}

// ---- the peer transport -----------------------------------------------------------------------------------------
__device__ uint32_t g_peer_wait_status;
constexpr uint64_t kPeerWaitNs = 2000ull * 1000 * 1000;

// The flags after the data: every thread fences its stores at system scope, the block counts itself in, and the block
// that finds all the others counted stores the flags (release, system scope) and zeroes the counter for the next use.
__device__ __forceinline__ void publish(uint32_t* const* flag, uint32_t n_ranks, uint32_t step, uint32_t* counter) {
  __shared__ bool last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(counter, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence_system();
  if (threadIdx.x < n_ranks)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag[threadIdx.x]), "r"(step) : "memory");
  if (threadIdx.x == 0) *counter = 0;
}

__global__ void __launch_bounds__(kThreads) push_kernel(const uint4* __restrict__ src, uint64_t n16, uint4* const* dst,
                                                        uint32_t* const* flag, uint32_t n_ranks, uint32_t step,
                                                        uint32_t* counter) {
  pdl_wait();  // (a dependent launch: what this kernel reads is the output of the kernels ahead)
  pdl_launch_next();
  for (uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x; i < n16; i += (uint64_t) gridDim.x * kThreads) {
    const uint4 v = src[i];
    for (uint32_t r = 0; r < n_ranks; r++) dst[r][i] = v;
  }
  publish(flag, n_ranks, step, counter);
}

__global__ void __launch_bounds__(kThreads) scatter_rows_peer_kernel(const float4* __restrict__ ye,
                                                                     const int32_t* __restrict__ row_of, uint32_t n_picks,
                                                                     uint32_t k, uint32_t tokens, uint32_t dim4,
                                                                     float4* const* recv, uint32_t* const* flag,
                                                                     uint32_t n_ranks, uint32_t step, uint32_t* counter) {
  pdl_wait();  // (a dependent launch: what this kernel reads is the output of the kernels ahead)
  pdl_launch_next();
  const uint64_t total = (uint64_t) n_picks * dim4;
  for (uint64_t i = (uint64_t) blockIdx.x * kThreads + threadIdx.x; i < total; i += (uint64_t) gridDim.x * kThreads) {
    const uint32_t pick = (uint32_t) (i / dim4), c = (uint32_t) (i % dim4);
    const int32_t row = row_of[pick];
    if (row < 0) continue;
    const uint32_t t = pick / k, j = pick % k;
    recv[t / tokens][((uint64_t) (t % tokens) * k + j) * dim4 + c] = ye[(uint64_t) row * dim4 + c];
  }
  publish(flag, n_ranks, step, counter);
}

// thread r polls the flag rank r writes (this GPU's own memory), napping between looks, until it has reached `step`
__global__ void peer_wait_kernel(const uint32_t* flags, uint32_t n_ranks, uint32_t step) {
  pdl_wait();  // (a dependent launch: what this kernel reads is the output of the kernels ahead)
  pdl_launch_next();
  if (threadIdx.x >= n_ranks) return;
  const uint32_t* f = flags + threadIdx.x;
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int32_t) (v - step) >= 0) return;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 > kPeerWaitNs) {
      atomicOr(&g_peer_wait_status, 1u);
      return;
    }
    __nanosleep(100);
  }
}

// ---- the fused step --------------------------------------------------------------------------------------------------
__host__ __device__ inline uint64_t up256(uint64_t v) { return (v + 255u) & ~(uint64_t) 255u; }

struct StepArgs {
  EpPeers peers;
  EpLayout lay;
  uint32_t rank, n_ranks, tokens, k, dim, n_exp;
  uint32_t* sync;  // [0] step, [1] [2] publish counters
  const float* bias;  // the scored routers'
  float rscale;
};

// A block a home token. Its last warp routes it (route.cuh) while the eight before it round its row to int8
// (q8_round.cuh); every result goes straight to its token-major place in every rank's buffer. The last block to finish
// releases this rank's dispatch flag everywhere and advances the step counter.
constexpr int kRoundWarps = 8, kStepThreads = (kRoundWarps + 1) * kWarp;
template <int R, int ROUTER>
__global__ void __launch_bounds__(kStepThreads) route_round_push_kernel(const StepArgs a, const float* __restrict__ x,
                                                                        const float* __restrict__ logits) {
  pdl_wait();  // (a dependent launch: the step before may still be reading what this one writes)
  pdl_launch_next();
  const uint32_t step = a.sync[0] + 1u, half = step & 1u;
  const uint32_t tl = blockIdx.x, t = a.rank * a.tokens + tl, lane = threadIdx.x % kWarp;
  if (threadIdx.x >= kRoundWarps * kWarp) {
    route::Pick p;
    if constexpr (ROUTER == EP_ROUTER_SOFTMAX) p = route::softmax_topk<R>(logits + (uint64_t) tl * a.n_exp, a.n_exp, a.k, lane);
    else if constexpr (ROUTER == EP_ROUTER_SIGMOID)
      p = route::scored_topk<R, route::kSigmoid>(logits + (uint64_t) tl * a.n_exp, a.bias, a.n_exp, a.k, a.rscale, lane);
    else p = route::scored_topk<R, route::kSqrtSoftplus>(logits + (uint64_t) tl * a.n_exp, a.bias, a.n_exp, a.k, a.rscale, lane);
    if (lane < a.k)
      for (uint32_t r = 0; r < a.n_ranks; r++) {
        ((int32_t*) (a.peers.base[r] + a.lay.ids[half]))[t * a.k + lane] = (int32_t) p.id;
        ((float*) (a.peers.base[r] + a.lay.weights[half]))[t * a.k + lane] = p.w;
      }
  } else {
    const uint32_t per = a.dim / 8;
    for (uint32_t c0 = 0; c0 < per; c0 += kRoundWarps * kWarp) {  // (whole warps: per is a multiple of 4)
      const uint32_t c = c0 + threadIdx.x;
      const bool live = c < per;
      float v[8], scale;
      load8(x + (uint64_t) tl * a.dim + (uint64_t) (live ? c : 0) * 8, v);
      const uint2 codes = round_block8<false>(v, &scale);
      if (!live) continue;
      for (uint32_t r = 0; r < a.n_ranks; r++) {
        *(uint2*) (a.peers.base[r] + a.lay.q[half] + (uint64_t) t * a.dim + (uint64_t) c * 8) = codes;
        if (c % 4 == 0) ((float*) (a.peers.base[r] + a.lay.d[half]))[(uint64_t) t * (a.dim / 32) + c / 4] = scale;
      }
    }
  }
  publish_step(a.peers, a.lay.flags_dispatch, a.rank, a.n_ranks, step, a.sync + 1, a.sync);
}

// A block a home token: a bounded wait on every rank's combine flag, the token's picks ordered by expert id (k is
// small: one thread sorts by insertion), then every thread its columns, the rows added in that order from 0.
__global__ void __launch_bounds__(kThreads) combine_wait_kernel(const StepArgs a, const float* __restrict__ add,
                                                                float* __restrict__ out) {
  __shared__ uint32_t order[32];
  pdl_wait();  // (a dependent launch)
  pdl_launch_next();
  const uint32_t step = a.sync[0], half = step & 1u;
  uint8_t* mine = a.peers.base[a.rank];
  if (threadIdx.x < a.n_ranks && !flag_wait((const uint32_t*) (mine + a.lay.flags_combine) + threadIdx.x, step, a.n_ranks == 1))
    atomicOr(&g_peer_wait_status, 1u);
  const uint32_t tl = blockIdx.x, k = a.k;
  if (threadIdx.x < kWarp) {  // pick j's place in the sum: how many of the token's picks have a lower expert id
    const int32_t* ids = (const int32_t*) (mine + a.lay.ids[half]) + (uint64_t) (a.rank * a.tokens + tl) * k;
    const int32_t e = threadIdx.x < k ? ids[threadIdx.x] : 0x7FFFFFFF;
    uint32_t place = 0;
    for (uint32_t j = 0; j < k; j++) place += __shfl_sync(0xFFFFFFFFu, e, (int) j, kWarp) < e;
    if (threadIdx.x < k) order[place] = threadIdx.x;  // (a token picks an expert once: the places are distinct)
  }
  __syncthreads();
  const float4* recv = (const float4*) (mine + a.lay.recv[half]) + (uint64_t) tl * k * (a.dim / 4);
  for (uint32_t c = threadIdx.x; c < a.dim / 4; c += kThreads) {
    float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint32_t j = 0; j < k; j++) {
      const float4 v = recv[(uint64_t) order[j] * (a.dim / 4) + c];
      s.x = __fadd_rn(s.x, v.x), s.y = __fadd_rn(s.y, v.y), s.z = __fadd_rn(s.z, v.z), s.w = __fadd_rn(s.w, v.w);
    }
    if (add) {
      const float4 v = ((const float4*) add)[(uint64_t) tl * (a.dim / 4) + c];
      s.x = __fadd_rn(s.x, v.x), s.y = __fadd_rn(s.y, v.y), s.z = __fadd_rn(s.z, v.z), s.w = __fadd_rn(s.w, v.w);
    }
    ((float4*) out)[(uint64_t) tl * (a.dim / 4) + c] = s;
  }
}

StepArgs step_args(const EpPlan* p) {
  StepArgs a{};
  for (uint32_t r = 0; r < p->n_ranks; r++) a.peers.base[r] = (uint8_t*) p->peer[r];
  a.lay = p->lay, a.rank = p->rank, a.n_ranks = p->n_ranks, a.tokens = p->n_tok / p->n_ranks, a.k = p->layer.k;
  a.dim = p->layer.dim, a.n_exp = p->layer.n_exp, a.sync = p->sync, a.bias = p->route_bias, a.rscale = p->route_scale;
  return a;
}

// the lane kernels' extras for the step: inputs by parity out of this rank's own buffer
LaneEp lane_ep(const EpPlan* p, bool gathered_inputs, bool push) {
  LaneEp e{};
  e.step = p->sync;
  if (gathered_inputs)
    e.half_q = p->lay.q[1] - p->lay.q[0], e.half_d = p->lay.d[1] - p->lay.d[0];  // (the rows' scales: a table of the step's)
  if (push) {
    e.out_rows = p->rows, e.publish = true, e.flags_off = p->lay.flags_combine, e.rank = p->rank, e.n_ranks = p->n_ranks;
    e.counter = p->sync + 2;
    for (uint32_t r = 0; r < p->n_ranks; r++) e.peers.base[r] = (uint8_t*) p->peer[r];
  }
  return e;
}

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" bool ep_layout(uint32_t n_ranks, uint32_t n_tok, uint32_t k, uint32_t dim, EpLayout* l) {
  if (!l || !n_ranks || n_ranks > EP_MAX_RANKS || !n_tok || n_tok % n_ranks || !k || k > 32 || !dim || dim % 32) return false;
  const uint64_t picks = (uint64_t) n_tok * k, tokens = n_tok / n_ranks;
  uint64_t at = 0;
  l->flags_dispatch = at, at += 256;
  l->flags_combine = at, at += 256;
  for (int h = 0; h < 2; h++) {
    l->ids[h] = at, at += up256(picks * 4);
    l->weights[h] = at, at += up256(picks * 4);
    l->q[h] = at, at += up256((uint64_t) n_tok * dim);
    l->d[h] = at, at += up256((uint64_t) n_tok * (dim / 32) * 4);
  }
  for (int h = 0; h < 2; h++) l->recv[h] = at, at += up256(tokens * k * dim * 4);
  l->bytes = at;
  return true;
}

extern "C" bool ep_plan_ok(const EpPlan* p) {
  if (!p || !p->n_ranks || p->n_ranks > EP_MAX_RANKS || p->rank >= p->n_ranks || !p->n_tok || p->n_tok % p->n_ranks ||
      !p->sync || !p->rows || p->expert0 >= p->expert1 || p->expert1 > p->layer.n_exp)
    return false;
  const LaneLayer& l = p->layer;
  EpLayout want;
  if (!l.dim || l.dim % 256 || !l.ff || l.ff % 256 || !l.k || l.k > 32 || !l.n_exp || l.n_exp > 1024 || l.k > l.n_exp ||
      (uint64_t) p->n_tok * l.k > 1024 || !ep_layout(p->n_ranks, p->n_tok, l.k, l.dim, &want) ||
      memcmp(&want, &p->lay, sizeof want) != 0 || p->scratch.max_tok < p->n_tok || p->router > EP_ROUTER_SIGMOID ||
      (p->router != EP_ROUTER_SOFTMAX && (!p->route_bias || l.k > 16)))
    return false;
  for (uint32_t r = 0; r < p->n_ranks; r++)
    if (!p->peer[r] || ((uintptr_t) p->peer[r] & 255u)) return false;
  const uint32_t ents = p->scratch.tab.max_entries;
  return q8_gate_up_ep(l.type_gu, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, ents, LANE_MAX_TOKENS, l.ff, l.dim,
                       nullptr, nullptr, nullptr, l.lim, nullptr, l.ff, LaneEp{}, true, nullptr) &&
         q8_group_tok_ep(l.type_down, nullptr, nullptr, nullptr, nullptr, ents, LANE_MAX_TOKENS, l.dim, l.ff, nullptr, nullptr,
                         nullptr, l.dim, LaneEp{}, true, nullptr);
}

extern "C" bool ep_route_round_push(const EpPlan* p, const float* x, const float* logits, void* stream) {
  if (!p || !x || !logits) return false;
  const StepArgs a = step_args(p);
  const dim3 grid(a.tokens), block(kStepThreads);
  const cudaStream_t s = stream_of(stream);
#define ROUTE(R, KIND) launch_dependent(route_round_push_kernel<R, KIND>, grid, block, 0, s, a, x, logits) == cudaSuccess
#define BY_REGS(KIND)                     \
  switch (route::regs_for(a.n_exp)) {     \
    case 4: return ROUTE(4, KIND);        \
    case 8: return ROUTE(8, KIND);        \
    case 16: return ROUTE(16, KIND);      \
    default: return ROUTE(32, KIND);      \
  }
  if (p->router == EP_ROUTER_SOFTMAX) BY_REGS(EP_ROUTER_SOFTMAX)
  if (p->router == EP_ROUTER_SIGMOID) BY_REGS(EP_ROUTER_SIGMOID)
  BY_REGS(EP_ROUTER_SQRT_SOFTPLUS)
#undef BY_REGS
#undef ROUTE
}

extern "C" bool ep_lane_tables(const EpPlan* p, void* stream) {
  if (!p) return false;
  uint8_t* mine = (uint8_t*) p->peer[p->rank];
  LaneTablesSync sy;
  sy.flags = (const uint32_t*) (mine + p->lay.flags_dispatch), sy.step = p->sync, sy.n_ranks = p->n_ranks;
  sy.half_bytes = p->lay.ids[1] - p->lay.ids[0];
  sy.weights = (const float*) (mine + p->lay.weights[0]), sy.weights_half = p->lay.weights[1] - p->lay.weights[0];
  void* status = nullptr;
  if (cudaGetSymbolAddress(&status, g_peer_wait_status) != cudaSuccess) return false;
  sy.status = (uint32_t*) status;
  LaneRowHomes homes;
  homes.rows = p->rows, homes.scale = (float*) (p->rows + (uint64_t) p->n_tok * p->layer.k), homes.recv[0] = p->lay.recv[0], homes.recv[1] = p->lay.recv[1];
  homes.tokens = p->n_tok / p->n_ranks, homes.dim = p->layer.dim;
  for (uint32_t r = 0; r < p->n_ranks; r++) homes.base[r] = (uint8_t*) p->peer[r];
  return lane_tables_launch((const int32_t*) (mine + p->lay.ids[0]), p->n_tok * p->layer.k, p->layer.k, p->layer.n_exp,
                            p->expert0, p->expert1, &p->layer.experts, &p->scratch.tab, sy, homes, stream_of(stream));
}

extern "C" bool ep_gate_up(const EpPlan* p, void* stream) {
  if (!p) return false;
  const LaneLayer& l = p->layer;
  const LaneTables& t = p->scratch.tab;
  const uint8_t* mine = (const uint8_t*) p->peer[p->rank];
  // (a row's scale is its routed weight, laid out by row by the tables' kernel: no index between a row and its scale)
  return q8_gate_up_ep(l.type_gu, t.w[0], t.w[1], t.cnt, t.xrow, t.tok, nullptr, t.max_entries, LANE_MAX_TOKENS, l.ff, l.dim,
                       (const int8_t*) (mine + p->lay.q[0]), (const float*) (mine + p->lay.d[0]),
                       (const float*) (p->rows + (uint64_t) p->n_tok * l.k), l.lim, p->scratch.hh, l.ff,
                       lane_ep(p, true, false), false, stream_of(stream));
}

extern "C" bool ep_down_push(const EpPlan* p, void* stream) {
  if (!p) return false;
  const LaneLayer& l = p->layer;
  const LaneTables& t = p->scratch.tab;
  return q8_group_tok_ep(l.type_down, t.w[2], t.cnt, t.xrow, nullptr, t.max_entries, LANE_MAX_TOKENS, l.dim, l.ff,
                         p->scratch.hq, p->scratch.hqd, nullptr, l.dim, lane_ep(p, false, true), false, stream_of(stream));
}

extern "C" bool ep_combine_wait(const EpPlan* p, const float* add, float* out, void* stream) {
  if (!p || !out || (((uintptr_t) out | (uintptr_t) add) & 15u)) return false;
  const StepArgs a = step_args(p);
  return launch_dependent(combine_wait_kernel, dim3(a.tokens), dim3(kThreads), 0, stream_of(stream), a, add, out) == cudaSuccess;
}

extern "C" bool ep_last_picks(const EpPlan* p, int32_t* ids, float* weights) {
  if (!p || !ids || !weights || cudaDeviceSynchronize() != cudaSuccess) return false;
  uint32_t step = 0;
  if (cudaMemcpy(&step, p->sync, sizeof step, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
  const uint8_t* mine = (const uint8_t*) p->peer[p->rank];
  const uint64_t n = (uint64_t) (p->n_tok / p->n_ranks) * p->layer.k, first = (uint64_t) p->rank * n;
  return cudaMemcpy(ids, (const int32_t*) (mine + p->lay.ids[step & 1u]) + first, n * 4, cudaMemcpyDeviceToHost) == cudaSuccess &&
         cudaMemcpy(weights, (const float*) (mine + p->lay.weights[step & 1u]) + first, n * 4, cudaMemcpyDeviceToHost) == cudaSuccess;
}

extern "C" bool ep_peer_alloc(uint64_t bytes, void** ptr, uint8_t handle[EP_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == EP_HANDLE_BYTES, "a CUDA IPC handle is 64 bytes");
  if (!bytes || !ptr || !handle) return false;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return false;
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
      cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return false;
  }
  memcpy(handle, &h, sizeof h);
  *ptr = p;
  return true;
}

extern "C" bool ep_peer_open(const uint8_t handle[EP_HANDLE_BYTES], void** ptr) {
  if (!handle || !ptr) return false;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return false;
  *ptr = p;
  return true;
}

extern "C" bool ep_peer_close(void* ptr) { return ptr && cudaIpcCloseMemHandle(ptr) == cudaSuccess; }
extern "C" bool ep_peer_free(void* ptr) { return ptr && cudaFree(ptr) == cudaSuccess; }

extern "C" bool ep_push(const void* src, uint64_t bytes, void* const* dst, uint32_t* const* flag, uint32_t n_ranks,
                        uint32_t step, uint32_t* counter, void* stream) {
  if (!src || !bytes || bytes % 16 || !dst || !flag || !n_ranks || n_ranks > EP_MAX_RANKS || !counter || ((uintptr_t) src & 15u))
    return false;
  const uint64_t n16 = bytes / 16;
  const unsigned blocks = (unsigned) (n16 / kThreads < 1 ? 1 : (n16 / kThreads > 64 ? 64 : n16 / kThreads));
  return launch_dependent(push_kernel, dim3(blocks), dim3(kThreads), 0, stream_of(stream), (const uint4*) src, n16,
                          (uint4* const*) dst, flag, n_ranks, step, counter) == cudaSuccess;
}

extern "C" bool ep_wait(const uint32_t* flags, uint32_t n_ranks, uint32_t step, void* stream) {
  if (!flags || !n_ranks || n_ranks > EP_MAX_RANKS) return false;
  return launch_dependent(peer_wait_kernel, dim3(1), dim3(32), 0, stream_of(stream), flags, n_ranks, step) == cudaSuccess;
}

extern "C" uint32_t ep_wait_status(void) {
  uint32_t v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_peer_wait_status, sizeof v) != cudaSuccess) return 0x80000000u;
  cudaMemcpyToSymbol(g_peer_wait_status, &zero, sizeof zero);
  return v;
}

extern "C" bool ep_scatter_rows_peer(const float* ye, const int32_t* row_of, uint32_t n_picks, uint32_t k, uint32_t tokens,
                                     uint32_t dim, float* const* recv, uint32_t* const* flag, uint32_t n_ranks,
                                     uint32_t step, uint32_t* counter, void* stream) {
  if (!ye || !row_of || !recv || !flag || !counter || !n_picks || !k || !tokens || !dim || dim % 4 || !n_ranks ||
      n_ranks > EP_MAX_RANKS || ((uintptr_t) ye & 15u))
    return false;
  const uint64_t work = (uint64_t) n_picks * (dim / 4);
  const unsigned blocks = (unsigned) (work / kThreads < 1 ? 1 : (work / kThreads > 592 ? 592 : work / kThreads));
  return launch_dependent(scatter_rows_peer_kernel, dim3(blocks), dim3(kThreads), 0, stream_of(stream), (const float4*) ye,
                          row_of, n_picks, k, tokens, dim / 4, (float4* const*) recv, flag, n_ranks, step, counter) == cudaSuccess;
}

extern "C" void ep_segment(uint32_t tokens, uint32_t k, uint32_t dim, EpSegment* s) { *s = segment_of(tokens, k, dim); }

extern "C" bool ep_unpack(const void* gathered, uint32_t n_ranks, uint32_t tokens, uint32_t k, uint32_t dim, int32_t* ids,
                          float* weights, int8_t* q, float* d, void* stream) {
  if (!gathered || !ids || !weights || !q || !d || !n_ranks || !tokens || !k || !dim || dim % 32) return false;
  const uint64_t words = ((uint64_t) tokens * k * 2 + (uint64_t) tokens * dim / 4 + (uint64_t) tokens * (dim / 32)) * n_ranks;
  return launch_dependent(unpack_kernel, dim3(blocks_for(words, kThreads)), dim3(kThreads), 0, stream_of(stream),
                          (const uint8_t*) gathered, n_ranks, tokens, k, dim, (uint32_t*) ids, (uint32_t*) weights, (uint32_t*) q,
                          (uint32_t*) d) == cudaSuccess;
}

extern "C" bool ep_scatter_rows(const float* ye, const int32_t* row_of, uint32_t n_picks, uint32_t k, uint32_t tokens,
                                uint32_t dim, float* send, void* stream) {
  if (!ye || !row_of || !send || !n_picks || !k || !tokens || !dim || dim % 4 ||
      (((uintptr_t) ye | (uintptr_t) send) & 15u))
    return false;
  const uint64_t work = (uint64_t) n_picks * (dim / 4);
  return launch_dependent(scatter_rows_kernel, dim3(blocks_for(work, kThreads)), dim3(kThreads), 0, stream_of(stream),
                          (const float4*) ye, row_of, n_picks, k, tokens, dim / 4, (float4*) send) == cudaSuccess;
}

extern "C" bool ep_combine(const float* recv, const int32_t* ids, uint32_t tokens, uint32_t k, uint32_t experts_per_rank,
                           uint32_t dim, const float* add, float* out, void* stream) {
  if (!recv || !ids || !out || !tokens || !k || k > 32 || !experts_per_rank || !dim) return false;
  return launch_dependent(combine_kernel, dim3(tokens), dim3(kThreads), 0, stream_of(stream), recv, ids, tokens, k,
                          experts_per_rank, dim, add, out) == cudaSuccess;
}
