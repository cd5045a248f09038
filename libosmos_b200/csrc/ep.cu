// Expert-parallel glue kernels (include/osmos_b200/ep.h): unpack of the gathered dispatch segments, the scatter of
// computed rows into the combine's send buffer, and the ordered per-token combine. Plain copies and a fixed-order sum:
// the bits are those of the single-GPU layer.
#include "common.cuh"
#include "osmos_b200/ep.h"

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

}  // namespace
}  // namespace osmos

using namespace osmos;

extern "C" void ep_segment(uint32_t tokens, uint32_t k, uint32_t dim, EpSegment* s) { *s = segment_of(tokens, k, dim); }

extern "C" bool ep_unpack(const void* gathered, uint32_t n_ranks, uint32_t tokens, uint32_t k, uint32_t dim, int32_t* ids,
                          float* weights, int8_t* q, float* d, void* stream) {
  if (!gathered || !ids || !weights || !q || !d || !n_ranks || !tokens || !k || !dim || dim % 32) return false;
  const uint64_t words = ((uint64_t) tokens * k * 2 + (uint64_t) tokens * dim / 4 + (uint64_t) tokens * (dim / 32)) * n_ranks;
  unpack_kernel<<<blocks_for(words, kThreads), kThreads, 0, stream_of(stream)>>>(
      (const uint8_t*) gathered, n_ranks, tokens, k, dim, (uint32_t*) ids, (uint32_t*) weights, (uint32_t*) q, (uint32_t*) d);
  return launched();
}

extern "C" bool ep_scatter_rows(const float* ye, const int32_t* row_of, uint32_t n_picks, uint32_t k, uint32_t tokens,
                                uint32_t dim, float* send, void* stream) {
  if (!ye || !row_of || !send || !n_picks || !k || !tokens || !dim || dim % 4 ||
      (((uintptr_t) ye | (uintptr_t) send) & 15u))
    return false;
  const uint64_t work = (uint64_t) n_picks * (dim / 4);
  scatter_rows_kernel<<<blocks_for(work, kThreads), kThreads, 0, stream_of(stream)>>>((const float4*) ye, row_of, n_picks, k,
                                                                                   tokens, dim / 4, (float4*) send);
  return launched();
}

extern "C" bool ep_combine(const float* recv, const int32_t* ids, uint32_t tokens, uint32_t k, uint32_t experts_per_rank,
                           uint32_t dim, const float* add, float* out, void* stream) {
  if (!recv || !ids || !out || !tokens || !k || k > 32 || !experts_per_rank || !dim) return false;
  combine_kernel<<<tokens, kThreads, 0, stream_of(stream)>>>(recv, ids, tokens, k, experts_per_rank, dim, add, out);
  return launched();
}
