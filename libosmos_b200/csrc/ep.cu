// Expert-parallel glue kernels (include/osmos_b200/ep.h): unpack of the gathered dispatch segments, the scatter of
// computed rows into the combine's send buffer, and the ordered per-token combine. Plain copies and a fixed-order sum:
// the bits are those of the single-GPU layer.
#include <cstring>

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

}  // namespace
}  // namespace osmos

using namespace osmos;

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
