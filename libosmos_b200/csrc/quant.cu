// quant_dequant / quant_dequant_f16 and the type table (include/osmos_b200/quant.h, qtype.h)
#include "decode.cuh"
#include "dispatch.cuh"
#include "osmos_b200/quant.h"

namespace osmos {
namespace {

constexpr int kThreads = 256;

// a thread a chunk of 8 values; the tables through shared memory
template <uint32_t T, bool HALF>
__global__ void __launch_bounds__(kThreads) dequant_kernel(const uint8_t* __restrict__ src, uint64_t chunks,
                                                           void* __restrict__ dst) {
  __shared__ __align__(16) uint8_t tables[grid_smem_bytes<T>() > 0 ? grid_smem_bytes<T>() : 16];
  const Grids g = stage_grids<T>(tables);
  for (uint64_t c = (uint64_t) blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (uint64_t) gridDim.x * kThreads) {
    float v[kChunk];
    decode8<T>(src + c / Fmt<T>::chunks * Fmt<T>::bytes, (int) (c % Fmt<T>::chunks), v, g);
    if constexpr (HALF) {
      __half* out = (__half*) dst + c * kChunk;
#pragma unroll
      for (int j = 0; j < kChunk; j++) out[j] = __float2half_rn(v[j]);
    } else {
      float4* out = (float4*) ((float*) dst + c * kChunk);
      out[0] = make_float4(v[0], v[1], v[2], v[3]), out[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
}

template <uint32_t T, bool HALF>
bool dequant(const void* src, uint64_t values, void* dst, cudaStream_t s) {
  if (!values || values % Fmt<T>::values) return false;
  const uint64_t chunks = values / kChunk;
  const uint64_t want = (chunks + kThreads - 1) / kThreads;
  dequant_kernel<T, HALF><<<(unsigned) (want < 148u * 16u ? want : 148u * 16u), kThreads, 0, s>>>((const uint8_t*) src,
                                                                                              chunks, dst);
  return launched();
}

}  // namespace
}  // namespace osmos

extern "C" const OsmosQTypeInfo* qtype_info(uint32_t id) { return osmos::qtype_row(id); }

extern "C" uint64_t qtype_tensor_bytes(uint32_t id, uint64_t rows, uint64_t cols) {
  const OsmosQTypeInfo* t = osmos::qtype_row(id);
  if (!t || cols % t->values) return 0;
  return rows * (cols / t->values) * t->bytes;
}

extern "C" bool quant_known(uint32_t type) {
  const OsmosQTypeInfo* t = osmos::qtype_row(type);
  return t && (t->paths & QTYPE_PATH_DECODE);
}

extern "C" bool quant_dequant(uint32_t type, const void* src, uint64_t values, float* dst, void* stream) {
  if (!src || !dst) return false;
#define CASE(T) return osmos::dequant<T, false>(src, values, dst, osmos::stream_of(stream));
  OSMOS_SWITCH_WEIGHTS(type, CASE, return false)
#undef CASE
}

extern "C" bool quant_dequant_f16(uint32_t type, const void* src, uint64_t values, void* dst, void* stream) {
  if (!src || !dst) return false;
#define CASE(T) return osmos::dequant<T, true>(src, values, dst, osmos::stream_of(stream));
  OSMOS_SWITCH_WEIGHTS(type, CASE, return false)
#undef CASE
}
