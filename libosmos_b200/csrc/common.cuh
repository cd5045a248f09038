// Shared host/device helpers for the sm_100a kernels behind the C ABI in include/osmos_b200/.
//
// Arithmetic rule for every kernel in this directory: the files are compiled with --fmad=false, so a product and a
// sum written separately are rounded separately; the only fused operations are explicit fmaf / __fmaf_rn calls.
// That is what makes a row's result a function of the row alone (the reference builds its kernels the same way:
// -ffp-contract=off, cuda.mk:18).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "osmos_b200/qtype.h"
#include "osmos_grids.h"

namespace osmos {

constexpr int kWarp = 32;

__host__ inline cudaStream_t stream_of(void* s) { return (cudaStream_t) s; }
// true when the launch just made was accepted (the entry points return this: "queued, not waited for")
__host__ inline bool launched() { return cudaGetLastError() == cudaSuccess; }
__host__ inline unsigned blocks_for(uint64_t work, unsigned per_block) {
  return (unsigned) ((work + per_block - 1) / per_block);
}

// A launch that may begin before the kernel ahead of it on the stream has finished (programmatic stream
// serialization): what such a kernel does before its `pdl_wait()` must not depend on that kernel's results - it is the
// place for barrier initialisation, codebook tables and the first weight copies (no kernel writes weights). After
// `pdl_wait()` the earlier kernel's writes are visible. `pdl_launch_next()` lets the kernel behind this one begin the
// same way. Both are no-ops in a kernel launched the ordinary way.
template <class... P, class... A>
__host__ inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                             A... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
// A kernel's dynamic shared-memory limit is an attribute of the kernel on ONE device: set it once per device. `done`
// is the caller's per-kernel record (a static array, one flag a device). false when the attribute was refused.
template <class K>
__host__ inline bool allow_dynamic_smem(K kernel, int bytes, bool (&done)[64]) {
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return false;
  if (done[d]) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  return done[d] = true;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// GGUF blocks are only 2-byte aligned in general (18, 34, 50, 66, 74, 82, 98 byte blocks; MXFP4's 17 is odd and is
// read by bytes): these readers never assume more.
__device__ __forceinline__ uint32_t ld8(const uint8_t* p) { return *p; }
__device__ __forceinline__ uint32_t ld16(const uint8_t* p) { return *(const uint16_t*) p; }
__device__ __forceinline__ uint32_t ld32(const uint8_t* p) { return ld16(p) | ld16(p + 2) << 16; }
__device__ __forceinline__ uint64_t ld64(const uint8_t* p) { return (uint64_t) ld32(p) | (uint64_t) ld32(p + 4) << 32; }
__device__ __forceinline__ float half_value(uint32_t bits) {
  return __half2float(__ushort_as_half((unsigned short) bits));
}
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }

// the fixed reduction every row sum ends with: lane l adds lane l ^ o for o = width / 2 .. 1 (a + b = b + a, so every
// lane of the group holds the same bits afterwards)
template <int WIDTH>
__device__ __forceinline__ float xor_tree(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, o, kWarp));
  return v;
}

// table row of a type (host side)
#define OSMOS_QTYPE_ROW(name, id, values, bytes, paths) {id, values, bytes, paths, #name},
static const OsmosQTypeInfo kQTypeRows[] = {OSMOS_QTYPE_TABLE(OSMOS_QTYPE_ROW)};
#undef OSMOS_QTYPE_ROW
__host__ inline const OsmosQTypeInfo* qtype_row(uint32_t id) {
  for (const OsmosQTypeInfo& r : kQTypeRows)
    if (r.id == id) return &r;
  return nullptr;
}

}  // namespace osmos
