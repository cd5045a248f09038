// what the expert-parallel step (ep.cu) asks of the int8 lane (q8.cu): the grouped entry points on the warp-ring /
// thread-a-row kernels only, with the step's extras (lane_ep.h) - inputs by step parity, rows stored through a table of
// addresses, the flags released after the last store. dry: only say whether a kernel takes the type and shape.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "lane_ep.h"

namespace osmos {

bool q8_gate_up_ep(uint32_t type, const void* const* wg, const void* const* wu, const int32_t* cnt, const int32_t* xrow,
                   const int32_t* xin, const int32_t* win, uint32_t n, uint32_t max_cnt, uint32_t rows, uint32_t cols,
                   const int8_t* q, const float* d, const float* scale, float lim, float* h, uint32_t hs, const LaneEp& ep,
                   bool dry, cudaStream_t s);
bool q8_group_tok_ep(uint32_t type, const void* const* w, const int32_t* cnt, const int32_t* xrow, const int32_t* xin,
                     uint32_t n, uint32_t max_cnt, uint32_t rows, uint32_t cols, const int8_t* q, const float* d, float* y,
                     uint32_t ys, const LaneEp& ep, bool dry, cudaStream_t s);
}  // namespace osmos
