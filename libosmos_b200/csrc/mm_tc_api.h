// what mm_fp4.cu asks of the f16 tensor-core product (mm_tc.cu)
#pragma once
#include <cstdint>

namespace osmos {
namespace mm_tc {

// whether a rows x cols matrix of `type` tiles for the kernel (rows in 16s, cols in 128s and whole blocks)
bool shape_ok(uint32_t type, uint32_t rows, uint32_t cols);
// y[t * ys + r] = scale * sum_c W[r, c] x16[t][c] over n <= MM_MAX_TOKENS tokens of a tiled x16 whose rows are cols
// long; true: queued on the stream, false: refused, nothing queued
bool run(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const void* x16, uint32_t n, float* y, uint32_t ys,
         float scale, void* stream);

}  // namespace mm_tc
}  // namespace osmos
