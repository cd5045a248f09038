// what mmq.cu asks of the tensor-core Q4_K x int8 kernel (mmq_tc.cu)
#pragma once
#include <cstdint>

namespace osmos {
namespace mmq_tc {

// 1: queued on the stream; 0: not a shape this kernel takes (rows in 128s, cols in 256s, 16-byte aligned activations):
// nothing queued, use the generic kernel; -1: the launch was refused
int try_launch(const void* const* w, const int32_t* cnt, uint32_t n_mat, uint32_t max_cnt, uint32_t rows, uint32_t cols,
               const int8_t* x8, const float* dx, const float* sx, const uint32_t* soff, float* y, const uint32_t* yoff,
               uint32_t ys, void* stream);
// the current device's status word, read and cleared (synchronizes): bit 0 a bounded wait ran out
uint32_t read_status();

}  // namespace mmq_tc
}  // namespace osmos
