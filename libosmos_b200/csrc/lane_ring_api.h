// what q8.cu asks of the warp-ring lane kernel (lane_ring.cu): the grouped entry points' fast path
#pragma once
#include <cstdint>

#include "lane_ep.h"

namespace osmos {
namespace ring {

struct Request {
  bool fused;
  const void* const* wg;  // the entries' matrices (gate, or the only one)
  const void* const* wu;  // fused: the entries' up matrices
  const int32_t *cnt, *xrow, *xin, *win;
  const int8_t* q;
  const float* d;
  const float* scale;
  float lim;
  float* out;
  uint32_t rows, cols, out_stride, n_entries, max_cnt;
  LaneEp ep;  // the expert-parallel step's extras (lane_ep.h); zero: none
  bool dry = false;  // only answer whether the kernel takes the type and shape (1 / 0): nothing is queued
};

// 1: queued on the stream; 0: not a type / shape this kernel takes (nothing queued); -1: the launch was refused
int try_launch(uint32_t type, const Request& r, void* stream);
// the current device's status word, read and cleared (synchronizes): bit 0 a copy never landed, bit 1 a matrix
// pointer was not 16-byte aligned
uint32_t read_status();

}  // namespace ring
}  // namespace osmos
