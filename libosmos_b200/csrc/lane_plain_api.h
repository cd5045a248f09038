// what q8.cu asks of the plain-block dense int8 matvec (lane_plain.cu)
#pragma once
#include <cstdint>

namespace osmos {
namespace plain {

struct Request {
  const void* w;
  const int8_t* q;
  const float* d;
  float* y;
  uint32_t rows, cols, ys, n_tok;
};

// 1: queued on the stream; 0: not a type / shape this kernel takes (nothing queued); -1: the launch was refused
int try_launch(uint32_t type, const Request& r, void* stream);
// the current device's status word, read and cleared (synchronizes): bit 0 a copy never landed
uint32_t read_status();

}  // namespace plain
}  // namespace osmos
