// what mv.cu asks of the staged F32-activation matvec (mv_staged.cu)
#pragma once
#include <cstdint>

namespace osmos {
namespace mvs {

struct Request {
  const void* w;
  const float* x;
  float* y;
  uint32_t rows, cols, xs, ys, n_tok;  // n_tok <= 8
};

// 1: queued on the stream; 0: not a shape this kernel takes (nothing queued: use the generic kernel); -1: the launch
// was refused
int try_launch(uint32_t type, const Request& r, void* stream);
// the current device's status word, read and cleared (synchronizes): bit 0 a copy never landed
uint32_t read_status();

}  // namespace mvs
}  // namespace osmos
