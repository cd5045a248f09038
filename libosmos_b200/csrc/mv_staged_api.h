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
  // grouped forms (wt not NULL; w unused): n_entries matrices of one shape, matrix m = wt[m] ...
  const void* const* wt = nullptr;
  uint32_t n_entries = 0;
  const int32_t* cnt = nullptr;   // ... by token: on its cnt[m] (0: skipped; at most n_tok) rows of x from row xrow[m], into the same rows of y
  const int32_t* xrow = nullptr;
  uint32_t x_mat = 0, x_div = 1;  // ... or (cnt NULL) on the one row x + (m / x_div) * x_mat, into y + m * rows
};

// 1: queued on the stream; 0: not a shape this kernel takes (nothing queued: use the generic kernel); -1: the launch
// was refused
int try_launch(uint32_t type, const Request& r, void* stream);
// the most tokens (0 .. 8) a dense launch takes for rows of `cols` values of `type`: their x must fit in shared memory
// beside the rows' ring (0: the type or the columns are not this kernel's)
uint32_t max_tokens(uint32_t type, uint32_t cols);
// the current device's status word, read and cleared (synchronizes): bit 0 a copy never landed, bit 1 a grouped
// entry's matrix was not 16-byte aligned (its rows were not written)
uint32_t read_status();

}  // namespace mvs
}  // namespace osmos
