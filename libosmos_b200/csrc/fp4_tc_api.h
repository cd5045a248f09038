// what mm_fp4.cu asks of the block-scaled FP4 tensor-core product (fp4_tc.cu)
#pragma once
#include <cstdint>

namespace osmos {
namespace fp4_tc {

// y[t * ys + r] = scale * sum_c W[r, c] xq[t, c] for t < n: W an NVFP4 (mx false) or MXFP4 (mx true) matrix of GGUF
// blocks; aq the tokens' E2M1 codes in K order, two a byte, a token's row aq_stride bytes on; as their scale bytes
// (UE4M3 a 16 / UE8M0 a 32 values), a token's row as_stride bytes on.
// 1: queued on the stream; 0: not a shape or alignment this kernel takes (nothing queued); -1: the launch was refused
int try_launch(bool mx, const void* w, uint32_t rows, uint32_t cols, const void* aq, uint32_t aq_stride, const void* as,
               uint32_t as_stride, uint32_t n, float scale, float* y, uint32_t ys, void* stream);
// the kernel's instruction descriptor for an N-token MMA (for the host test against CUTLASS's encoder); sf_id: the first
// scale factor's byte in its tensor-memory word
uint32_t instr_desc(bool mx, uint32_t n, uint32_t sf_id);
// the current device's status word, read and cleared (synchronizes): bit 0 a wait ran out
uint32_t read_status();

}  // namespace fp4_tc
}  // namespace osmos
