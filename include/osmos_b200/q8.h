/* The int8 "lane": routed-expert matvecs over activations rounded to int8 in blocks of 32.
 *
 * Drop-in for the reference's include/osmos/gpu/q8.h:7-13 (q8_round, q8_group_tok, q8_gate_up): same names,
 * argument meaning, limits and refusals. The arithmetic is the reference's lane contract (kernels/lane.h:43-75):
 *   - x per 32 values: q = rint(x * (127 / amax)), scale d_x = amax / 127 (F32);
 *   - a weight's 32-value sub-block against it: two exact integer half dots (16 values each);
 *   - each half  part = d_w * (float)(2s+1) * 0.125f * (float)isum,  block = part0 + part1;
 *   - a row's blocks go to L lanes (L = 32 when cols >= 4096, else 16), lane l takes blocks l, l + L, ... in order,
 *     acc = fmaf(d_x, block, acc); the L lane sums are combined by the xor tree L/2 .. 1;
 *   - the activation lane_swiglu uses its own 7-term exp, so CPU and GPU agree bit for bit.
 * An expert therefore gives the same bits whatever the batch, the launch shape, the GPU count, or the side (the
 * reference's CPU lane, src/cpu/q8.c) that computed it.
 *
 * Every entry returns true when the work was queued on `stream` (a cudaStream_t, NULL = default stream; not
 * waited for) and false when it was refused - then nothing was queued.
 */
#ifndef OSMOS_B200_Q8_H
#define OSMOS_B200_Q8_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* rows of x (cols values, rows xs floats apart) to int8 q (row r at q + r * cols) and block scales d (row r at
   d + r * cols / 32). false for cols not whole blocks of 32, xs < cols, rows 0
   (reference: q8.h:7, kernels/q8.hip:81-88, kernels/q8.h:265-277). */
bool q8_round(const float *x, uint32_t rows, uint32_t cols, uint32_t xs, int8_t *q, float *d, void *stream);

/* matrix m (w[m], `rows` x `cols` of a lane type: Q2_K, IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ2_S, IQ1_M) on its cnt[m]
   (1 .. max_cnt <= 8) rows of q / d from row xrow[m], into y's rows from xrow[m] (ys floats apart). Output row r
   reads input row r (xin NULL) or row xin[r]. w, cnt, xrow, xin are device arrays. false for another type, cols not
   whole 256-blocks, n 0 or past 65535, max_cnt 0 or past 8 (reference: q8.h:8-10, kernels/q8.hip:90-107). */
bool q8_group_tok(uint32_t type, const void *const *w, const int32_t *cnt, const int32_t *xrow, const int32_t *xin,
                  uint32_t n, uint32_t max_cnt, uint32_t rows, uint32_t cols, const int8_t *q, const float *d, float *y,
                  uint32_t ys, void *stream);

/* gate and up (both `type`) of entry m on the same input rows, and instead of the two sums the activation:
   h[r][row] = lane_swiglu(gate, up, lim, scale[win ? win[r] : r]) (h rows hs floats apart). false as q8_group_tok,
   and for scale NULL or hs < rows (reference: q8.h:11-13, kernels/q8.hip:109-129). */
bool q8_gate_up(uint32_t type, const void *const *wg, const void *const *wu, const int32_t *cnt, const int32_t *xrow,
                const int32_t *xin, const int32_t *win, uint32_t n, uint32_t max_cnt, uint32_t rows, uint32_t cols,
                const int8_t *q, const float *d, const float *scale, float lim, float *h, uint32_t hs, void *stream);

/* ---- extensions: no counterpart in the reference -------------------------------------------------------------- */

/* true for the types q8_group_tok and q8_gate_up take (the reference's int8 lane types) */
bool q8_known(uint32_t type);

/* One dense matrix over n_tok >= 1 int8 rows: y[t * ys + r] from q row t / d row t - q8_group_tok's sums without
   the tables. Takes the lane types and, beyond the reference, the plain 32-value blocks Q4_0 and Q8_0, for which
   the block value is d_w * (float)isum with isum the whole block's exact integer dot (the lane's rules applied to
   a block with one scale; the reference only multiplies these types with F32 activations, kernels/quant.h:244).
   false for another type, cols not whole blocks (and of 32), n_tok 0, ys < rows with more than one token. */
bool q8_run(uint32_t type, const void *w, uint32_t rows, uint32_t cols, const int8_t *q, const float *d,
            uint32_t n_tok, float *y, uint32_t ys, void *stream);

/* ggml's Q8_0 activation rounding (the rule of the reference's kernels/block.h:88-96): per 32 values
   d = amax / 127, q = roundf(x * (1 / d)) (halves away from zero), and the scale kept is the f16 nearest d,
   written here as that f16's F32 value so q8_run reads it like q8_round's. Same layout and refusals as q8_round. */
bool q8_0_round(const float *x, uint32_t rows, uint32_t cols, uint32_t xs, int8_t *q, float *d, void *stream);

/* The lane entry points choose among kernels that give the same bits. For whole 256-value blocks and 16-byte aligned
   matrices and activations the weights come into shared memory by bulk copies: a kernel whose warps each own a ring
   of rows and keep their activations in registers (the grouped entry points, the common types and shapes; q8_run for
   the plain blocks), else one that stages tiles for the whole block of threads. Every other shape runs a generic
   kernel. q8_set_staged(0) forces the generic kernel, 2 leaves out the warp-ring kernel (the tests compare all
   three); the default is 1. */
void q8_set_staged(int on);
/* The staged kernel never waits without a bound and never faults on a misaligned matrix: it records the event and
   leaves. Reads and clears the current device's record (synchronizes the device): bit 0 a bulk copy did not land
   within the bound, bit 1 a matrix address was not 16-byte aligned; after either, the launch's outputs are not
   valid. */
uint32_t q8_status(void);

#ifdef __cplusplus
}
#endif

#endif
