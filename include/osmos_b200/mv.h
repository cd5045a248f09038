/* The decode step's dequant-fused matrix-vector products over F32 activations.
 *
 * Drop-in for the reference's include/osmos/gpu/mv.h:7-20 (mv_run, mv_group, mv_group_tok, mv_strided): same names,
 * argument meaning, limits and refusals. W is any GGUF block type of qtype.h (QTYPE_PATH_MV / _MV_TOK), row-major
 * `rows` x `cols` as the file stores it; x and y are F32 in device-readable memory.
 *
 * A row's sum is a function of the row alone: its 8-value chunks are dealt to 32 lanes (chunk c to lane c % 32),
 * each lane adds its chunks in order with one fmaf a value, and the 32 lane sums are combined by the xor tree
 * 16, 8, 4, 2, 1 - the reference's order (kernels/mv.h:14-70), so a token's output has the same bits alone or in a
 * batch, on any stream, at any launch shape.
 *
 * Every entry returns true when the work was queued on `stream` (a cudaStream_t, NULL = default stream; not
 * waited for) and false when it was refused - then nothing was queued.
 */
#ifndef OSMOS_B200_MV_H
#define OSMOS_B200_MV_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MV_MAX_TOKENS 8    /* tokens a call of mv_run / an entry of mv_group_tok takes (reference: mv.h:7) */
#define MV_MAX_GROUP 65535 /* matrices a grouped call takes (reference: mv.h:8) */

/* y[t * rows + r] = sum_c W[r, c] x[t * cols + c], t < n_tok <= MV_MAX_TOKENS (reference: mv.h:10, mv.hip:264-268).
   false for an unknown type, cols not whole blocks, n_tok 0 or past MV_MAX_TOKENS. */
bool mv_run(uint32_t type, const void *w, uint32_t rows, uint32_t cols, const float *x, uint32_t n_tok, float *y,
            void *stream);
/* n matrices of one type and shape (w: device table of n pointers), one vector each:
   y[m * rows + r] = sum_c W_m[r, c] x[(m / x_div) * x_mat + c] (reference: mv.h:12, mv.hip:234-262).
   false as mv_run, and for n 0 or past MV_MAX_GROUP, x_div 0, x_mat not a multiple of 8. */
bool mv_group(uint32_t type, const void *const *w, uint32_t n, uint32_t rows, uint32_t cols, const float *x,
              uint32_t x_mat, uint32_t x_div, float *y, void *stream);
/* n matrices, matrix m on its cnt[m] (0 = entry skipped; at most max_cnt <= MV_MAX_TOKENS) rows of x starting at
   row xrow[m] (rows xs floats apart) into the same rows of y (ys apart); w, cnt, xrow are device arrays
   (reference: mv.h:14, mv.hip:168-231). false as mv_run, and for n 0 or past MV_MAX_GROUP, max_cnt 0 or past
   MV_MAX_TOKENS, xs shorter than a row or not a multiple of 8. */
bool mv_group_tok(uint32_t type, const void *const *w, const int32_t *cnt, const int32_t *xrow, uint32_t n,
                  uint32_t max_cnt, uint32_t rows, uint32_t cols, const float *x, uint32_t xs, float *y, uint32_t ys,
                  void *stream);
/* mv_run with token t's x at x + t * x_stride and y at y + t * y_stride, any n_tok >= 1 (reference: mv.h:17,
   mv.hip:270-299). false as mv_run (but for the token limit), and for a stride not a multiple of 8 or, with more
   than one token, shorter than its row. */
bool mv_strided(uint32_t type, const void *w, uint32_t rows, uint32_t cols, const float *x, uint32_t x_stride,
                uint32_t n_tok, float *y, uint32_t y_stride, void *stream);

/* NVFP4 (QTYPE_NVFP4: 64-value blocks of four UE4M3 scales and 32 bytes of E2M1) over n = 1 .. 4 tokens, the tensor's
   own scale on each sum: y[t * ys + r] = scale * sum_c W[r, c] x[t * xs + c] (reference: mv.h:19-22,
   kernels/mv_fp4.hip:25-107, 301-320). Its own order of sums, not mv_run's: a row's blocks go to 32 lanes (lane l takes
   blocks l, l + 32, ...), a block adds its four 16-value sub-blocks in turn - part = fmaf(v[j], x[j], fmaf(v[j + 8],
   x[j + 8], part)) for j = 0 .. 7, then acc = fmaf(d, part, acc) - and the lanes meet in the xor tree. false for n
   outside 1 .. 4, cols not whole blocks, xs not a multiple of 4, x not 16-byte or w not 4-byte aligned. */
bool mv_fp4(const void *w, uint32_t rows, uint32_t cols, const float *x, uint32_t xs, uint32_t n, float *y,
            uint32_t ys, float scale, void *stream);
/* NVFP4 matrices each over its own 1 .. 4 tokens (mv_group_tok's tables; an entry of count 0 - or past 4 - is
   skipped), no tensor scale (reference: mv.h:23-27, kernels/mv_fp4.hip:213-298, 322-341). A row's blocks go to 8
   lanes (up to 24 blocks a row), 16 (up to 48) or 32, lane l taking blocks l, l + lanes, ...; the block's sums and the
   tree as mv_fp4's. A token's bits are the same at every count. false for n 0 or past 65535, cols not whole blocks,
   xs not a multiple of 4, x not 16-byte aligned. */
bool mv_fp4_tok(const void *const *w, const int32_t *cnt, const int32_t *xrow, uint32_t n, uint32_t rows,
                uint32_t cols, const float *x, uint32_t xs, float *y, uint32_t ys, void *stream);

/* Not in the reference. mv_run / mv_strided have two kernels that give the same bits: one that stages whole rows
   through shared memory with bulk copies (16-byte aligned w and x, rows whose bytes are a multiple of 16, x and a
   ring of rows fitting shared memory) and a generic one for every other shape. mv_set_staged(0) forces the generic
   kernel (the tests compare the two). mv_status() reads and clears the staged kernel's record on the current device
   (it synchronizes): bit 0 = a bulk copy never landed within the kernel's wait limit, whose rows were not written. */
void mv_set_staged(int on);
uint32_t mv_status(void);

#ifdef __cplusplus
}
#endif

#endif
