/* The f16 activation layout the prefill matrix products read, and the conversions into it.
 *
 * Drop-in for the activation side of the reference's include/osmos/gpu/mm.h: mm_x16 (:13), mm_x16_rows (:35),
 * mm_x16_heads (:37) and the layout function of kernels/mm.h:41-51 - same names, argument meaning, limits and
 * refusals. (The products themselves - mm_run, mm_run2, mm_tokens, mm_group - are not in this library yet.)
 *
 * x16 holds token t's column c, of rows xts values long, at half index
 *   (t / 16) * 16 * xts + (c / 16) * 256 + (t % 16) * 16 + c % 16
 * so every 16-token x 16-column fragment is 512 contiguous bytes. Values are rounded F32 -> f16 to nearest even; a
 * value past f16's range (or a NaN) sets *overflow (a device int32 the caller clears before the step and reads after
 * it: the step's results are then refused). Rows past the last token, up to the next multiple of 16, are zero.
 *
 * Every entry returns true when the work was queued on `stream` (a cudaStream_t, NULL = default stream; not waited
 * for) and false when it was refused - then nothing was queued.
 */
#ifndef OSMOS_B200_MM_H
#define OSMOS_B200_MM_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MM_TILE 16         /* reference: mm.h:7 */
#define MM_MAX_TOKENS 2048 /* reference: mm.h:8 */

/* where token t's column c lies in a tiled x16 of rows xts long, in halves (reference: kernels/mm.h:47-49) */
static inline uint64_t mm_x16_at(uint32_t t, uint32_t c, uint32_t xts) {
  return (uint64_t)(t / MM_TILE) * MM_TILE * xts + (uint64_t)(c / MM_TILE) * (MM_TILE * MM_TILE) + (t % MM_TILE) * MM_TILE +
         c % MM_TILE;
}

/* n rows of cols F32 (row t at x + t * xs) into x16: n rounded up to whole tiles of rows, cols f16 each
   (reference: mm.h:13, mm.hip:467-479). false for n 0 or past MM_MAX_TOKENS, cols 0 or not a multiple of 16, or,
   with more than one row, xs shorter than a row. */
bool mm_x16(const float *x, uint32_t xs, uint32_t n, uint32_t cols, void *x16, int32_t *overflow, void *stream);
/* slot s is row idx[s] of x (-1: zeros; idx a device array of `slots` ints), slots rounded up to whole tiles
   (reference: mm.h:35, mm.hip:608-617). false for no slots, cols 0 or not a multiple of 16, xs shorter than a row or
   not a multiple of 4, or x not 16-byte aligned. */
bool mm_x16_rows(const float *x, uint32_t xs, const int32_t *idx, uint32_t slots, uint32_t cols, void *x16,
                 int32_t *overflow, void *stream);
/* every head's slice of n rows (head h's cols values at x + t * xs + h * hs) to its own tiled x16, head h's at
   x16 + h * n16 * cols halves, n16 = n in whole tiles: each as mm_x16(x + h * hs, xs, n, cols) would put it
   (reference: mm.h:37, mm.hip:593-606). false for n 0 or past MM_MAX_TOKENS, no heads, cols 0 or not a multiple of
   16, hs or xs not a multiple of 4, x or x16 not 16-byte aligned, or a last head reaching past a row. */
bool mm_x16_heads(const float *x, uint32_t xs, uint32_t n, uint32_t heads, uint32_t hs, uint32_t cols, void *x16,
                  int32_t *overflow, void *stream);

#ifdef __cplusplus
}
#endif

#endif
