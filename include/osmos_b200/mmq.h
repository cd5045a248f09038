/* Q4_K weights x int8 activations: the prefill / batched-expert matmul with exact integer group dots.
 *
 * Drop-in for the reference's include/osmos/gpu/mmq.h:7-33 (mmq_x8_at, mmq_dx_at, mmq_x8_rows, mmq_group,
 * mmq_known): same names, layouts, argument meaning and refusals.
 *
 * The contract (reference: mmq.h:36-56, kernels/mmq.hip:33-52,60-151): activations per 32-value group
 * dx = amax / 127, x8 = clamp(rint(x / dx), +-127), sx = dx * (float)sum(x8); a weight is d sc q - dmin m, so a
 * group's share of an output is (d sc) dx I - (dmin m) sx with I = sum q x8 (exact); in F32 and a fixed order: K split
 * in 4 partitions by 256-value block (partition p: blocks p, p + 4, ...), each its groups in order
 *   v = (d sc) * dx;  acc = fmaf(v, (float)I, acc);  acc = fmaf(dmin m, -sx, acc);
 * and the four partitions added in order 0..3. A token's bits are the same whatever its batch.
 *
 * Every bool entry returns true when the work was queued on `stream` (a cudaStream_t, NULL = default stream; not
 * waited for) and false when it was refused - then nothing was queued.
 */
#ifndef OSMOS_B200_MMQ_H
#define OSMOS_B200_MMQ_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MMQ_GROUP 32    /* an activation group: one scale a 32 values (reference: mmq.h:7) */
#define MMQ_MAX_TILES 4 /* (reference: mmq.h:8) */
#define MMQ_SLOTS 16    /* the layouts' slot tile (reference: mmq.h:9) */

#if defined(__CUDACC__)
#define MMQ_HD __host__ __device__
#else
#define MMQ_HD
#endif
/* slot s's value c in x8: tiles of 16 slots, a group at a time, each slot's 32 codes together (reference: mmq.h:17-21) */
static inline MMQ_HD uint64_t mmq_x8_at(uint32_t s, uint32_t c, uint32_t cols)
{
  return (uint64_t)(s / MMQ_SLOTS) * MMQ_SLOTS * cols + (uint64_t)(c / MMQ_GROUP) * (MMQ_SLOTS * MMQ_GROUP) +
         (s % MMQ_SLOTS) * MMQ_GROUP + c % MMQ_GROUP;
}
/* slot s's group g in dx / sx: a tile's 16 slots side by side a group (reference: mmq.h:23-27) */
static inline MMQ_HD uint64_t mmq_dx_at(uint32_t s, uint32_t g, uint32_t groups)
{
  return (uint64_t)(s / MMQ_SLOTS) * MMQ_SLOTS * groups + (uint64_t)g * MMQ_SLOTS + s % MMQ_SLOTS;
}

/* slot s = row idx[s] of x (xs floats apart; -1: zeros) quantized a group at a time into x8 / dx / sx (buffers of
   whole 16-slot tiles). false for a NULL, slots 0, cols not a multiple of 32, xs < cols (reference: mmq.h:29-30) */
bool mmq_x8_rows(const float *x, uint32_t xs, const int32_t *idx, uint32_t slots, uint32_t cols, int8_t *x8, float *dx,
                 float *sx, void *stream);
/* n_mat matrices of `type` (Q4_K), matrix m over its first cnt[m] (<= max_cnt) tokens = slots soff[m] .. (a multiple
   of 16) into y + yoff[m] + t * ys. rows a multiple of 16, cols of 256; w, cnt, soff, yoff device arrays
   (reference: mmq.h:31-33) */
bool mmq_group(uint32_t type, const void *const *w, const int32_t *cnt, uint32_t n_mat, uint32_t max_cnt, uint32_t rows,
               uint32_t cols, const int8_t *x8, const float *dx, const float *sx, const uint32_t *soff, float *y,
               const uint32_t *yoff, uint32_t ys, void *stream);
bool mmq_known(uint32_t type);

/* ---- extensions: no counterpart in the reference -------------------------------------------------------------- */
/* mmq_group runs one of two kernels that give the same bits: a tensor-core one (tcgen05 kind::i8, for rows in 128s
   and 16-byte aligned activations) and a generic one for every other shape. mmq_set_tensor(0) forces the generic kernel
   (the tests compare the two); the default is 1. */
void mmq_set_tensor(int on);
/* the tensor-core kernel's waits are bounded: reads and clears the current device's record (synchronizes the device);
   bit 0: a wait ran out and the launch's outputs are not valid */
uint32_t mmq_status(void);

#ifdef __cplusplus
}
#endif

#endif
