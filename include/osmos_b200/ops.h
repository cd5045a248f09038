/* The small steps around the routed-expert FFN: routers, activations, row gathers and sums, the host-flag wait,
 * and the MX-format activation rounding.
 *
 * Drop-in for the part of the reference's include/osmos/gpu/ops.h that lies on the quantized-weight matrix path
 * (ops.h:51,55,98-124): same names, argument meaning and refusals. Every entry returns true when the work was
 * queued on `stream` (a cudaStream_t, NULL = default stream; not waited for) and false when it was refused -
 * then nothing was queued.
 */
#ifndef OSMOS_B200_OPS_H
#define OSMOS_B200_OPS_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OPS_MAX_EXPERTS 1024 /* reference: ops.h:9 */
#define OPS_MAX_TOPK 16      /* reference: ops.h:10 */

typedef enum OpsScore
{
  OPS_SCORE_SQRT_SOFTPLUS, /* DeepSeek's */
  OPS_SCORE_SIGMOID        /* sigmoid scores */
} OpsScore;

/* DeepSeek-style router: score = sqrt(softplus(logit)) (or sigmoid), the k experts of the highest score + bias
   (ties to the lower id, NaN least) in that order into idx, w = score / (sum of the picked scores + 1e-20) * scale
   (reference: ops.h:98-106, kernels/ops.hip:456-484,794-809). */
bool ops_router(const float *logits, const float *bias, uint32_t n_exp, uint32_t k, float scale, uint32_t n_tok,
                int32_t *idx, float *w, void *stream);
bool ops_router_scored(const float *logits, const float *bias, uint32_t n_exp, uint32_t k, float scale, OpsScore score,
                       uint32_t n_tok, int32_t *idx, float *w, void *stream);
/* h = silu(min(g, lim)) * clamp(u, -lim, lim), times scale[t] when scale is not NULL (reference: ops.h:107,
   kernels/ops.hip:487-499) */
bool ops_swiglu(const float *g, const float *u, uint32_t n, float lim, const float *scale, uint32_t n_tok, float *h,
                void *stream);
/* the same activation in the lane's own operations, scale required (reference: ops.h:111, kernels/ops.hip:502-507) */
bool ops_swiglu_lane(const float *g, const float *u, uint32_t n, float lim, const float *scale, uint32_t n_tok,
                     float *h, void *stream);
/* dst[i][:] = src[idx[i]][:], n rows of len (reference: ops.h:113, kernels/ops.hip:510) */
bool ops_gather_rows(float *dst, const float *src, const int32_t *idx, uint32_t n, uint32_t len, void *stream);
/* y[t][:] = sum over j < m of src[idx[t * m + j]][:] from 0 in j's order (reference: ops.h:114,
   kernels/ops.hip:517-525) */
bool ops_gather_sum(float *y, const float *src, const int32_t *idx, uint32_t m, uint32_t n, uint32_t dim,
                    void *stream);
/* ops_gather_sum, then add's values added to the sums (reference: ops.h:116) */
bool ops_gather_sum_add(float *y, const float *src, const int32_t *idx, uint32_t m, uint32_t n, uint32_t dim,
                        const float *add, void *stream);
/* rows idx[0 .. n) of src copied to the same rows of dst (reference: ops.h:124, kernels/ops.hip:555) */
bool ops_copy_rows(float *dst, const float *src, const int32_t *idx, uint32_t n, uint32_t len, void *stream);
/* the stream held until *flag (host memory the GPU maps) holds value, or value with its top bit set
   (reference: ops.h:123, kernels/ops.hip:544-552). Unlike the reference's, this wait is bounded: after about
   ops_wait_limit_ms() milliseconds without the value it stops, sets bit 0 of the word ops_wait_status() returns
   and lets the stream go on, so a poster that died cannot hang the GPU. */
bool ops_wait(const uint32_t *flag, uint32_t value, void *stream);
/* the bound of ops_wait in milliseconds (default 2000); set before queueing the wait */
void ops_wait_set_limit_ms(uint32_t ms);
uint32_t ops_wait_limit_ms(void);
/* reads and clears the status word of the current device (synchronizes the device): bit 0 = an ops_wait ran out */
uint32_t ops_wait_status(void);

/* each `block` values rounded to E2M1 under a scale - a power of two 2^ceil(log2(max(amax, 6 * 2^-126) / 6)), or
   amax / 6 rounded to E4M3 (e4m3_scale) - in place; packed (or NULL): rows of dim as dim / 2 code bytes (even value
   in the low nibble) then a scale byte a block (UE8M0, or the E4M3 code) (reference: ops.h:55,
   kernels/round.hip:49-78,140-148). */
bool ops_fp4_round(float *x, uint64_t n, uint32_t block, bool e4m3_scale, void *packed, uint32_t dim, void *stream);
/* each 32 values rounded to E4M3 under the power-of-two scale 2^ceil(log2(max(amax, 1e-4) / 448)); packed (or
   NULL): rows of dim code bytes then dim / 32 UE8M0 bytes (reference: ops.h:51, kernels/round.hip:32-45,150-154) */
bool ops_fp8_round(float *x, uint64_t n, void *packed, uint32_t dim, void *stream);

#ifdef __cplusplus
}
#endif

#endif
