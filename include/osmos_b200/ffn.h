/* Host drivers of a layer's feed-forward parts: plain C that only queues kernels through this library's C ABI, with
 * every buffer the caller's (one allocation carved by *_scratch_bytes / *_scratch_bind). They play the role of the
 * reference's per-family forward code around these kernels, so that a layer can be run (and measured, and checked)
 * without the engine above:
 *   lane_ffn_f32   the routed experts over F32 activations, an expert read once for the tokens that picked it
 *                  (mv_group_tok) - what the reference's lane runs for the types without an int8 form
 *                  (src/run/hip_lane.c:71-113 with q8 false, :194-221);
 *   shared_ffn     a dense (shared) expert on every token through the f16 tensor-core product
 *                  (src/run/hip_ffn.c:171-185: mm_tokens on gate and up, the clamped activation, mm_tokens on down);
 *                  up to MV_MAX_TOKENS tokens (a decode step) through the F32 matvec instead (mv_strided: the
 *                  reference's product for the types without an f16 kernel, src/run/hip_mat.c:27-35);
 *   q4x_moe        the routed experts through the grouped f16 product, tables built on the GPU
 *                  (src/q4x/hip_layers.c:317-368: q4x_expert_tiles, mm_x16_rows, mm_group x 2, q4x_swiglu_rows,
 *                  mm_group, q4x_moe_sum).
 * Every entry returns true when all its work was queued on `stream` and false when it was refused; what a refusal
 * depends on is checked before the first launch, so false means nothing was queued.
 */
#ifndef OSMOS_B200_FFN_H
#define OSMOS_B200_FFN_H

#include <stdbool.h>
#include <stdint.h>

#include "osmos_b200/lane.h"
#include "osmos_b200/moe.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- the routed experts over F32 activations ---------------------------------------------------------------------- */
typedef struct LaneScratchF32
{
  uint32_t max_tok;
  float *xg;  /* [picks][dim]: each row's input (its token's x) */
  float *wg;  /* [picks]: each row's routed weight */
  float *ga;  /* [picks][ff] */
  float *up;  /* [picks][ff] */
  float *hh;  /* [picks][ff] */
  float *ye;  /* [picks][dim] */
  LaneTables tab;
} LaneScratchF32;
uint64_t lane_f32_scratch_bytes(const LaneLayer *l, uint32_t max_tok);
bool lane_f32_scratch_bind(const LaneLayer *l, uint32_t max_tok, void *mem, uint64_t bytes, LaneScratchF32 *s);
/* as lane_ffn (lane.h) with the experts' matrices of any type mv_group_tok takes and the activation in the lane's own
   operations (ops_swiglu_lane); l->type_gu is the gate's and the up's type */
bool lane_ffn_f32(const LaneLayer *l, const LaneScratchF32 *s, const float *x, const int32_t *ids, const float *weights,
                  uint32_t n_tok, const float *add, float *out, void *stream);

/* ---- a dense expert on every token ---------------------------------------------------------------------------------- */
typedef struct SharedExpert
{
  uint32_t type_gu, type_down; /* the gate's and up's type (one), the down's: types with a matrix-product kernel */
  uint32_t dim, ff;
  float lim;                   /* the activation's clamp (ops_swiglu's) */
  const void *gate, *up, *down; /* [ff][dim], [ff][dim], [dim][ff] on the device */
} SharedExpert;
typedef struct SharedScratch
{
  uint32_t max_tok;
  float *g, *u, *h;  /* [max_tok][ff] each */
  void *x16;         /* f16 activations of the larger of dim and ff, max_tok (at most 2048) rounded up to 16 */
  int32_t *overflow; /* one word: set when a value left f16's range (the caller reads it after the step) */
} SharedScratch;
uint64_t shared_scratch_bytes(const SharedExpert *e, uint32_t max_tok);
bool shared_scratch_bind(const SharedExpert *e, uint32_t max_tok, void *mem, uint64_t bytes, SharedScratch *s);
/* y[t][:] = down (silu(min(gate x, lim)) * clamp(up x, +-lim)) for n tokens of x ([n][dim], row stride dim). More than
   MV_MAX_TOKENS tokens: f16 operands, F32 sums (mm_tokens' bound). Fewer: F32 operands in the matvec's order (mv_run's
   bits) - a token's bits are those of its step's path, not the same on both. */
bool shared_ffn(const SharedExpert *e, const SharedScratch *s, const float *x, uint32_t n, float *y, void *stream);

/* ---- the routed experts through the grouped f16 product -------------------------------------------------------------- */
typedef struct Q4xMoeLayer
{
  uint32_t type[Q4X_GROUP_TENSORS]; /* gate, up, down */
  uint32_t dim, ff, n_exp, k;
  const void *base[Q4X_GROUP_TENSORS]; /* each tensor's experts one after another ... */
  uint64_t bytes[Q4X_GROUP_TENSORS];
  const void *const *tab[Q4X_GROUP_TENSORS]; /* ... or a device table of their addresses */
} Q4xMoeLayer;
typedef struct Q4xMoeScratch
{
  uint32_t max_tok;
  Q4xExpertBounds bounds; /* for max_tok * k picks */
  int32_t *ids, *rows;    /* [picks] */
  float *w;               /* [picks] */
  const void **ptr;       /* [3][entries] */
  int32_t *cnt, *gidx, *hidx, *where, *off;
  uint32_t *xg, *yg, *xd, *yd;
  void *xe16;        /* f16 slots x max(dim, ff) */
  float *ga, *up, *y; /* [picks][ff], [picks][ff], [picks][dim] */
  int32_t *overflow;
} Q4xMoeScratch;
uint64_t q4x_moe_scratch_bytes(const Q4xMoeLayer *l, uint32_t max_tok);
bool q4x_moe_scratch_bind(const Q4xMoeLayer *l, uint32_t max_tok, void *mem, uint64_t bytes, Q4xMoeScratch *s);
/* logits [n][n_exp] (the router's matrix product is the caller's), x [n][dim], shared [n][dim] and shared_logit [n]
   (the shared expert's output and its gate's logit, as q4x_moe_sum takes them), out [n][dim]; n <= max_tok, and at most
   2048 * 16 / k tokens so that an expert's part fits one x16 */
bool q4x_moe(const Q4xMoeLayer *l, const Q4xMoeScratch *s, const float *x, const float *logits, const float *shared,
             const float *shared_logit, uint32_t n, float *out, void *stream);

#ifdef __cplusplus
}
#endif

#endif
