/* Routing, expert tables, activation and combine of a routed-expert (MoE) FFN layer.
 *
 * Drop-in for the MoE block of the reference's include/osmos/gpu/q4x_ops.h:10-16,131-162 (q4x_route,
 * q4x_expert_bounds, q4x_expert_tiles, q4x_swiglu, q4x_moe_sum): same names, structs, argument meaning and
 * refusals. Every bool entry returns true when the work was queued on `stream` (a cudaStream_t, NULL = default
 * stream; not waited for) and false when it was refused - then nothing was queued.
 */
#ifndef OSMOS_B200_MOE_H
#define OSMOS_B200_MOE_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MM_TILE 16 /* the expert tables' slot tile (reference: include/osmos/gpu/mm.h:7) */

/* an op's output also written as f16 in the 16 x 16 tiled activation layout (token t, column c at
   (t / 16) * 16 * cols + (c / 16) * 256 + (t % 16) * 16 + c % 16); x16 NULL: none. A value past f16's range sets
   *overflow (reference: q4x_ops.h:10-16, kernels/mm.h:41-51). */
typedef struct Q4xX16
{
  void *x16;
  int32_t *overflow;
  uint32_t cols;
  uint32_t row0;
} Q4xX16;

/* softmax over all n_exp (<= 1024) logits of each token, the k (<= 32) greatest probabilities in order (ties to the
   lower id, NaN least) into ids, w = p / max(sum of the picked p, 2^-14), rows[t * k + j] = t
   (reference: q4x_ops.h:131-132, kernels/q4x_moe.hip:38-65,204-210). */
bool q4x_route(const float *logits, uint32_t n_tok, uint32_t n_exp, uint32_t k, int32_t *ids, float *w, int32_t *rows,
               void *stream);

#define Q4X_GROUP_TENSORS 3 /* gate, up, down */
typedef struct Q4xExpertTiles
{
  const void *base[Q4X_GROUP_TENSORS];       /* each tensor's bytes: its experts one after another */
  uint64_t bytes[Q4X_GROUP_TENSORS];         /* an expert's */
  const void *const *tab[Q4X_GROUP_TENSORS]; /* or each tensor's experts' addresses [n_exp] on the device */
  const void **ptr[Q4X_GROUP_TENSORS];       /* out: each tensor's entries' matrices */
  int32_t *cnt;                              /* out: an entry's tokens (0: past the live ones) */
  int32_t *gidx, *hidx;                      /* out: a slot's token, its place; -1 pad */
  uint32_t *xg, *yg, *xd, *yd;               /* out: an entry's input and output offsets, gate / up then down */
  int32_t *where;                            /* out: a pick's place */
  int32_t *off;                              /* scratch: 3 * n_exp ints */
} Q4xExpertTiles;

#define Q4X_TILE_RUNS 4 /* an entry's token tiles: 1, 2, 4 or 8 (16 .. 128 tokens), a launch each */
typedef struct Q4xExpertBounds
{
  uint32_t first[Q4X_TILE_RUNS], count[Q4X_TILE_RUNS];
  uint32_t entries, slots;
} Q4xExpertBounds;

/* the tables' sizes for n picks over n_exp experts (reference: q4x_ops.h:154, kernels/q4x_moe.hip:212-219) */
void q4x_expert_bounds(uint32_t n, uint32_t n_exp, Q4xExpertBounds *b);
/* a step's n picks (ids, k a token) as per-expert tables, built on the GPU: picks stably sorted by expert into
   places (where), each expert's tokens in slots padded to whole tiles of 16 (gidx, hidx), its entries of at most
   128 tokens bucketed in 4 runs by tile count with their offsets and matrix pointers
   (reference: q4x_ops.h:155-156, kernels/q4x_moe.hip:70-165,221-233). */
bool q4x_expert_tiles(const int32_t *ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t dim, uint32_t ff,
                      const Q4xExpertTiles *t, void *stream);
/* q4x_expert_tiles for callers that cannot allocate device memory. No counterpart in the reference.
   Who needs it: an engine step that runs inside a fixed memory budget handed out at start-up (the step path of an
   inference server must never call cudaMalloc: it synchronizes the whole device and can fail under load), or host
   code embedded in a runtime that owns the allocator and gives a plug-in none. Such a caller still passes every
   input and output table; only the tables' scratch (t->off, which is ignored here and may be NULL) lives in a
   fixed 12 KB array inside this library - room for the entry point's own limit of 1024 experts; more is refused
   (false, nothing queued). The array exists once per device that loads the library and is kept until the process
   exits. Nothing is allocated or freed by any call. The first call on a device looks up the array's device address
   (cudaGetSymbolAddress, with that device current) and keeps it: make that first call during set-up, before any
   stream capture. Every call on a device shares the one array and each call overwrites all of it that it reads,
   so calls one after another on a stream are fine, but two calls whose kernels overlap on the GPU (different
   streams without an event between them) race on it. Same results, same refusals otherwise, as q4x_expert_tiles. */
bool q4x_expert_tiles_static(const int32_t *ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t dim, uint32_t ff,
                             const Q4xExpertTiles *t, void *stream);
/* y = silu(g) * u (libm expf), also to side when not NULL (reference: q4x_ops.h:157, q4x_moe.hip:167-170,253-259) */
bool q4x_swiglu(const float *g, const float *u, uint64_t n, float *y, const Q4xX16 *side, void *stream);
/* the activation straight into down's tiled f16 input: slot s (of `slots`, whole tiles of 16 included) gets
   silu(g[idx[s]][c]) * u[idx[s]][c] for c < ff as f16 at (s / 16) * 16 * ff + (c / 16) * 256 + (s % 16) * 16 + c % 16, a
   pad slot (idx[s] < 0) zeros; a value past f16's range sets *overflow. false for ff not a multiple of 16
   (reference: q4x_ops.h:159-160, kernels/q4x_moe.hip:236-259). */
bool q4x_swiglu_rows(const float *g, const float *u, uint32_t ff, const int32_t *idx, uint32_t slots, void *x16,
                     int32_t *overflow, void *stream);
/* out[t][d] = sum_j y[where[t k + j]][d] * w[t k + j] in pick order from 0, + shared[t][d] * sigmoid(shared_logit[t])
   (reference: q4x_ops.h:161-162, kernels/q4x_moe.hip:172-200,274-285) */
bool q4x_moe_sum(const float *y, const int32_t *where, const float *w, uint32_t n_tok, uint32_t k, uint32_t dim,
                 const float *shared, const float *shared_logit, float *out, void *stream);

#ifdef __cplusplus
}
#endif

#endif
