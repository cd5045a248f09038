/* Device-built tables and the host-side driver of the int8 lane's routed-expert FFN.
 *
 * The reference builds these tables on the host after waiting for the router's picks
 * (src/run/hip_lane.c:16-27,115-192: LaneTabs, fwd_lane_experts) and then launches once per token count
 * (hip_lane.c:71-113). Here the tables are built on the GPU, so a layer needs no host round trip, and one launch
 * covers every entry whatever its count. The arithmetic is q8.h's; the tables only say which rows go where, so the
 * results are the reference's bits.
 *
 * lane_tables / lane_max_entries have no counterpart entry point in the reference (their job is done by host code
 * there). lane_ffn plays the role of fwd_lane_experts' GPU half (hip_lane.c:194-221).
 */
#ifndef OSMOS_B200_LANE_H
#define OSMOS_B200_LANE_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LANE_MAX_TOKENS 8 /* rows an entry holds: MV_MAX_TOKENS (reference: mv.h:7, hip_lane.c:143) */

/* where the experts' matrices are: each tensor's experts one after another (base + e * bytes), or a device table of
   addresses (tab[j][e]); j = 0 gate, 1 up, 2 down */
typedef struct LaneExperts
{
  const void *base[3];
  uint64_t bytes[3];
  const void *const *tab[3];
} LaneExperts;

/* all device memory, sized by the caller: n = picks (tokens * k), max_entries >= lane_max_entries(n, n_exp) */
typedef struct LaneTables
{
  const void **w[3]; /* out [max_entries]: an entry's gate, up, down */
  int32_t *cnt;      /* out [max_entries]: an entry's rows, 1 .. 8; 0 past the live entries */
  int32_t *xrow;     /* out [max_entries]: an entry's first row */
  int32_t *tok;      /* out [n]: row r's token (the gate / up input row) */
  int32_t *pair;     /* out [n]: row r's pick index (its routed weight's place) */
  int32_t *row_of;   /* out [n]: pick i's row, -1 when its expert is outside [expert0, expert1) */
  int32_t *order;    /* out [n]: token t's rows in ascending expert id at order[t * k ..], the -1s last */
  int32_t *off;      /* scratch [2 * n_exp] */
  int32_t *counts;   /* out [2]: live entries, rows */
  uint32_t max_entries;
} LaneTables;

/* an upper bound of the entries n picks over n_exp experts make */
uint32_t lane_max_entries(uint32_t n, uint32_t n_exp);

/* rows = the picks whose expert lies in [expert0, expert1), sorted by (expert, pick index); an expert's rows cut into
   entries of at most 8. ids[n] (k a token) on the device. false for a shape it refuses (n not a multiple of k,
   k > 32, n_exp > 1024, an empty expert range, tables too small or missing). */
bool lane_tables(const int32_t *ids, uint32_t n, uint32_t k, uint32_t n_exp, uint32_t expert0, uint32_t expert1,
                 const LaneExperts *ex, const LaneTables *t, void *stream);

/* ---- the layer's driver (host code, libosmos_b200/host/lane_ffn.c) --------------------------------------------- */

typedef struct LaneLayer
{
  uint32_t type_gu, type_down; /* the experts' block types (q8.h's lane types) */
  uint32_t dim, ff;            /* the FFN's width and an expert's hidden width */
  uint32_t n_exp, k;           /* experts, and picks a token */
  float lim;                   /* the activation's clamp */
  LaneExperts experts;
} LaneLayer;

/* a step's device scratch for at most max_tok tokens; made by lane_scratch_bytes / lane_scratch_bind over one
   caller-owned allocation (256-byte aligned) */
typedef struct LaneScratch
{
  uint32_t max_tok;
  int8_t *xq;    /* [max_tok][dim] */
  float *xqd;    /* [max_tok][dim / 32] */
  float *hh;     /* [picks][ff] */
  int8_t *hq;    /* [picks][ff] */
  float *hqd;    /* [picks][ff / 32] */
  float *ye;     /* [picks][dim] */
  LaneTables tab;
} LaneScratch;

uint64_t lane_scratch_bytes(const LaneLayer *l, uint32_t max_tok);
bool lane_scratch_bind(const LaneLayer *l, uint32_t max_tok, void *mem, uint64_t bytes, LaneScratch *s);

/* one layer's routed experts for n_tok tokens: x [n_tok][dim] F32, ids / weights [n_tok * k] (the router's), add
   (or NULL) [n_tok][dim] added after the experts' sum (the shared expert's output), out [n_tok][dim]; all on the
   device. Queues: the tables, q8_round(x), q8_gate_up, q8_round(h), q8_group_tok(down), and the per-token sum in
   ascending expert id. false when any step refuses. */
bool lane_ffn(const LaneLayer *l, const LaneScratch *s, const float *x, const int32_t *ids, const float *weights,
              uint32_t n_tok, const float *add, float *out, void *stream);

#ifdef __cplusplus
}
#endif

#endif
