/* The routed-expert FFN of one layer through the int8 lane: host code that only queues kernels through the C ABI
 * (include/osmos_b200/{lane,q8,ops}.h). It plays the role of the GPU half of the reference's fwd_lane_experts
 * (src/run/hip_lane.c:194-221) and entries() (hip_lane.c:71-113), with the tables built on the device instead of
 * on the host, so nothing here waits for the GPU.
 */
#include <stddef.h>

#include "osmos_b200/ep.h"
#include "osmos_b200/lane.h"
#include "osmos_b200/ops.h"
#include "osmos_b200/q8.h"

static uint64_t up256(uint64_t v) { return (v + 255u) & ~(uint64_t)255u; }

/* the scratch's parts in order; with mem NULL only the total is computed */
static uint64_t carve(const LaneLayer *l, uint32_t max_tok, uint8_t *mem, LaneScratch *s)
{
  const uint64_t picks = (uint64_t)max_tok * l->k, ents = lane_max_entries((uint32_t)picks, l->n_exp);
  uint64_t at = 0;
#define PART(field, type, count)                      \
  do                                                  \
  {                                                   \
    if (mem)                                          \
      s->field = (type *)(mem + at);                  \
    at += up256((uint64_t)(count) * sizeof(type));    \
  } while (0)
  PART(xq, int8_t, (uint64_t)max_tok * l->dim);
  PART(xqd, float, (uint64_t)max_tok * (l->dim / 32));
  PART(hh, float, picks * l->ff);
  PART(hq, int8_t, picks * l->ff);
  PART(hqd, float, picks * (l->ff / 32));
  PART(ye, float, picks * l->dim);
  PART(tab.w[0], const void *, ents);
  PART(tab.w[1], const void *, ents);
  PART(tab.w[2], const void *, ents);
  PART(tab.cnt, int32_t, ents);
  PART(tab.xrow, int32_t, ents);
  PART(tab.tok, int32_t, picks);
  PART(tab.pair, int32_t, picks);
  PART(tab.row_of, int32_t, picks);
  PART(tab.order, int32_t, picks);
  PART(tab.off, int32_t, 2u * l->n_exp);
  PART(tab.counts, int32_t, 2);
#undef PART
  if (mem)
    s->tab.max_entries = (uint32_t)ents, s->max_tok = max_tok;
  return at;
}

/* every refusal of every stage (lane_tables, q8_round, q8_gate_up, q8_group_tok, ops_gather_sum[_add]) that depends on
   the layer alone: checked before the first launch, so false means nothing was queued */
static bool layer_ok(const LaneLayer *l)
{
  return l && l->dim && l->ff && l->dim % 256 == 0 && l->ff % 256 == 0 && l->n_exp && l->n_exp <= 1024 && l->k &&
         l->k <= 32 && l->k <= l->n_exp && q8_known(l->type_down) && (!l->type_gu || q8_known(l->type_gu));
}

static bool experts_ok(const LaneExperts *e)
{
  for (int j = 0; j < 3; j++)
    if (!e->tab[j] && (!e->base[j] || !e->bytes[j]))
      return false;
  return true;
}

static bool scratch_ok(const LaneLayer *l, const LaneScratch *s, uint32_t n_tok)
{
  const LaneTables *t = s ? &s->tab : NULL;
  const uint64_t picks = (uint64_t)n_tok * (l ? l->k : 0);
  return s && n_tok && n_tok <= s->max_tok && s->xq && s->xqd && s->hh && s->hq && s->hqd && s->ye && t->w[0] && t->w[1] &&
         t->w[2] && t->cnt && t->xrow && t->tok && t->pair && t->row_of && t->order && t->off && t->counts &&
         t->max_entries >= lane_max_entries((uint32_t)picks, l->n_exp) && t->max_entries <= 65535u;
}

uint64_t lane_scratch_bytes(const LaneLayer *l, uint32_t max_tok)
{
  if (!layer_ok(l) || !max_tok)
    return 0;
  return carve(l, max_tok, NULL, NULL);
}

bool lane_scratch_bind(const LaneLayer *l, uint32_t max_tok, void *mem, uint64_t bytes, LaneScratch *s)
{
  if (!layer_ok(l) || !max_tok || !mem || !s || ((uintptr_t)mem & 255u) || bytes < carve(l, max_tok, NULL, NULL))
    return false;
  carve(l, max_tok, (uint8_t *)mem, s);
  return true;
}

bool lane_ffn(const LaneLayer *l, const LaneScratch *s, const float *x, const int32_t *ids, const float *weights,
              uint32_t n_tok, const float *add, float *out, void *stream)
{
  if (!layer_ok(l) || !experts_ok(&l->experts) || !scratch_ok(l, s, n_tok) || !x || !ids || !weights || !out)
    return false;
  const uint32_t picks = n_tok * l->k, D = l->dim, FF = l->ff;
  const LaneTables *t = &s->tab;
  /* the tables, and each token's input rounded once for all its experts */
  bool ok = lane_tables(ids, picks, l->k, l->n_exp, 0, l->n_exp, &l->experts, t, stream) &&
            q8_round(x, n_tok, D, D, s->xq, s->xqd, stream);
  /* gate, up and the activation (each row's input by token, its routed weight by pick), one launch for every entry */
  if (l->type_gu)
    ok = ok && q8_gate_up(l->type_gu, t->w[0], t->w[1], t->cnt, t->xrow, t->tok, t->pair, t->max_entries,
                          LANE_MAX_TOKENS, FF, D, s->xq, s->xqd, weights, l->lim, s->hh, FF, stream);
  /* the activations to int8, then down; every row of hh below `picks` was written (each pick has a row) */
  ok = ok && q8_round(s->hh, picks, FF, FF, s->hq, s->hqd, stream) &&
       q8_group_tok(l->type_down, t->w[2], t->cnt, t->xrow, NULL, t->max_entries, LANE_MAX_TOKENS, D, FF, s->hq,
                    s->hqd, s->ye, D, stream);
  /* each token's rows summed in ascending expert id, then the shared expert's output */
  ok = ok && (add ? ops_gather_sum_add(out, s->ye, t->order, l->k, n_tok, D, add, stream)
                  : ops_gather_sum(out, s->ye, t->order, l->k, n_tok, D, stream));
  return ok;
}

/* the layer's experts [e0, e1) on tokens that are already int8 (another rank may have rounded them): tables for that
   range, gate / up / activation, the activations to int8, down - rows into s->ye, none of the final sum */
bool lane_ffn_rows(const LaneLayer *l, const LaneScratch *s, const int8_t *q, const float *d, const int32_t *ids,
                   const float *weights, uint32_t n_tok, uint32_t e0, uint32_t e1, void *stream)
{
  if (!layer_ok(l) || !l->type_gu || !experts_ok(&l->experts) || !scratch_ok(l, s, n_tok) || !q || !d || !ids ||
      !weights || e0 >= e1 || e1 > l->n_exp)
    return false;
  const uint32_t picks = n_tok * l->k, D = l->dim, FF = l->ff;
  const LaneTables *t = &s->tab;
  return lane_tables(ids, picks, l->k, l->n_exp, e0, e1, &l->experts, t, stream) &&
         q8_gate_up(l->type_gu, t->w[0], t->w[1], t->cnt, t->xrow, t->tok, t->pair, t->max_entries, LANE_MAX_TOKENS, FF,
                    D, q, d, weights, l->lim, s->hh, FF, stream) &&
         q8_round(s->hh, picks, FF, FF, s->hq, s->hqd, stream) &&
         q8_group_tok(l->type_down, t->w[2], t->cnt, t->xrow, NULL, t->max_entries, LANE_MAX_TOKENS, D, FF, s->hq,
                      s->hqd, s->ye, D, stream);
}
