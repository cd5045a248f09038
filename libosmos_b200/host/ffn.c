/* Host drivers of a layer's feed-forward parts (include/osmos_b200/ffn.h): plain C over the kernel C ABI. Nothing here
 * waits for the GPU; every refusal is decided before the first launch.
 */
#include <stddef.h>
#include <string.h>

#include "osmos_b200/ffn.h"
#include "osmos_b200/mm.h"
#include "osmos_b200/mv.h"
#include "osmos_b200/ops.h"
#include "osmos_b200/qtype.h"

static uint64_t up256(uint64_t v) { return (v + 255u) & ~(uint64_t)255u; }

#define PART(field, type, count)                   \
  do                                               \
  {                                                \
    if (mem)                                       \
      s->field = (type *)(mem + at);               \
    at += up256((uint64_t)(count) * sizeof(type)); \
  } while (0)

/* ---- the F32 lane --------------------------------------------------------------------------------------------------- */
static bool takes_mv_tok(uint32_t type)
{
  const OsmosQTypeInfo *t = qtype_info(type);
  return t && (t->paths & QTYPE_PATH_MV_TOK);
}

static bool f32_layer_ok(const LaneLayer *l)
{
  const OsmosQTypeInfo *g = l ? qtype_info(l->type_gu) : NULL, *d = l ? qtype_info(l->type_down) : NULL;
  return l && g && d && takes_mv_tok(l->type_gu) && takes_mv_tok(l->type_down) && l->dim && l->ff && l->dim % 8 == 0 &&
         l->ff % 8 == 0 && l->dim % g->values == 0 && l->ff % d->values == 0 && l->n_exp && l->n_exp <= 1024 && l->k &&
         l->k <= 32 && l->k <= l->n_exp;
}

static uint64_t carve_f32(const LaneLayer *l, uint32_t max_tok, uint8_t *mem, LaneScratchF32 *s)
{
  const uint64_t picks = (uint64_t)max_tok * l->k, ents = lane_max_entries((uint32_t)picks, l->n_exp);
  uint64_t at = 0;
  PART(xg, float, picks * l->dim);
  PART(wg, float, picks);
  PART(ga, float, picks * l->ff);
  PART(up, float, picks * l->ff);
  PART(hh, float, picks * l->ff);
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
  if (mem)
    s->tab.max_entries = (uint32_t)ents, s->max_tok = max_tok;
  return at;
}

uint64_t lane_f32_scratch_bytes(const LaneLayer *l, uint32_t max_tok)
{
  return f32_layer_ok(l) && max_tok ? carve_f32(l, max_tok, NULL, NULL) : 0;
}

bool lane_f32_scratch_bind(const LaneLayer *l, uint32_t max_tok, void *mem, uint64_t bytes, LaneScratchF32 *s)
{
  if (!f32_layer_ok(l) || !max_tok || !mem || !s || ((uintptr_t)mem & 255u) || bytes < carve_f32(l, max_tok, NULL, NULL))
    return false;
  carve_f32(l, max_tok, (uint8_t *)mem, s);
  return true;
}

bool lane_ffn_f32(const LaneLayer *l, const LaneScratchF32 *s, const float *x, const int32_t *ids, const float *weights,
                  uint32_t n_tok, const float *add, float *out, void *stream)
{
  if (!f32_layer_ok(l) || !s || !x || !ids || !weights || !out || !n_tok || n_tok > s->max_tok)
    return false;
  const LaneTables *t = &s->tab;
  const uint32_t picks = n_tok * l->k, D = l->dim, FF = l->ff;
  for (int j = 0; j < 3; j++)
    if ((!l->experts.tab[j] && (!l->experts.base[j] || !l->experts.bytes[j])) || !t->w[j])
      return false;
  if (!s->xg || !s->wg || !s->ga || !s->up || !s->hh || !s->ye || !t->cnt || !t->xrow || !t->tok || !t->pair || !t->row_of ||
      !t->order || !t->off || !t->counts || t->max_entries < lane_max_entries(picks, l->n_exp) || t->max_entries > MV_MAX_GROUP)
    return false;
  /* the tables; each row's input and routed weight gathered (the F32 matvec reads its rows where an entry's lie) */
  return lane_tables(ids, picks, l->k, l->n_exp, 0, l->n_exp, &l->experts, t, stream) &&
         ops_gather_rows(s->xg, x, t->tok, picks, D, stream) && ops_gather_rows(s->wg, weights, t->pair, picks, 1, stream) &&
         mv_group_tok(l->type_gu, t->w[0], t->cnt, t->xrow, t->max_entries, LANE_MAX_TOKENS, FF, D, s->xg, D, s->ga, FF, stream) &&
         mv_group_tok(l->type_gu, t->w[1], t->cnt, t->xrow, t->max_entries, LANE_MAX_TOKENS, FF, D, s->xg, D, s->up, FF, stream) &&
         ops_swiglu_lane(s->ga, s->up, FF, l->lim, s->wg, picks, s->hh, stream) &&
         mv_group_tok(l->type_down, t->w[2], t->cnt, t->xrow, t->max_entries, LANE_MAX_TOKENS, D, FF, s->hh, FF, s->ye, D, stream) &&
         (add ? ops_gather_sum_add(out, s->ye, t->order, l->k, n_tok, D, add, stream)
              : ops_gather_sum(out, s->ye, t->order, l->k, n_tok, D, stream));
}

/* ---- the shared expert ---------------------------------------------------------------------------------------------- */
static bool shared_ok(const SharedExpert *e)
{
  return e && e->dim && e->ff && e->gate && e->up && e->down && mm_fits(e->type_gu, e->ff, e->dim) &&
         mm_fits(e->type_down, e->dim, e->ff);
}

static uint64_t carve_shared(const SharedExpert *e, uint32_t max_tok, uint8_t *mem, SharedScratch *s)
{
  const uint64_t widest = e->dim > e->ff ? e->dim : e->ff;
  const uint64_t n16 = ((max_tok < MM_MAX_TOKENS ? max_tok : MM_MAX_TOKENS) + 15u) / 16u * 16u;
  uint64_t at = 0;
  PART(g, float, (uint64_t)max_tok * e->ff);
  PART(u, float, (uint64_t)max_tok * e->ff);
  PART(h, float, (uint64_t)max_tok * e->ff);
  PART(x16, uint16_t, n16 * widest);
  PART(overflow, int32_t, 1);
  if (mem)
    s->max_tok = max_tok;
  return at;
}

uint64_t shared_scratch_bytes(const SharedExpert *e, uint32_t max_tok)
{
  return shared_ok(e) && max_tok ? carve_shared(e, max_tok, NULL, NULL) : 0;
}

bool shared_scratch_bind(const SharedExpert *e, uint32_t max_tok, void *mem, uint64_t bytes, SharedScratch *s)
{
  if (!shared_ok(e) || !max_tok || !mem || !s || ((uintptr_t)mem & 255u) || bytes < carve_shared(e, max_tok, NULL, NULL))
    return false;
  carve_shared(e, max_tok, (uint8_t *)mem, s);
  return true;
}

bool shared_ffn(const SharedExpert *e, const SharedScratch *s, const float *x, uint32_t n, float *y, void *stream)
{
  if (!shared_ok(e) || !s || !x || !y || !n || n > s->max_tok || !s->g || !s->u || !s->h || !s->x16 || !s->overflow ||
      ((uintptr_t)s->x16 & 15u))
    return false;
  /* a decode step's few tokens: the F32 matvec, which reads each matrix once at the rate of its bytes (the tensor-core
     product decodes 128-row tiles a block: a 2048-row matrix would keep 16 of the GPU's blocks busy). Its sums are the
     reference's mv order, bit for bit; nothing it can refuse is left unchecked above (mm_fits holds the shapes) */
  if (n <= MV_MAX_TOKENS)
    return mv_strided(e->type_gu, e->gate, e->ff, e->dim, x, e->dim, n, s->g, e->ff, stream) &&
           mv_strided(e->type_gu, e->up, e->ff, e->dim, x, e->dim, n, s->u, e->ff, stream) &&
           ops_swiglu(s->g, s->u, e->ff, e->lim, NULL, n, s->h, stream) &&
           mv_strided(e->type_down, e->down, e->dim, e->ff, s->h, e->ff, n, y, e->dim, stream);
  /* gate and up in one pass over x's f16 (each the bits it has alone), the clamped activation, then down */
  return mm_tokens(e->type_gu, e->gate, e->ff, s->g, e->ff, e->up, e->ff, s->u, e->ff, e->dim, x, e->dim, n, s->x16, s->overflow,
                   false, stream) &&
         ops_swiglu(s->g, s->u, e->ff, e->lim, NULL, n, s->h, stream) &&
         mm_tokens(e->type_down, e->down, e->dim, y, e->dim, NULL, 0, NULL, 0, e->ff, s->h, e->ff, n, s->x16, s->overflow, false,
                   stream);
}

/* ---- the routed experts through the grouped f16 product -------------------------------------------------------------- */
static bool q4x_layer_ok(const Q4xMoeLayer *l)
{
  if (!l || !l->dim || !l->ff || !l->n_exp || l->n_exp > 1024 || !l->k || l->k > 32 || l->k > l->n_exp)
    return false;
  for (int j = 0; j < Q4X_GROUP_TENSORS; j++)
    if (!l->tab[j] && (!l->base[j] || !l->bytes[j]))
      return false;
  return mm_fits(l->type[0], l->ff, l->dim) && mm_fits(l->type[1], l->ff, l->dim) && mm_fits(l->type[2], l->dim, l->ff);
}

static uint64_t carve_q4x(const Q4xMoeLayer *l, uint32_t max_tok, uint8_t *mem, Q4xMoeScratch *s)
{
  const uint32_t picks = max_tok * l->k;
  Q4xExpertBounds b;
  q4x_expert_bounds(picks, l->n_exp, &b);
  const uint64_t widest = l->dim > l->ff ? l->dim : l->ff;
  uint64_t at = 0;
  PART(ids, int32_t, picks);
  PART(rows, int32_t, picks);
  PART(w, float, picks);
  PART(ptr, const void *, (uint64_t)Q4X_GROUP_TENSORS * b.entries);
  PART(cnt, int32_t, b.entries);
  PART(gidx, int32_t, b.slots);
  PART(hidx, int32_t, b.slots);
  PART(where, int32_t, picks);
  PART(off, int32_t, 3u * l->n_exp);
  PART(xg, uint32_t, b.entries);
  PART(yg, uint32_t, b.entries);
  PART(xd, uint32_t, b.entries);
  PART(yd, uint32_t, b.entries);
  PART(xe16, uint16_t, (uint64_t)b.slots * widest);
  PART(ga, float, (uint64_t)picks * l->ff);
  PART(up, float, (uint64_t)picks * l->ff);
  PART(y, float, (uint64_t)picks * l->dim);
  PART(overflow, int32_t, 1);
  if (mem)
    s->max_tok = max_tok, s->bounds = b;
  return at;
}

/* the tables' 32-bit offsets must hold: slots x the wider of dim and ff, in halves */
static bool q4x_fits32(const Q4xMoeLayer *l, uint32_t max_tok)
{
  Q4xExpertBounds b;
  q4x_expert_bounds(max_tok * l->k, l->n_exp, &b);
  const uint64_t widest = l->dim > l->ff ? l->dim : l->ff;
  return (uint64_t)max_tok * l->k <= 0x7FFFFFFFu && (uint64_t)b.slots * widest <= 0xFFFFFFFFu;
}

uint64_t q4x_moe_scratch_bytes(const Q4xMoeLayer *l, uint32_t max_tok)
{
  return q4x_layer_ok(l) && max_tok && q4x_fits32(l, max_tok) ? carve_q4x(l, max_tok, NULL, NULL) : 0;
}

bool q4x_moe_scratch_bind(const Q4xMoeLayer *l, uint32_t max_tok, void *mem, uint64_t bytes, Q4xMoeScratch *s)
{
  if (!q4x_layer_ok(l) || !max_tok || !q4x_fits32(l, max_tok) || !mem || !s || ((uintptr_t)mem & 255u) ||
      bytes < carve_q4x(l, max_tok, NULL, NULL))
    return false;
  carve_q4x(l, max_tok, (uint8_t *)mem, s);
  return true;
}

/* one expert tensor over the tables' runs of tile counts, a launch a run (hip_layers.c:317-329) */
static bool experts(uint32_t type, const void *const *ptr, const Q4xMoeScratch *s, const Q4xExpertBounds *bd, uint32_t rows,
                    uint32_t cols, const uint32_t *xo, float *y, const uint32_t *yo, void *stream)
{
  bool ok = true;
  for (int r = 0; ok && r < Q4X_TILE_RUNS; r++)
    if (bd->count[r])
    {
      const uint32_t at = bd->first[r];
      ok = mm_group(type, ptr + at, s->cnt + at, bd->count[r], (uint32_t)MM_TILE << r, rows, cols, s->xe16, xo + at, cols, y,
                    yo + at, rows, stream);
    }
  return ok;
}

bool q4x_moe(const Q4xMoeLayer *l, const Q4xMoeScratch *s, const float *x, const float *logits, const float *shared,
             const float *shared_logit, uint32_t n, float *out, void *stream)
{
  if (!q4x_layer_ok(l) || !s || !x || !logits || !shared || !shared_logit || !out || !n || n > s->max_tok || !s->ids || !s->rows ||
      !s->w || !s->ptr || !s->cnt || !s->gidx || !s->hidx || !s->where || !s->off || !s->xg || !s->yg || !s->xd || !s->yd ||
      !s->xe16 || !s->ga || !s->up || !s->y || !s->overflow || ((uintptr_t)x & 15u) || l->dim % 4)
    return false;
  const uint32_t picks = n * l->k, D = l->dim, FF = l->ff;
  Q4xExpertBounds bd;
  q4x_expert_bounds(picks, l->n_exp, &bd);
  if (bd.entries > s->bounds.entries || bd.slots > s->bounds.slots || bd.count[Q4X_TILE_RUNS - 1] > 65535u)
    return false;
  Q4xExpertTiles et;
  memset(&et, 0, sizeof et);
  et.cnt = s->cnt, et.gidx = s->gidx, et.hidx = s->hidx, et.xg = s->xg, et.yg = s->yg, et.xd = s->xd, et.yd = s->yd;
  et.where = s->where, et.off = s->off;
  for (int j = 0; j < Q4X_GROUP_TENSORS; j++)
    et.ptr[j] = s->ptr + (uint64_t)j * bd.entries, et.base[j] = l->base[j], et.bytes[j] = l->bytes[j], et.tab[j] = l->tab[j];
  /* each expert read once for up to 128 of the step's tokens that picked it */
  return q4x_route(logits, n, l->n_exp, l->k, s->ids, s->w, s->rows, stream) &&
         q4x_expert_tiles(s->ids, picks, l->k, l->n_exp, D, FF, &et, stream) &&
         mm_x16_rows(x, D, s->gidx, bd.slots, D, s->xe16, s->overflow, stream) &&
         experts(l->type[0], et.ptr[0], s, &bd, FF, D, s->xg, s->ga, s->yg, stream) &&
         experts(l->type[1], et.ptr[1], s, &bd, FF, D, s->xg, s->up, s->yg, stream) &&
         q4x_swiglu_rows(s->ga, s->up, FF, s->hidx, bd.slots, s->xe16, s->overflow, stream) &&
         experts(l->type[2], et.ptr[2], s, &bd, D, FF, s->xd, s->y, s->yd, stream) &&
         q4x_moe_sum(s->y, s->where, s->w, n, l->k, D, shared, shared_logit, out, stream);
}
