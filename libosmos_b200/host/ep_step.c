/* The expert-parallel layer step as one call: host code that only queues the six dependent launches of
 * include/osmos_b200/ep.h's fused step on the caller's stream. No counterpart in the reference (it is single-GPU);
 * the single-GPU layer is this step with one rank. Everything is checked before the first launch, so a refusal
 * leaves the stream untouched.
 */
#include <stddef.h>

#include "osmos_b200/ep.h"
#include "osmos_b200/q8.h"

bool ep_layer_step(const EpPlan *p, const float *x, const float *logits, const float *add, float *out, void *stream)
{
  if (!ep_plan_ok(p) || !x || !logits || !out || (((uintptr_t)out | (uintptr_t)add) & 15u))
    return false;
  const LaneLayer *l = &p->layer;
  const LaneScratch *s = &p->scratch;
  const uint32_t picks = p->n_tok * l->k;
  return ep_route_round_push(p, x, logits, stream) &&                     /* route, round, dispatch */
         ep_lane_tables(p, stream) &&                                     /* wait, tables, row homes */
         ep_gate_up(p, stream) &&                                         /* gate, up, activation */
         q8_round(s->hh, picks, l->ff, l->ff, s->hq, s->hqd, stream) &&   /* the activations to int8 */
         ep_down_push(p, stream) &&                                       /* down, rows to their homes */
         ep_combine_wait(p, add, out, stream);                            /* wait, ordered sum */
}
