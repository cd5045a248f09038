/* A layer's feed-forward tensors and their checks (include/osmos_b200/weights.h): plain C over the GGUF reader and the
 * type table. Nothing is read from the files here - only the header's records are compared. */
#include <stdio.h>
#include <string.h>

#include "osmos_b200/qtype.h"
#include "osmos_b200/weights.h"

/* what a part asks of its tensor's type */
typedef enum Kind
{
  RAW_F32, /* F32 as stored */
  MATVEC,  /* any type mv_run reads (the router's projection) */
  PRODUCT, /* a block type the f16 product decodes (the shared expert) */
  EXPERTS  /* the int8 lane's types, or mv_group_tok's (the routed experts) */
} Kind;

static bool takes(Kind kind, uint32_t type)
{
  const OsmosQTypeInfo *t = qtype_info(type);
  if (!t)
    return false;
  switch (kind)
  {
  case RAW_F32: return type == QTYPE_F32;
  case MATVEC: return (t->paths & QTYPE_PATH_MV) != 0;
  case PRODUCT: return (t->paths & QTYPE_PATH_DECODE) != 0;
  default: return (t->paths & (QTYPE_PATH_Q8 | QTYPE_PATH_MV_TOK)) != 0;
  }
}

static bool fail(char *err, const char *name, const char *why)
{
  snprintf(err, WEIGHTS_ERR, "%s: %s", name, why);
  return false;
}

/* blk.<layer>.<part> of n_dims dimensions `dims` (0: any size - the caller learns it from this tensor), a type the
   part takes, the bytes its type gives its shape; an optional part may be absent (*field NULL then) */
static bool take(const Gguf *g, int layer, const char *part, Kind kind, uint32_t n_dims, const uint64_t *dims, bool optional,
                 const GgufTensor **field, char *err)
{
  char name[96];
  snprintf(name, sizeof name, "blk.%d.%s", layer, part);
  const GgufTensor *t = gguf_tensor(g, name);
  *field = NULL;
  if (!t)
    return optional || fail(err, name, "missing");
  if (t->n_dims != n_dims)
    return fail(err, name, "of another shape");
  uint64_t values = 1;
  for (uint32_t i = 0; i < n_dims; i++)
  {
    if (!t->dims[i] || (dims[i] && t->dims[i] != dims[i]) || values > UINT64_MAX / t->dims[i])
      return fail(err, name, "of another shape");
    values *= t->dims[i];
  }
  if (!takes(kind, t->type))
    return fail(err, name, "of a type this role does not take");
  if (t->bytes != gguf_bytes(t->type, values))
    return fail(err, name, "not the bytes of its type");
  if (kind == EXPERTS && t->bytes % t->dims[2])
    return fail(err, name, "experts of unequal bytes");
  *field = t;
  return true;
}

bool weights_ffn(const Gguf *g, int layer, FfnWeights *out, char err[WEIGHTS_ERR])
{
  char none[WEIGHTS_ERR];
  if (!err)
    err = none;
  err[0] = 0;
  if (!g || !out || layer < 0)
    return fail(err, "weights_ffn", "no model, no place for the result, or a negative layer");
  FfnWeights w;
  memset(&w, 0, sizeof w);
  memset(out, 0, sizeof *out);
  /* the experts' gate says what the layer's sizes are; every other tensor must agree with it */
  const uint64_t any3[3] = {0, 0, 0};
  if (!take(g, layer, "ffn_gate_exps.weight", EXPERTS, 3, any3, false, &w.exp_gate, err))
    return false;
  const uint64_t D = w.exp_gate->dims[0], FF = w.exp_gate->dims[1], E = w.exp_gate->dims[2];
  if (D > UINT32_MAX || FF > UINT32_MAX || E > UINT32_MAX)
    return fail(err, w.exp_gate->name, "of another shape");
  const uint64_t up3[3] = {D, FF, E}, down3[3] = {FF, D, E}, router2[2] = {D, E}, embd1[1] = {D}, experts1[1] = {E};
  if (!take(g, layer, "ffn_up_exps.weight", EXPERTS, 3, up3, false, &w.exp_up, err) ||
      !take(g, layer, "ffn_down_exps.weight", EXPERTS, 3, down3, false, &w.exp_down, err) ||
      !take(g, layer, "ffn_gate_inp.weight", MATVEC, 2, router2, false, &w.router, err) ||
      !take(g, layer, "ffn_norm.weight", RAW_F32, 1, embd1, true, &w.ffn_norm, err) ||
      !take(g, layer, "exp_probs_b.bias", RAW_F32, 1, experts1, true, &w.router_bias, err))
    return false;
  /* the shared expert: all three or none, its width its own */
  const uint64_t gate2[2] = {D, 0};
  if (!take(g, layer, "ffn_gate_shexp.weight", PRODUCT, 2, gate2, true, &w.sh_gate, err))
    return false;
  const uint64_t SF = w.sh_gate ? w.sh_gate->dims[1] : 0;
  if (SF > UINT32_MAX)
    return fail(err, w.sh_gate->name, "of another shape");
  const uint64_t shup2[2] = {D, SF}, shdown2[2] = {SF, D}, any2[2] = {0, 0};
  if (!take(g, layer, "ffn_up_shexp.weight", PRODUCT, 2, w.sh_gate ? shup2 : any2, true, &w.sh_up, err) ||
      !take(g, layer, "ffn_down_shexp.weight", PRODUCT, 2, w.sh_gate ? shdown2 : any2, true, &w.sh_down, err))
    return false;
  if (!w.sh_gate != !w.sh_up || !w.sh_gate != !w.sh_down)
  {
    char name[96];
    snprintf(name, sizeof name, "blk.%d.ffn_%s_shexp.weight", layer, !w.sh_gate ? "gate" : !w.sh_up ? "up" : "down");
    return fail(err, name, "missing");
  }
  w.n_embd = (uint32_t)D, w.expert_ff = (uint32_t)FF, w.n_experts = (uint32_t)E, w.shared_ff = (uint32_t)SF;
  w.expert_bytes[0] = w.exp_gate->bytes / E, w.expert_bytes[1] = w.exp_up->bytes / E, w.expert_bytes[2] = w.exp_down->bytes / E;
  *out = w;
  return true;
}
