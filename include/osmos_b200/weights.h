/* A layer's feed-forward tensors out of a model's GGUF: which tensor plays which part for the kernels of this library,
 * checked against each other before anything is loaded.
 *
 * The feed-forward rows of the reference's role table (src/model/weights.c:97-106, checked by its take(), :205-246):
 * the same tensor names under "blk.<layer>.", the same shapes (innermost dimension first, as the file stores them),
 * the same refusals in the same words - "missing", "of another shape", "of a type this role does not take", "not the
 * bytes of its type", "experts of unequal bytes". The reference checks the shapes against the model's metadata; here
 * they are checked against one another (the routed experts' gate gives hidden size, expert width and expert count),
 * so a layer can be taken from a file without the rest of the model's geometry. Everything else of the reference's
 * table (attention, norms outside the FFN, the model-specific extras) is outside this library's path.
 */
#ifndef OSMOS_B200_WEIGHTS_H
#define OSMOS_B200_WEIGHTS_H

#include <stdbool.h>
#include <stdint.h>

#include "osmos_b200/gguf.h"

#ifdef __cplusplus
extern "C" {
#endif

#define WEIGHTS_ERR 256

typedef struct FfnWeights
{
  /* required: the router's matrix [n_embd][n_experts] (any type the matvec reads) and the routed experts' three
     tensors, gate and up [n_embd][expert_ff][n_experts], down [expert_ff][n_embd][n_experts] (a type the expert
     kernels read: the int8 lane's, or mv_group_tok's) */
  const GgufTensor *router, *exp_gate, *exp_up, *exp_down;
  /* optional, NULL when absent: the FFN's norm [n_embd] F32, the router's bias [n_experts] F32, and the shared expert
     (all three or none): gate and up [n_embd][shared_ff], down [shared_ff][n_embd], a type the f16 product reads */
  const GgufTensor *ffn_norm, *router_bias, *sh_gate, *sh_up, *sh_down;
  uint32_t n_embd, expert_ff, n_experts, shared_ff; /* shared_ff 0: no shared expert */
  uint64_t expert_bytes[3];                          /* one expert's bytes in gate, up, down: expert e's matrix is at
                                                        the tensor's offset + e * expert_bytes[j] of its file */
} FfnWeights;

/* layer `layer`'s feed-forward tensors of g. false - *out untouched beyond zeroing, the tensor's name and the reason in
   err - when a required one is missing, when one is of another shape or type than its part takes, when a tensor's
   bytes are not its type's for its shape, or when an expert tensor does not split into experts of equal bytes. */
bool weights_ffn(const Gguf *g, int layer, FfnWeights *out, char err[WEIGHTS_ERR]);

#ifdef __cplusplus
}
#endif

#endif
