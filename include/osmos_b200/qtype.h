/* GGUF quantization types this library reads, by their ggml type ids.
 *
 * Replaces (same ids, same block sizes) the reference's type table
 * include/osmos/model/qtype.h:28-84 for the types on the quantized-weight matrix path.
 * A "block" is the unit a GGUF tensor row is made of: `values` weights stored in `bytes` bytes.
 */
#ifndef OSMOS_B200_QTYPE_H
#define OSMOS_B200_QTYPE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum OsmosQType
{
  QTYPE_F32 = 0,
  QTYPE_Q4_0 = 2,
  QTYPE_Q5_1 = 7,
  QTYPE_Q8_0 = 8,
  QTYPE_Q2_K = 10,
  QTYPE_Q3_K = 11,
  QTYPE_Q4_K = 12,
  QTYPE_Q5_K = 13,
  QTYPE_Q6_K = 14,
  QTYPE_IQ2_XXS = 16,
  QTYPE_IQ2_XS = 17,
  QTYPE_IQ3_XXS = 18,
  QTYPE_IQ1_S = 19,
  QTYPE_IQ4_NL = 20,
  QTYPE_IQ2_S = 22,
  QTYPE_IQ4_XS = 23,
  QTYPE_IQ1_M = 29,
  QTYPE_BF16 = 30,
  QTYPE_MXFP4 = 39,
  QTYPE_NVFP4 = 40,
  QTYPE_Q2_0 = 42,
  QTYPE_MXFP8 = 43
};

/* which entry points take a type */
#define QTYPE_PATH_DECODE (1u << 1) /* quant_dequant */
#define QTYPE_PATH_MV (1u << 2)     /* mv_run, mv_strided, mv_group */
#define QTYPE_PATH_MV_TOK (1u << 3) /* mv_group_tok */
#define QTYPE_PATH_Q8 (1u << 5)     /* q8_group_tok, q8_gate_up: the reference's int8 lane types */
#define QTYPE_PATH_Q8_EXT (1u << 9) /* q8_run only: int8 lane order extended by this library (no reference path) */
#define QTYPE_PATH_MMQ (1u << 10)   /* mmq_group */

typedef struct OsmosQTypeInfo
{
  uint32_t id;     /* ggml type id */
  uint32_t values; /* weights in a block */
  uint32_t bytes;  /* bytes in a block */
  uint32_t paths;  /* QTYPE_PATH_* */
  const char *name;
} OsmosQTypeInfo;

/* the row for a ggml type id, or NULL for a type this library does not read
   (reference: qtype_info, include/osmos/model/qtype.h:73) */
const OsmosQTypeInfo *qtype_info(uint32_t id);
/* bytes of a row-major tensor of rows x cols values, or 0 for an unknown type or cols not whole blocks */
uint64_t qtype_tensor_bytes(uint32_t id, uint64_t rows, uint64_t cols);

/* one definition of the table for every translation unit that wants it inline (kernels, oracle) */
#define OSMOS_QTYPE_TABLE(X)                                                                                   \
  X(F32, 0, 1, 4, QTYPE_PATH_MV)                                                                               \
  X(Q4_0, 2, 32, 18, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8_EXT)                \
  X(Q5_1, 7, 32, 24, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                    \
  X(Q8_0, 8, 32, 34, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8_EXT)                \
  X(Q2_K, 10, 256, 84, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8)                  \
  X(Q3_K, 11, 256, 110, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                 \
  X(Q4_K, 12, 256, 144, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_MMQ)                \
  X(Q5_K, 13, 256, 176, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                 \
  X(Q6_K, 14, 256, 210, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                 \
  X(IQ2_XXS, 16, 256, 66, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8)               \
  X(IQ2_XS, 17, 256, 74, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8)                \
  X(IQ3_XXS, 18, 256, 98, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8)               \
  X(IQ1_S, 19, 256, 50, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8)                 \
  X(IQ4_NL, 20, 32, 18, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                 \
  X(IQ2_S, 22, 256, 82, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8)                 \
  X(IQ4_XS, 23, 256, 136, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                               \
  X(IQ1_M, 29, 256, 56, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK | QTYPE_PATH_Q8)                 \
  X(BF16, 30, 1, 2, QTYPE_PATH_DECODE | QTYPE_PATH_MV)                                                         \
  X(MXFP4, 39, 32, 17, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                  \
  X(NVFP4, 40, 64, 36, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                  \
  X(Q2_0, 42, 64, 18, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)                                   \
  X(MXFP8, 43, 32, 33, QTYPE_PATH_DECODE | QTYPE_PATH_MV | QTYPE_PATH_MV_TOK)

#ifdef __cplusplus
}
#endif

#endif
