// run-time type id -> compile-time instantiation
#pragma once
#include "osmos_b200/qtype.h"

// every block type with a decoder
#define OSMOS_SWITCH_QUANT(type, CASE, OTHERWISE) \
  switch (type) {                                  \
    case QTYPE_Q4_0: CASE(QTYPE_Q4_0)              \
    case QTYPE_Q8_0: CASE(QTYPE_Q8_0)              \
    case QTYPE_Q2_K: CASE(QTYPE_Q2_K)              \
    case QTYPE_Q4_K: CASE(QTYPE_Q4_K)              \
    case QTYPE_IQ2_XXS: CASE(QTYPE_IQ2_XXS)        \
    case QTYPE_IQ2_XS: CASE(QTYPE_IQ2_XS)          \
    case QTYPE_IQ3_XXS: CASE(QTYPE_IQ3_XXS)        \
    case QTYPE_IQ1_S: CASE(QTYPE_IQ1_S)            \
    case QTYPE_IQ2_S: CASE(QTYPE_IQ2_S)            \
    case QTYPE_IQ1_M: CASE(QTYPE_IQ1_M)            \
    case QTYPE_MXFP4: CASE(QTYPE_MXFP4)            \
    case QTYPE_NVFP4: CASE(QTYPE_NVFP4)            \
    case QTYPE_Q5_1: CASE(QTYPE_Q5_1)              \
    case QTYPE_Q3_K: CASE(QTYPE_Q3_K)              \
    case QTYPE_Q5_K: CASE(QTYPE_Q5_K)              \
    case QTYPE_Q6_K: CASE(QTYPE_Q6_K)              \
    case QTYPE_IQ4_NL: CASE(QTYPE_IQ4_NL)          \
    case QTYPE_IQ4_XS: CASE(QTYPE_IQ4_XS)          \
    case QTYPE_Q2_0: CASE(QTYPE_Q2_0)              \
    case QTYPE_MXFP8: CASE(QTYPE_MXFP8)            \
    default: OTHERWISE;                            \
  }

// those and the unquantized weights a matvec may meet (a router's F32 matrix, BF16)
#define OSMOS_SWITCH_WEIGHTS(type, CASE, OTHERWISE)                     \
  switch (type) {                                                       \
    case QTYPE_F32: CASE(QTYPE_F32)                                     \
    case QTYPE_BF16: CASE(QTYPE_BF16)                                   \
    default: OSMOS_SWITCH_QUANT(type, CASE, OTHERWISE)                  \
  }

// the reference's int8 lane types (q8_group_tok, q8_gate_up)
#define OSMOS_SWITCH_LANE(type, CASE, OTHERWISE) \
  switch (type) {                                 \
    case QTYPE_Q2_K: CASE(QTYPE_Q2_K)             \
    case QTYPE_IQ2_XXS: CASE(QTYPE_IQ2_XXS)       \
    case QTYPE_IQ2_XS: CASE(QTYPE_IQ2_XS)         \
    case QTYPE_IQ3_XXS: CASE(QTYPE_IQ3_XXS)       \
    case QTYPE_IQ1_S: CASE(QTYPE_IQ1_S)           \
    case QTYPE_IQ2_S: CASE(QTYPE_IQ2_S)           \
    case QTYPE_IQ1_M: CASE(QTYPE_IQ1_M)           \
    default: OTHERWISE;                           \
  }

// the lane types and this library's extension of the lane order to plain 32-value blocks (q8_run)
#define OSMOS_SWITCH_LANE_EXT(type, CASE, OTHERWISE) \
  switch (type) {                                     \
    case QTYPE_Q4_0: CASE(QTYPE_Q4_0)                 \
    case QTYPE_Q8_0: CASE(QTYPE_Q8_0)                 \
    case QTYPE_Q2_K: CASE(QTYPE_Q2_K)                 \
    case QTYPE_IQ2_XXS: CASE(QTYPE_IQ2_XXS)           \
    case QTYPE_IQ2_XS: CASE(QTYPE_IQ2_XS)             \
    case QTYPE_IQ3_XXS: CASE(QTYPE_IQ3_XXS)           \
    case QTYPE_IQ1_S: CASE(QTYPE_IQ1_S)               \
    case QTYPE_IQ2_S: CASE(QTYPE_IQ2_S)               \
    case QTYPE_IQ1_M: CASE(QTYPE_IQ1_M)               \
    default: OTHERWISE;                               \
  }
