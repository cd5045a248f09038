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
    default: OTHERWISE;                            \
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
