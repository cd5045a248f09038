/* Whole-tensor dequantization of GGUF blocks on the GPU.
 *
 * Drop-in for the reference's include/osmos/gpu/quant.h:7-10 (quant_known, quant_dequant, quant_dequant_f16):
 * same names, argument meaning and refusals. Every value is the bits gguf-py's dequantize gives.
 * Every entry returns true when the work was queued on `stream` (a cudaStream_t, NULL = default stream; not
 * waited for) and false when it was refused - then nothing was queued.
 */
#ifndef OSMOS_B200_QUANT_H
#define OSMOS_B200_QUANT_H

#include <stdbool.h>
#include <stdint.h>

#include "osmos_b200/qtype.h"

#ifdef __cplusplus
extern "C" {
#endif

/* whether quant_dequant takes `type` (reference: include/osmos/gpu/quant.h:7) */
bool quant_known(uint32_t type);
/* `values` weights of `type` at src (device-readable GGUF blocks) as F32 into dst. false for an unknown type or
   values not whole blocks (reference: include/osmos/gpu/quant.h:8, kernels/quant.hip:96-121) */
bool quant_dequant(uint32_t type, const void *src, uint64_t values, float *dst, void *stream);
/* the same values rounded to f16 (nearest even), 2 bytes a value (reference: include/osmos/gpu/quant.h:9,
   kernels/quant.hip:123-147) */
bool quant_dequant_f16(uint32_t type, const void *src, uint64_t values, void *dst, void *stream);

#ifdef __cplusplus
}
#endif

#endif
