/* CPU oracle for the quantized-weight matrix path - TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain scalar C restatement of the arithmetic the CUDA kernels must reproduce. Only the test suite, the
 * smoke check and the benchmark's CPU-baseline leg may load this file's library; the product never does and
 * has no CPU fallback.
 *
 * Parity pin: every block decoder here is checked bit-for-bit against gguf-py's dequantize on committed golden
 * blocks (tests/golden/dequant_*.npz), and the int8 "lane" sums, the F32 matvec and the expert FFN are checked
 * bit-for-bit against the reference's own CPU lane (src/cpu/q8.c, src/cpu/expert.c, src/cpu/lane.c compiled
 * unmodified into oracle/_ref) on committed golden inputs/outputs (tests/golden/lane_*.npz) and live where
 * that library is present.
 *
 * Build with -ffp-contract=off: every product and sum below is rounded where it is written; the only fused
 * operations are the explicit fmaf calls (the reference builds the same way, Makefile:82 and cuda.mk:18).
 *
 * Each function cites the reference lines it follows (paths inside the reference tree).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "osmos_b200/qtype.h"
#include "osmos_grids.h"

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------------------
 * the type table (include/osmos/model/qtype.h:29-53)
 * ---------------------------------------------------------------------------------------------------------- */
#define ORC_ROW(name, id, values, bytes, paths) {id, values, bytes, paths, #name},
static const OsmosQTypeInfo kTypes[] = {OSMOS_QTYPE_TABLE(ORC_ROW)};
#undef ORC_ROW

static const OsmosQTypeInfo *type_row(uint32_t id)
{
  for (size_t i = 0; i < sizeof kTypes / sizeof kTypes[0]; i++)
    if (kTypes[i].id == id)
      return &kTypes[i];
  return NULL;
}

ORC_API int orc_block_values(uint32_t type) { const OsmosQTypeInfo *t = type_row(type); return t ? (int)t->values : 0; }
ORC_API int orc_block_bytes(uint32_t type) { const OsmosQTypeInfo *t = type_row(type); return t ? (int)t->bytes : 0; }

/* ------------------------------------------------------------------------------------------------------------
 * small readers
 * ---------------------------------------------------------------------------------------------------------- */
static uint32_t rd16(const uint8_t *p) { return (uint32_t)p[0] | (uint32_t)p[1] << 8; }
static uint32_t rd32(const uint8_t *p) { return rd16(p) | rd16(p + 2) << 16; }
static uint64_t rd64(const uint8_t *p) { return (uint64_t)rd32(p) | (uint64_t)rd32(p + 4) << 32; }
static float half_value(uint32_t bits)
{
  const uint16_t b = (uint16_t)bits;
  _Float16 h;
  memcpy(&h, &b, sizeof h);
  return (float)h;
}
static uint16_t half_bits(float v)
{
  const _Float16 h = (_Float16)v; /* round to nearest even */
  uint16_t b;
  memcpy(&b, &h, sizeof b);
  return b;
}

/* Q4_K's packed 6-bit (scale, min) of sub-block g out of its 12 scale bytes (kernels/quant.h:96-99) */
static void q4k_scale_min(const uint8_t *s, int g, int *sc, int *mn)
{
  if (g < 4)
    *sc = s[g] & 0x3F, *mn = s[g + 4] & 0x3F;
  else
    *sc = (s[g + 4] & 0x0F) | ((s[g - 4] >> 6) << 4), *mn = (s[g + 4] >> 4) | ((s[g] >> 6) << 4);
}

/* IQ1_M's f16 block scale, spread over the top nibbles of its four 16-bit scale words (kernels/quant.h:337-340) */
static float iq1m_d(const uint8_t *b)
{
  const uint32_t s0 = rd16(b + 48), s1 = rd16(b + 50), s2 = rd16(b + 52), s3 = rd16(b + 54);
  return half_value((s0 >> 12) | ((s1 >> 8) & 0x00F0) | ((s2 >> 4) & 0x0F00) | (s3 & 0xF000));
}

/* E4M3 scale as ggml reads an NVFP4 block's (kernels/round.h:99-117): the byte 0x7F reads as zero, any other
   byte without its sign bit (so 0xFF is 480) */
static float ue4m3_value(uint32_t c)
{
  const uint32_t mag = c & 0x7F;
  if (c == 0x7F)
    return 0.0f;
  if (mag >> 3)
    return ldexpf(1.0f + (float)(mag & 7) * 0.125f, (int)(mag >> 3) - 7);
  return (float)mag * 0.001953125f; /* subnormals: m * 2^-9 */
}

/* ------------------------------------------------------------------------------------------------------------
 * block decoders: all `values` weights of one block as F32, each the bits gguf-py's dequantize gives
 * (kernels/quant.h:65-362; every product is its own rounding)
 * ---------------------------------------------------------------------------------------------------------- */
static void signed_grid8(uint64_t grid, uint32_t signs, float scale, float *out)
{
  for (int j = 0; j < 8; j++)
  {
    const float v = scale * (float)(uint8_t)(grid >> (8 * j));
    out[j] = (signs >> j) & 1 ? -v : v;
  }
}

static void decode_block(uint32_t type, const uint8_t *b, float *out)
{
  switch (type)
  {
  case QTYPE_Q4_0: /* kernels/quant.h:244-248 */
  {
    const float d = half_value(rd16(b));
    for (int j = 0; j < 16; j++)
    {
      out[j] = d * (float)((int)(b[2 + j] & 0x0F) - 8);
      out[16 + j] = d * (float)((int)(b[2 + j] >> 4) - 8);
    }
    break;
  }
  case QTYPE_Q8_0: /* kernels/quant.h:68-71 */
  {
    const float d = half_value(rd16(b));
    for (int j = 0; j < 32; j++)
      out[j] = (float)(int8_t)b[2 + j] * d;
    break;
  }
  case QTYPE_Q4_K: /* kernels/quant.h:93-103 */
  {
    const float d = half_value(rd16(b)), dmin = half_value(rd16(b + 2));
    for (int g = 0; g < 8; g++)
    {
      int sc, mn;
      q4k_scale_min(b + 4, g, &sc, &mn);
      const float ds = d * (float)sc, dm = dmin * (float)mn;
      for (int i = 0; i < 32; i++)
      {
        const int q = (b[16 + (g / 2) * 32 + i] >> (4 * (g % 2))) & 0x0F;
        out[g * 32 + i] = ds * (float)q - dm;
      }
    }
    break;
  }
  case QTYPE_Q2_K: /* kernels/quant.h:262-268 */
  {
    const float d = half_value(rd16(b + 80)), dmin = half_value(rd16(b + 82));
    for (int i = 0; i < 256; i++)
    {
      const int g = i / 16;
      const float dl = d * (float)(b[g] & 0x0F), ml = dmin * (float)(b[g] >> 4);
      const int q = (b[16 + 32 * (i / 128) + i % 32] >> (2 * ((i % 128) / 32))) & 0x03;
      out[i] = dl * (float)q - ml;
    }
    break;
  }
  case QTYPE_IQ2_XXS: /* kernels/quant.h:187-198 */
  {
    const float d = half_value(rd16(b));
    for (int g = 0; g < 8; g++)
    {
      const uint8_t *q = b + 2 + 8 * g;
      const uint32_t aux = rd32(q + 4);
      const float db = (d * (0.5f + (float)(aux >> 28))) * 0.25f;
      for (int k = 0; k < 4; k++)
        signed_grid8(osmos_grid_iq2xxs[q[k]], osmos_ksigns[(aux >> (7 * k)) & 0x7F], db, out + g * 32 + k * 8);
    }
    break;
  }
  case QTYPE_IQ2_XS: /* kernels/quant.h:201-212 */
  {
    const float d = half_value(rd16(b));
    for (int k = 0; k < 32; k++)
    {
      const uint32_t q = rd16(b + 2 + 2 * k);
      const int s = (b[66 + k / 4] >> (4 * ((k / 2) % 2))) & 0x0F;
      const float db = (d * (0.5f + (float)s)) * 0.25f;
      signed_grid8(osmos_grid_iq2xs[q & 511], osmos_ksigns[q >> 9], db, out + k * 8);
    }
    break;
  }
  case QTYPE_IQ2_S: /* kernels/quant.h:316-326 */
  {
    const float d = half_value(rd16(b));
    for (int k = 0; k < 32; k++)
    {
      const int s = (b[74 + k / 4] >> (4 * ((k / 2) % 2))) & 0x0F;
      const float db = (d * (0.5f + (float)s)) * 0.25f;
      const uint32_t idx = b[2 + k] | ((b[66 + k / 4] >> (2 * (k % 4))) & 0x03) << 8;
      signed_grid8(osmos_grid_iq2s[idx], b[34 + k], db, out + k * 8);
    }
    break;
  }
  case QTYPE_IQ3_XXS: /* kernels/quant.h:221-231 */
  {
    const float d = half_value(rd16(b));
    for (int g = 0; g < 8; g++)
    {
      const uint32_t aux = rd32(b + 66 + 4 * g);
      const float db = (d * (0.5f + (float)(aux >> 28))) * 0.5f;
      for (int k = 0; k < 4; k++)
      {
        const uint8_t *q = b + 2 + 8 * g + 2 * k;
        const uint64_t grid = (uint64_t)osmos_grid_iq3xxs[q[0]] | (uint64_t)osmos_grid_iq3xxs[q[1]] << 32;
        signed_grid8(grid, osmos_ksigns[(aux >> (7 * k)) & 0x7F], db, out + g * 32 + k * 8);
      }
    }
    break;
  }
  case QTYPE_IQ1_S: /* kernels/quant.h:328-334 */
  {
    const float d = half_value(rd16(b));
    for (int k = 0; k < 32; k++)
    {
      const uint32_t h = rd16(b + 34 + 2 * (k / 4));
      const float dl = d * (float)(2 * (int)((h >> 12) & 0x07) + 1);
      const float delta = h & 0x8000 ? -0.125f : 0.125f;
      const uint64_t grid = osmos_grid_iq1s[b[2 + k] | ((h >> (3 * (k % 4))) & 0x07) << 8];
      for (int j = 0; j < 8; j++)
        out[k * 8 + j] = dl * ((float)(int8_t)(grid >> (8 * j)) + delta);
    }
    break;
  }
  case QTYPE_IQ1_M: /* kernels/quant.h:335-349 */
  {
    const float d = iq1m_d(b);
    const uint64_t sc = rd64(b + 48);
    for (int k = 0; k < 32; k++)
    {
      const int s = (int)((sc >> (16 * (k / 8) + 3 * ((k / 2) % 4))) & 0x07);
      const float dl = d * (float)(2 * s + 1);
      const uint32_t h = (b[32 + k / 2] >> (4 * (k % 2))) & 0x0F;
      const float delta = h & 0x08 ? -0.125f : 0.125f;
      const uint64_t grid = osmos_grid_iq1s[b[k] | (h & 0x07) << 8];
      for (int j = 0; j < 8; j++)
        out[k * 8 + j] = dl * ((float)(int8_t)(grid >> (8 * j)) + delta);
    }
    break;
  }
  case QTYPE_MXFP4: /* kernels/quant.h:289-293: E2M1 doubled times 2^(e-128) */
  {
    const float d = ldexpf(1.0f, (int)b[0] - 128);
    for (int j = 0; j < 16; j++)
    {
      out[j] = d * (float)osmos_e2m1_doubled[b[1 + j] & 0x0F];
      out[16 + j] = d * (float)osmos_e2m1_doubled[b[1 + j] >> 4];
    }
    break;
  }
  case QTYPE_NVFP4: /* kernels/quant.h:300-304: four UE4M3 scales, one a 16 values */
  {
    for (int s = 0; s < 4; s++)
    {
      const float d = ue4m3_value(b[s]) * 0.5f;
      for (int j = 0; j < 8; j++)
      {
        out[16 * s + j] = d * (float)osmos_e2m1_doubled[b[4 + 8 * s + j] & 0x0F];
        out[16 * s + 8 + j] = d * (float)osmos_e2m1_doubled[b[4 + 8 * s + j] >> 4];
      }
    }
    break;
  }
  case QTYPE_Q5_1: /* kernels/quant.h:108-116: d q + m, q a nibble and a fifth bit (value i: bit i of the word at 4) */
  {
    const float d = half_value(rd16(b)), m = half_value(rd16(b + 2));
    const uint32_t qh = (uint32_t)rd16(b + 4) | (uint32_t)rd16(b + 6) << 16;
    for (int i = 0; i < 32; i++)
    {
      const int nib = i < 16 ? b[8 + i] & 0x0F : b[8 + i - 16] >> 4;
      out[i] = d * (float)(nib | (int)((qh >> i) & 1) << 4) + m;
    }
    break;
  }
  case QTYPE_Q5_K: /* kernels/quant.h:75-90: Q4_K's scales; q a nibble of the 128 bytes at 48 and bit g of byte i % 32 at 16 */
  {
    const float d = half_value(rd16(b)), dmin = half_value(rd16(b + 2));
    for (int i = 0; i < 256; i++)
    {
      const int g = i / 32, l = i % 32;
      int sc, mn;
      q4k_scale_min(b + 4, g, &sc, &mn);
      const int q = ((b[48 + (g / 2) * 32 + l] >> (4 * (g % 2))) & 0x0F) | ((b[16 + l] >> g) & 1) << 4;
      out[i] = (d * (float)sc) * (float)q - dmin * (float)mn;
    }
    break;
  }
  case QTYPE_Q6_K: /* kernels/quant.h:170-183: (d sc) (q - 32), sixteen int8 scales at 192, d at 208 */
  {
    const float d = half_value(rd16(b + 208));
    for (int i = 0; i < 256; i++)
    {
      const int h = i / 128, r = (i % 128) / 32, l = i % 32;
      const int lo = (b[h * 64 + (r % 2) * 32 + l] >> (4 * (r / 2))) & 0x0F, hi = (b[128 + h * 32 + l] >> (2 * r)) & 0x03;
      out[i] = (d * (float)(int8_t)b[192 + i / 16]) * (float)((lo | hi << 4) - 32);
    }
    break;
  }
  case QTYPE_Q3_K: /* kernels/quant.h:270-287: (d (sc - 32)) (q - (high bit ? 0 : 4)) */
  {
    const float d = half_value(rd16(b + 108));
    for (int i = 0; i < 256; i++)
    {
      const int n = i / 128, j = (i % 128) / 32, l = i % 32, g = i / 16;
      const int low = g < 8 ? b[96 + g] & 0x0F : b[96 + g - 8] >> 4;
      const int sc = (low | ((b[104 + g % 4] >> (2 * (g / 4))) & 0x03) << 4) - 32;
      const int q = ((b[32 + 32 * n + l] >> (2 * j)) & 0x03) - ((b[l] >> (4 * n + j)) & 1 ? 0 : 4);
      out[i] = (d * (float)sc) * (float)q;
    }
    break;
  }
  case QTYPE_IQ4_NL: /* kernels/quant.h:214-219: d times the table's value, Q4_0's nibble order */
  {
    const float d = half_value(rd16(b));
    for (int i = 0; i < 32; i++)
      out[i] = d * (float)osmos_iq4nl_values[i < 16 ? b[2 + i] & 0x0F : b[2 + i - 16] >> 4];
    break;
  }
  case QTYPE_IQ4_XS: /* kernels/quant.h:233-241: (d (ls - 32)) times the table's value, a 6-bit ls a 32 values */
  {
    const float d = half_value(rd16(b));
    const uint32_t top = rd16(b + 2);
    for (int i = 0; i < 256; i++)
    {
      const int g = i / 32, l = i % 32;
      const int ls = ((b[4 + g / 2] >> (4 * (g % 2))) & 0x0F) | (int)((top >> (2 * g)) & 0x03) << 4;
      const int nib = l < 16 ? b[8 + 16 * g + l] & 0x0F : b[8 + 16 * g + l - 16] >> 4;
      out[i] = (d * (float)(ls - 32)) * (float)osmos_iq4nl_values[nib];
    }
    break;
  }
  case QTYPE_Q2_0: /* kernels/quant.h:252-256: d (code - 1), value i bits 2 (i % 4) of byte 2 + i / 4 */
  {
    const float d = half_value(rd16(b));
    for (int i = 0; i < 64; i++)
      out[i] = d * (float)(((b[2 + i / 4] >> (2 * (i % 4))) & 0x03) - 1);
    break;
  }
  case QTYPE_MXFP8: /* kernels/quant.h:308-311: 2^(e - 127) times an E4M3 value (0x7F / 0xFF are NaN) */
  {
    const float d = ldexpf(1.0f, (int)b[0] - 127);
    for (int i = 0; i < 32; i++)
    {
      const uint32_t c = b[1 + i], mag = c & 0x7F;
      float v = (mag >> 3) ? ldexpf(1.0f + (float)(mag & 7) * 0.125f, (int)(mag >> 3) - 7) : (float)mag * 0.001953125f;
      if (mag == 0x7F)
        v = NAN;
      out[i] = d * (c & 0x80 ? -v : v);
    }
    break;
  }
  case QTYPE_F32: /* kernels/quant.h:357-359 */
    memcpy(out, b, 4);
    break;
  case QTYPE_BF16: /* kernels/quant.h:352-354: the top half of an F32 */
  {
    const uint32_t bits = (uint32_t)rd16(b) << 16;
    memcpy(out, &bits, 4);
    break;
  }
  default:
    break;
  }
}

/* quant_dequant's result (kernels/quant.hip:96-121): `values` weights at src as F32; 0 on a refusal */
ORC_API int orc_dequant(uint32_t type, const void *src, uint64_t values, float *dst)
{
  const OsmosQTypeInfo *t = type_row(type);
  if (!t || !(t->paths & (QTYPE_PATH_DECODE | QTYPE_PATH_MV)) || !values || values % t->values)
    return 0;
  const uint64_t nb = values / t->values;
  for (uint64_t i = 0; i < nb; i++)
    decode_block(type, (const uint8_t *)src + i * t->bytes, dst + i * t->values);
  return 1;
}

/* ------------------------------------------------------------------------------------------------------------
 * the F32-activation matvec (kernels/mv.h:14-70): a row's 8-value chunks dealt to 32 lanes (chunk c to lane
 * c % 32), each lane one fmaf chain over its chunks in order, value by value, then the xor tree 16, 8, 4, 2, 1
 * ---------------------------------------------------------------------------------------------------------- */
static float xor_tree(float *s, int lanes)
{
  float nx[32];
  for (int o = lanes / 2; o > 0; o >>= 1)
  {
    for (int l = 0; l < lanes; l++)
      nx[l] = s[l] + s[l ^ o];
    memcpy(s, nx, (size_t)lanes * sizeof *s);
  }
  return s[0];
}

ORC_API int orc_mv_rows(uint32_t type, const void *w, uint32_t cols, uint32_t r0, uint32_t r1, const float *x,
                        uint32_t xs, uint32_t n_tok, float *y, uint32_t ys)
{
  const OsmosQTypeInfo *t = type_row(type);
  if (!t || !(t->paths & QTYPE_PATH_MV) || r1 < r0 || !cols || cols % t->values || cols % 8 ||
      !n_tok || xs < cols)
    return 0;
  const uint64_t row_bytes = (uint64_t)(cols / t->values) * t->bytes;
  for (uint32_t r = r0; r < r1; r++)
  {
    float *vals = malloc((size_t)cols * sizeof *vals);
    const uint8_t *row = (const uint8_t *)w + r * row_bytes;
    for (uint32_t b = 0; b < cols / t->values; b++)
      decode_block(type, row + (uint64_t)b * t->bytes, vals + (uint64_t)b * t->values);
    for (uint32_t tk = 0; tk < n_tok; tk++)
    {
      const float *xt = x + (uint64_t)tk * xs;
      float lane[32] = {0};
      for (uint32_t c = 0; c < cols / 8; c++)
      {
        float s = lane[c % 32];
        for (int j = 0; j < 8; j++)
          s = fmaf(vals[c * 8 + j], xt[c * 8 + j], s);
        lane[c % 32] = s;
      }
      y[(uint64_t)tk * ys + r] = xor_tree(lane, 32);
    }
    free(vals);
  }
  return 1;
}

/* ------------------------------------------------------------------------------------------------------------
 * the int8 lane (kernels/lane.h:43-66, kernels/q8.h:28-212)
 * ---------------------------------------------------------------------------------------------------------- */

/* q8_round (kernels/q8.h:265-277, lane.h:54-56): per 32 values q = rint(x * (127 / amax)), d = amax / 127 */
ORC_API int orc_q8_round(const float *x, uint32_t rows, uint32_t cols, uint32_t xs, int8_t *q, float *d)
{
  if (!rows || !cols || cols % 32 || xs < cols)
    return 0;
  for (uint32_t r = 0; r < rows; r++)
    for (uint32_t s = 0; s < cols / 32; s++)
    {
      const float *v = x + (uint64_t)r * xs + (uint64_t)s * 32;
      float amax = 0.0f;
      for (int i = 0; i < 32; i++)
        amax = fmaxf(amax, fabsf(v[i]));
      const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
      for (int i = 0; i < 32; i++)
        q[(uint64_t)r * cols + (uint64_t)s * 32 + i] = (int8_t)(int)rintf(v[i] * inv);
      d[(uint64_t)r * (cols / 32) + s] = amax / 127.0f;
    }
  return 1;
}

/* ggml's Q8_0 activation rounding (kernels/block.h:88-96): d = amax / 127, q = roundf(x * (1 / d)) - halves away
   from zero - and the scale kept as the f16 nearest d; returned here as that f16's F32 value */
ORC_API int orc_q8_0_round(const float *x, uint32_t rows, uint32_t cols, uint32_t xs, int8_t *q, float *d)
{
  if (!rows || !cols || cols % 32 || xs < cols)
    return 0;
  for (uint32_t r = 0; r < rows; r++)
    for (uint32_t s = 0; s < cols / 32; s++)
    {
      const float *v = x + (uint64_t)r * xs + (uint64_t)s * 32;
      float amax = 0.0f;
      for (int i = 0; i < 32; i++)
        amax = fmaxf(amax, fabsf(v[i]));
      const float dd = amax / 127.0f, id = dd ? 1.0f / dd : 0.0f;
      for (int i = 0; i < 32; i++)
        q[(uint64_t)r * cols + (uint64_t)s * 32 + i] = (int8_t)roundf(v[i] * id);
      d[(uint64_t)r * (cols / 32) + s] = half_value(half_bits(dd));
    }
  return 1;
}

/* a 32-value weight sub-block as the lane sees it (kernels/q8.h:32-128): integer codes, per-half 2s+1 factors,
   IQ1's per-chunk delta sign, the block scale; Q2_K's minimum terms */
typedef struct
{
  int code[32];
  int delta[4]; /* 0, or +-1: IQ1 weights are 8 * grid + delta in eighths */
  int s21[2];
  float d;
  int m8[2];
  float dmin;
  int plain; /* 1: extension types - one scale, no eighths: block = d * isum */
} LaneBlock;

static void grid_signed(uint64_t grid, uint32_t signs, int *code)
{
  for (int i = 0; i < 8; i++)
  {
    const int v = (int)(uint8_t)(grid >> (8 * i));
    code[i] = (signs >> i) & 1 ? -v : v;
  }
}

static int lane_block(uint32_t type, const uint8_t *b, int j, LaneBlock *o)
{
  memset(o, 0, sizeof *o);
  switch (type)
  {
  case QTYPE_IQ2_XXS: /* q8.h:46-55 */
  {
    const uint8_t *q = b + 2 + 8 * j;
    const uint32_t aux = rd32(q + 4);
    for (int k = 0; k < 4; k++)
      grid_signed(osmos_grid_iq2xxs[q[k]], osmos_ksigns[(aux >> (7 * k)) & 0x7F], o->code + 8 * k);
    o->s21[0] = o->s21[1] = 2 * (int)(aux >> 28) + 1;
    o->d = half_value(rd16(b));
    return 1;
  }
  case QTYPE_IQ2_XS: /* q8.h:57-66 */
  {
    for (int k = 0; k < 4; k++)
    {
      const uint32_t q = rd16(b + 2 + 2 * (4 * j + k));
      grid_signed(osmos_grid_iq2xs[q & 511], osmos_ksigns[q >> 9], o->code + 8 * k);
    }
    o->s21[0] = 2 * (int)(b[66 + j] & 0x0F) + 1, o->s21[1] = 2 * (int)(b[66 + j] >> 4) + 1;
    o->d = half_value(rd16(b));
    return 1;
  }
  case QTYPE_IQ2_S: /* q8.h:86-95 */
  {
    for (int k = 0; k < 4; k++)
    {
      const int kk = 4 * j + k;
      grid_signed(osmos_grid_iq2s[b[2 + kk] | ((b[66 + j] >> (2 * k)) & 0x03) << 8], b[34 + kk], o->code + 8 * k);
    }
    o->s21[0] = 2 * (int)(b[74 + j] & 0x0F) + 1, o->s21[1] = 2 * (int)(b[74 + j] >> 4) + 1;
    o->d = half_value(rd16(b));
    return 1;
  }
  case QTYPE_IQ3_XXS: /* q8.h:98-108: the quarter-step scale as 2 (2s + 1) eighths */
  {
    const uint8_t *q = b + 2 + 8 * j;
    const uint32_t aux = rd32(b + 66 + 4 * j);
    for (int k = 0; k < 4; k++)
    {
      const uint64_t g = (uint64_t)osmos_grid_iq3xxs[q[2 * k]] | (uint64_t)osmos_grid_iq3xxs[q[2 * k + 1]] << 32;
      grid_signed(g, osmos_ksigns[(aux >> (7 * k)) & 0x7F], o->code + 8 * k);
    }
    o->s21[0] = o->s21[1] = 2 * (2 * (int)(aux >> 28) + 1);
    o->d = half_value(rd16(b));
    return 1;
  }
  case QTYPE_IQ1_S: /* q8.h:121-130 */
  {
    const uint32_t h = rd16(b + 34 + 2 * j);
    for (int k = 0; k < 4; k++)
    {
      const uint64_t g = osmos_grid_iq1s[b[2 + 4 * j + k] | ((h >> (3 * k)) & 0x07) << 8];
      for (int i = 0; i < 8; i++)
        o->code[8 * k + i] = (int)(int8_t)(g >> (8 * i));
      o->delta[k] = h & 0x8000 ? -1 : 1;
    }
    o->s21[0] = o->s21[1] = 2 * (int)((h >> 12) & 0x07) + 1;
    o->d = half_value(rd16(b));
    return 1;
  }
  case QTYPE_IQ1_M: /* q8.h:68-84 */
  {
    const uint64_t sc = rd64(b + 48);
    for (int k = 0; k < 4; k++)
    {
      const int kk = 4 * j + k;
      const uint32_t h = (b[32 + kk / 2] >> (4 * (kk % 2))) & 0x0F;
      const uint64_t g = osmos_grid_iq1s[b[kk] | (h & 0x07) << 8];
      for (int i = 0; i < 8; i++)
        o->code[8 * k + i] = (int)(int8_t)(g >> (8 * i));
      o->delta[k] = h & 0x08 ? -1 : 1;
    }
    for (int h = 0; h < 2; h++)
    {
      const int kk = 4 * j + 2 * h;
      o->s21[h] = 2 * (int)((sc >> (16 * (kk / 8) + 3 * ((kk / 2) % 4))) & 0x07) + 1;
    }
    o->d = iq1m_d(b);
    return 1;
  }
  case QTYPE_Q2_K: /* q8.h:111-118 */
  {
    for (int i = 0; i < 32; i++)
      o->code[i] = (b[16 + 32 * (j / 4) + i] >> (2 * (j % 4))) & 0x03;
    for (int h = 0; h < 2; h++)
      o->s21[h] = 8 * (b[2 * j + h] & 0x0F), o->m8[h] = 8 * (b[2 * j + h] >> 4);
    o->d = half_value(rd16(b + 80)), o->dmin = half_value(rd16(b + 82));
    return 1;
  }
  /* Extension (no reference path): a 32-value block with one f16 scale and integer codes. The reference never
     runs Q4_0 / Q8_0 against int8 activations; the order below is this library's, built from the lane's rules:
     the whole block's integer dot (exact), block = d * (float)isum, then the usual fmaf with x's scale. */
  case QTYPE_Q4_0:
  {
    for (int i = 0; i < 16; i++)
      o->code[i] = (int)(b[2 + i] & 0x0F) - 8, o->code[16 + i] = (int)(b[2 + i] >> 4) - 8;
    o->d = half_value(rd16(b));
    o->plain = 1;
    return 1;
  }
  case QTYPE_Q8_0:
  {
    for (int i = 0; i < 32; i++)
      o->code[i] = (int)(int8_t)b[2 + i];
    o->d = half_value(rd16(b));
    o->plain = 1;
    return 1;
  }
  default:
    return 0;
  }
}

/* a half's (or a plain block's) exact integer sums: codes . x, and for IQ1 8 (grid . x) + delta (sum x) a chunk */
static void lane_isums(uint32_t type, const LaneBlock *c, const int8_t *x, int isum[2], int xsum[2])
{
  for (int h = 0; h < 2; h++)
  {
    int s = 0, sx = 0;
    for (int k = 2 * h; k < 2 * h + 2; k++)
    {
      int gx = 0, cx = 0;
      for (int i = 0; i < 8; i++)
        gx += c->code[8 * k + i] * (int)x[8 * k + i], cx += (int)x[8 * k + i];
      s += (type == QTYPE_IQ1_M || type == QTYPE_IQ1_S) ? 8 * gx + c->delta[k] * cx : gx;
      sx += cx;
    }
    isum[h] = s, xsum[h] = sx;
  }
}

static float lane_part(float d, int s21, int isum) { return d * (float)s21 * 0.125f * (float)isum; } /* lane.h:66 */

/* the block's value before x's scale (q8.h:131-162) */
static float lane_block_sum(uint32_t type, const LaneBlock *c, const int8_t *x)
{
  int isum[2], xsum[2];
  lane_isums(type, c, x, isum, xsum);
  if (c->plain)
    return c->d * (float)(isum[0] + isum[1]);
  if (type == QTYPE_Q2_K)
  {
    const float p0 = lane_part(c->d, c->s21[0], isum[0]) - lane_part(c->dmin, c->m8[0], xsum[0]);
    const float p1 = lane_part(c->d, c->s21[1], isum[1]) - lane_part(c->dmin, c->m8[1], xsum[1]);
    return p0 + p1;
  }
  return lane_part(c->d, c->s21[0], isum[0]) + lane_part(c->d, c->s21[1], isum[1]);
}

static int lane_type_ok(uint32_t type)
{
  const OsmosQTypeInfo *t = type_row(type);
  return t && (t->paths & (QTYPE_PATH_Q8 | QTYPE_PATH_Q8_EXT));
}

/* the exact integer half-block dots of one row against one int8 input row: out[2 * s + h] for 32-value block s
   (the numbers the "bit-exact integer dot" requirement is about; the kernels can dump the same) */
ORC_API int orc_q8_block_dots(uint32_t type, const void *w_row, uint32_t cols, const int8_t *q, int32_t *out)
{
  const OsmosQTypeInfo *t = type_row(type);
  if (!lane_type_ok(type) || !cols || cols % t->values)
    return 0;
  const int per = (int)t->values / 32;
  for (uint32_t s = 0; s < cols / 32; s++)
  {
    LaneBlock c;
    int isum[2], xsum[2];
    lane_block(type, (const uint8_t *)w_row + (uint64_t)(s / per) * t->bytes, (int)(s % per), &c);
    lane_isums(type, &c, q + (uint64_t)s * 32, isum, xsum);
    out[2 * s] = isum[0], out[2 * s + 1] = isum[1];
  }
  return 1;
}

/* q8_group_tok's sums for one matrix (kernels/q8.h:179-212): rows r0 .. r1 against n int8 rows; a row's blocks to
   L = 32 lanes when cols >= 4096, else 16 (lane.h:50-51), lane l its blocks l, l + L, ... in order, each
   acc = fmaf(d_x, block, acc); then the lanes' xor tree */
ORC_API int orc_q8_rows(uint32_t type, const void *w, uint32_t cols, uint32_t r0, uint32_t r1, const int8_t *q,
                        const float *d, uint32_t n, float *y, uint32_t ys)
{
  const OsmosQTypeInfo *t = type_row(type);
  if (!lane_type_ok(type) || !w || !cols || cols % t->values || r1 < r0 || !n)
    return 0;
  const int per = (int)t->values / 32, lanes = cols >= 4096 ? 32 : 16;
  const uint32_t nblk = cols / 32;
  const uint64_t row_bytes = (uint64_t)(cols / t->values) * t->bytes;
  for (uint32_t r = r0; r < r1; r++)
  {
    const uint8_t *row = (const uint8_t *)w + r * row_bytes;
    LaneBlock *blk = malloc((size_t)nblk * sizeof *blk);
    for (uint32_t s = 0; s < nblk; s++)
      lane_block(type, row + (uint64_t)(s / per) * t->bytes, (int)(s % per), &blk[s]);
    for (uint32_t tk = 0; tk < n; tk++)
    {
      float acc[32] = {0};
      for (uint32_t s = 0; s < nblk; s++)
        acc[s % lanes] = fmaf(d[(uint64_t)tk * nblk + s], lane_block_sum(type, &blk[s], q + (uint64_t)tk * cols + (uint64_t)s * 32),
                              acc[s % lanes]);
      y[(uint64_t)tk * ys + r] = xor_tree(acc, lanes);
    }
    free(blk);
  }
  return 1;
}

/* the lane's exp and activation (kernels/lane.h:17-41, 69-75) */
static float lane_exp(float x)
{
  if (x > 88.72283905f)
    return INFINITY;
  const float k = rintf(x * 1.44269504089f);
  float r = fmaf(-k, 0.693145751953125f, x);
  r = fmaf(-k, 1.428606765330187e-06f, r);
  float p = 1.0f / 5040.0f;
  p = fmaf(p, r, 1.0f / 720.0f);
  p = fmaf(p, r, 1.0f / 120.0f);
  p = fmaf(p, r, 1.0f / 24.0f);
  p = fmaf(p, r, 1.0f / 6.0f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  return ldexpf(p, (int)k);
}

static float lane_swiglu(float g, float u, float lim, float scale)
{
  const float gv = fminf(g, lim), uv = fminf(fmaxf(u, -lim), lim);
  return gv / (1.0f + lane_exp(-gv)) * uv * scale;
}

ORC_API float orc_lane_exp(float x) { return lane_exp(x); }

/* ops_swiglu_lane (kernels/ops.hip:502-507): h[t][c] = lane_swiglu(g, u, lim, scale[t]) */
ORC_API void orc_swiglu_lane(const float *g, const float *u, uint32_t n, float lim, const float *scale, uint32_t n_tok,
                             float *h)
{
  for (uint64_t i = 0; i < (uint64_t)n * n_tok; i++)
    h[i] = lane_swiglu(g[i], u[i], lim, scale[i / n]);
}

/* one expert of the lane's FFN on `cnt` rows (src/cpu/lane.c:98-124, src/run/hip_lane.c:71-113): x rows to int8,
   gate and up, the activation with each row's routed weight, the activations to int8, down */
ORC_API int orc_lane_expert(uint32_t type_gu, uint32_t type_down, const void *gate, const void *up, const void *down,
                            uint32_t dim, uint32_t ff, float lim, const float *x, const float *scale, uint32_t cnt,
                            float *y)
{
  if (!cnt || !dim || !ff)
    return 0;
  int8_t *q = malloc((size_t)cnt * dim), *qh = malloc((size_t)cnt * ff);
  float *qd = malloc((size_t)cnt * (dim / 32) * sizeof *qd), *qhd = malloc((size_t)cnt * (ff / 32) * sizeof *qhd);
  float *g = malloc((size_t)cnt * ff * sizeof *g), *u = malloc((size_t)cnt * ff * sizeof *u);
  int ok = orc_q8_round(x, cnt, dim, dim, q, qd) && orc_q8_rows(type_gu, gate, dim, 0, ff, q, qd, cnt, g, ff) &&
           orc_q8_rows(type_gu, up, dim, 0, ff, q, qd, cnt, u, ff);
  if (ok)
  {
    orc_swiglu_lane(g, u, ff, lim, scale, cnt, g);
    ok = orc_q8_round(g, cnt, ff, ff, qh, qhd) && orc_q8_rows(type_down, down, ff, 0, dim, qh, qhd, cnt, y, dim);
  }
  free(q), free(qh), free(qd), free(qhd), free(g), free(u);
  return ok;
}

/* ops_gather_sum_add (kernels/ops.hip:517-525): y[t] = sum over j of src[idx[t m + j]] from 0 in j's order, + add */
ORC_API void orc_gather_sum(float *y, const float *src, const int32_t *idx, uint32_t m, uint32_t n, uint32_t dim,
                            const float *add)
{
  for (uint32_t t = 0; t < n; t++)
    for (uint32_t c = 0; c < dim; c++)
    {
      float s = 0.0f;
      for (uint32_t j = 0; j < m; j++)
        s += src[(uint64_t)idx[t * m + j] * dim + c];
      y[(uint64_t)t * dim + c] = add ? s + add[(uint64_t)t * dim + c] : s;
    }
}

/* ------------------------------------------------------------------------------------------------------------
 * mmq: Q4_K x int8 (include/osmos/gpu/mmq.h:17-27; kernels/mmq.hip:33-52, 60-151; the host replay in
 * tests/gpu/test_mmq_gpu.hip:66-121)
 * ---------------------------------------------------------------------------------------------------------- */
static uint64_t x8_at(uint32_t s, uint32_t c, uint32_t cols)
{
  return (uint64_t)(s / 16) * 16 * cols + (uint64_t)(c / 32) * (16 * 32) + (s % 16) * 32 + c % 32;
}
static uint64_t dx_at(uint32_t s, uint32_t g, uint32_t groups)
{
  return (uint64_t)(s / 16) * 16 * groups + (uint64_t)g * 16 + s % 16;
}
ORC_API uint64_t orc_mmq_x8_at(uint32_t s, uint32_t c, uint32_t cols) { return x8_at(s, c, cols); }
ORC_API uint64_t orc_mmq_dx_at(uint32_t s, uint32_t g, uint32_t groups) { return dx_at(s, g, groups); }

/* mmq_x8_rows: slot s = row idx[s] of x (-1: zeros) per 32: dx = amax / 127, x8 = clamp(rint(x / dx), +-127),
   sx = dx * (float)sum(x8); the buffers hold whole tiles of 16 slots (the pad slots are not written) */
ORC_API int orc_mmq_x8_rows(const float *x, uint32_t xs, const int32_t *idx, uint32_t slots, uint32_t cols, int8_t *x8,
                            float *dx, float *sx)
{
  if (!slots || !cols || cols % 32 || xs < cols)
    return 0;
  const uint32_t groups = cols / 32;
  for (uint32_t s = 0; s < slots; s++)
    for (uint32_t g = 0; g < groups; g++)
    {
      float v[32], a = 0.0f;
      for (int i = 0; i < 32; i++)
      {
        v[i] = idx[s] >= 0 ? x[(uint64_t)idx[s] * xs + g * 32 + i] : 0.0f;
        a = fmaxf(a, fabsf(v[i]));
      }
      const float d = a / 127.0f;
      int sum = 0;
      for (int i = 0; i < 32; i++)
      {
        const int qv = a == 0.0f ? 0 : (int)fminf(fmaxf(rintf(v[i] / d), -127.0f), 127.0f);
        x8[x8_at(s, g * 32 + i, cols)] = (int8_t)qv;
        sum += qv;
      }
      const uint64_t at = dx_at(s, g, groups);
      dx[at] = a == 0.0f ? 0.0f : d;
      sx[at] = dx[at] * (float)sum;
    }
  return 1;
}

/* mmq_group for one matrix: y[t * ys + r] for t < cnt over slots soff .. ; K split in 4 partitions by 256-value
   block (partition p: blocks p, p + 4, ...), in a partition per 32-group: v = (d sc) dx; acc = fmaf(v, I, acc);
   acc = fmaf(dmin m, -sx, acc); the four partitions added in order. ints[] (or NULL) receives the exact group
   dots I of (row, token) laid [row][token][group] */
ORC_API int orc_mmq_rows(const void *w, uint32_t r0, uint32_t r1, uint32_t cols, const int8_t *x8, const float *dx,
                         const float *sx, uint32_t soff, uint32_t cnt, float *y, uint32_t ys, int32_t *ints)
{
  if (r1 < r0 || !cols || cols % 256 || !cnt)
    return 0;
  const uint32_t nb = cols / 256, groups = cols / 32;
  for (uint32_t r = r0; r < r1; r++)
  {
    const uint8_t *row = (const uint8_t *)w + (uint64_t)r * nb * 144;
    for (uint32_t t = 0; t < cnt; t++)
    {
      const uint32_t slot = soff + t;
      float part[4] = {0, 0, 0, 0};
      for (uint32_t p = 0; p < 4; p++)
        for (uint32_t b = p; b < nb; b += 4)
        {
          const uint8_t *blk = row + (uint64_t)b * 144;
          const float d = half_value(rd16(blk)), dmin = half_value(rd16(blk + 2));
          for (int g = 0; g < 8; g++)
          {
            int sc, mn, isum = 0;
            q4k_scale_min(blk + 4, g, &sc, &mn);
            const float dsc = d * (float)sc, dm = dmin * (float)mn;
            const uint32_t gg = b * 8 + (uint32_t)g;
            for (int i = 0; i < 32; i++)
              isum += (int)((blk[16 + (g / 2) * 32 + i] >> (4 * (g % 2))) & 0x0F) * (int)x8[x8_at(slot, gg * 32 + i, cols)];
            if (ints)
              ints[((uint64_t)r * cnt + t) * groups + gg] = isum;
            const uint64_t at = dx_at(slot, gg, groups);
            const float v = dsc * dx[at];
            part[p] = fmaf(v, (float)isum, part[p]);
            part[p] = fmaf(dm, -sx[at], part[p]);
          }
        }
      float s = part[0];
      for (int p = 1; p < 4; p++)
        s = s + part[p];
      y[(uint64_t)t * ys + r] = s;
    }
  }
  return 1;
}

/* ------------------------------------------------------------------------------------------------------------
 * MX activation rounding (kernels/round.hip:49-78, kernels/round.h:23-61,99-126): per `block` values a scale -
 * a power of two 2^ceil(log2(max(amax, 6 * 2^-126) / 6)), or amax / 6 rounded to E4M3 - and E2M1 values under it
 * ---------------------------------------------------------------------------------------------------------- */
static float e2m1_round(float v) /* nearest, ties to the even mantissa; |v| <= 6 */
{
  const float a = fabsf(v);
  const float q = a <= 0.25f ? 0.0f : a < 0.75f ? 0.5f : a <= 1.25f ? 1.0f : a < 1.75f ? 1.5f
                : a <= 2.5f ? 2.0f : a < 3.5f ? 3.0f : a <= 5.0f ? 4.0f : 6.0f;
  return copysignf(q, v);
}
static uint32_t e2m1_code(float q)
{
  const float a = fabsf(q);
  const uint32_t i = a == 0.0f ? 0 : a == 0.5f ? 1 : a == 1.0f ? 2 : a == 1.5f ? 3 : a == 2.0f ? 4 : a == 3.0f ? 5 : a == 4.0f ? 6 : 7;
  uint32_t bits;
  memcpy(&bits, &q, 4);
  return (bits >> 31) << 3 | i;
}
static float e4m3_round(float x) /* nearest even, no infinities, |x| <= 448 */
{
  const float a = fabsf(x);
  float q;
  if (a < ldexpf(1.0f, -6))
  {
    const float step = ldexpf(1.0f, -9);
    q = rintf(a / step) * step;
  }
  else
  {
    int e;
    frexpf(a, &e);
    const float step = ldexpf(1.0f, e - 1 - 3);
    q = rintf(a / step) * step;
  }
  return copysignf(q, x);
}
static uint32_t e4m3_code(float q)
{
  uint32_t bits;
  memcpy(&bits, &q, 4);
  const uint32_t sign = bits >> 31 << 7;
  const float a = fabsf(q);
  if (a < ldexpf(1.0f, -6))
    return sign | (uint32_t)(a * ldexpf(1.0f, 9));
  int e;
  const float m = frexpf(a, &e);
  return sign | (uint32_t)(e - 1 + 7) << 3 | (uint32_t)((m * 2.0f - 1.0f) * 8.0f);
}

/* ops_fp4_round (power-of-two scale, block 32): x rounded in place; packed (or NULL) rows of dim: dim / 2 code bytes
   (even value in the low nibble) then dim / 32 UE8M0 scale bytes */
ORC_API int orc_fp4_round(float *x, uint64_t n, uint32_t block, int e4m3_scale, uint8_t *packed, uint32_t dim)
{
  if (!n || !block || n % block || block > 32)
    return 0;
  if (packed && (!dim || dim % block || dim % 4 || n % dim || block != (e4m3_scale ? 16u : 32u)))
    return 0;
  const uint64_t row_bytes = packed ? dim / 2 + dim / block : 0;
  for (uint64_t b = 0; b < n / block; b++)
  {
    float *v = x + b * block, amax = 0.0f;
    for (uint32_t j = 0; j < block; j++)
      amax = fmaxf(amax, fabsf(v[j]));
    float s;
    if (e4m3_scale)
      s = e4m3_round(fmaxf(amax, 6.0f * ldexpf(1.0f, -9)) / 6.0f);
    else
      s = exp2f(ceilf(log2f(fmaxf(amax, 6.0f * ldexpf(1.0f, -126)) / 6.0f)));
    for (uint32_t j = 0; j < block; j++)
    {
      const float q = e2m1_round(fminf(fmaxf(v[j] / s, -6.0f), 6.0f));
      v[j] = q * s;
      if (packed)
      {
        const uint64_t i = b * block + j;
        uint8_t *row = packed + i / dim * row_bytes;
        const uint32_t c = (uint32_t)(i % dim);
        const uint32_t code = e2m1_code(q);
        if (c % 2 == 0)
          row[c / 2] = (uint8_t)((row[c / 2] & 0xF0) | code);
        else
          row[c / 2] = (uint8_t)((row[c / 2] & 0x0F) | code << 4);
      }
    }
    if (packed)
    {
      const uint64_t i = b * block;
      uint8_t *row = packed + i / dim * row_bytes;
      row[dim / 2 + (i % dim) / block] =
          (uint8_t)(e4m3_scale ? (s > 448.0f ? 0x7F : e4m3_code(s)) : (uint32_t)(ilogbf(s) + 127));
    }
  }
  return 1;
}

/* ops_fp8_round: per 32 a power-of-two scale 2^ceil(log2(max(amax, 1e-4) / 448)), E4M3 values under it; packed rows:
   dim code bytes then dim / 32 UE8M0 bytes */
ORC_API int orc_fp8_round(float *x, uint64_t n, uint8_t *packed, uint32_t dim)
{
  if (!n || n % 32 || (packed && (!dim || dim % 32 || n % dim)))
    return 0;
  for (uint64_t b = 0; b < n / 32; b++)
  {
    float *v = x + b * 32, amax = 0.0f;
    for (int j = 0; j < 32; j++)
      amax = fmaxf(amax, fabsf(v[j]));
    const float s = exp2f(ceilf(log2f(fmaxf(amax, 1e-4f) / 448.0f)));
    for (int j = 0; j < 32; j++)
    {
      const float q = e4m3_round(fminf(fmaxf(v[j] / s, -448.0f), 448.0f));
      v[j] = q * s;
      if (packed)
      {
        const uint64_t i = b * 32 + (uint64_t)j;
        packed[i / dim * (dim + dim / 32) + i % dim] = (uint8_t)e4m3_code(q);
      }
    }
    if (packed)
    {
      const uint64_t i = b * 32;
      packed[i / dim * (dim + dim / 32) + dim + (i % dim) / 32] = (uint8_t)(ilogbf(s) + 127);
    }
  }
  return 1;
}

/* ------------------------------------------------------------------------------------------------------------
 * mm_x16 / mm_x16_rows (kernels/mm.h:41-51, kernels/mm.hip:77-159): F32 rows to f16 (nearest even) in the tiled
 * layout token t, column c -> (t / 16) 16 xts + (c / 16) 256 + (t % 16) 16 + c % 16; slot s is row idx[s] of x (idx
 * NULL: row s; -1 or a slot past `slots`: zeros), slots rounded up to whole tiles of 16. Returns 1 when a value was
 * past f16's range (or NaN): the overflow flag.
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API int orc_x16_rows(const float *x, uint32_t xs, const int32_t *idx, uint32_t slots, uint32_t cols, uint16_t *x16)
{
  int over = 0;
  const uint32_t padded = (slots + 15) / 16 * 16;
  for (uint32_t t = 0; t < padded; t++)
  {
    const int64_t r = t < slots ? (idx ? idx[t] : (int64_t)t) : -1;
    for (uint32_t c = 0; c < cols; c++)
    {
      const float v = r >= 0 ? x[(uint64_t)r * xs + c] : 0.0f;
      if (!(fabsf(v) <= 65504.0f))
        over = 1;
      x16[(uint64_t)(t / 16) * 16 * cols + (uint64_t)(c / 16) * 256 + (t % 16) * 16 + c % 16] = half_bits(v);
    }
  }
  return over;
}

/* ------------------------------------------------------------------------------------------------------------
 * mv_fp4 / mv_fp4_tok (kernels/mv_fp4.hip:25-107, 213-273): NVFP4 rows over F32 activations in that file's own order.
 * A row's 64-value blocks go to `lanes` lanes (32 for mv_fp4; 8, 16 or 32 by the row's length for mv_fp4_tok), lane l
 * taking blocks l, l + lanes, ...; of a block, each 16-value sub-block s: part = 0, then for j = 0 .. 7
 * part = fmaf(v[j], x[j], fmaf(v[j + 8], x[j + 8], part)), acc = fmaf(d_s, part, acc) with d_s the UE4M3 scale halved
 * and v the E2M1 values doubled; the lanes by the xor tree; the sum times `scale`.
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API void orc_mv_fp4_rows(const uint8_t *w, uint32_t rows, uint32_t cols, const float *x, uint32_t xs, uint32_t n,
                             uint32_t lanes, float scale, int use_scale, float *y, uint32_t ys)
{
  const uint32_t nb = cols / 64;
  for (uint32_t t = 0; t < n; t++)
    for (uint32_t r = 0; r < rows; r++)
    {
      float acc[32];
      for (uint32_t l = 0; l < lanes; l++)
      {
        acc[l] = 0.0f;
        for (uint32_t b = l; b < nb; b += lanes)
        {
          const uint8_t *blk = w + ((uint64_t)r * nb + b) * 36;
          const float *xb = x + (uint64_t)t * xs + (uint64_t)b * 64;
          for (int s = 0; s < 4; s++)
          {
            const float d = ue4m3_value(blk[s]) * 0.5f;
            float part = 0.0f;
            for (int j = 0; j < 8; j++)
            {
              const uint8_t q = blk[4 + 8 * s + j];
              const float a = (float)osmos_e2m1_doubled[q & 0x0F], c = (float)osmos_e2m1_doubled[q >> 4];
              part = fmaf(a, xb[16 * s + j], fmaf(c, xb[16 * s + j + 8], part));
            }
            acc[l] = fmaf(d, part, acc[l]);
          }
        }
      }
      for (uint32_t o = lanes / 2; o > 0; o >>= 1)
        for (uint32_t l = 0; l < o; l++)
          acc[l] = acc[l] + acc[l + o];
      y[(uint64_t)t * ys + r] = use_scale ? acc[0] * scale : acc[0];
    }
}

/* ------------------------------------------------------------------------------------------------------------
 * mm_fp4_act / mm_fp4_quant (kernels/mm_fp4.hip:23-104): the activations of the W4A4 product. Every 16 values one
 * E4M3 scale - the code of min(amax / 6 / gs, 448) to nearest even (frexpf's fraction rounded to 3 bits; below 2^-6
 * whole numbers of 2^-9) - and E2M1 codes of v / (scale gs) clamped to +-6: to nearest with a tie to the even index,
 * or (seed != 0) up with probability (distance from the grid point below) / step under a hash of (seed, element).
 * x: F32, or (bf16) the upper halves of F32. q: n x cols / 2 bytes, k order, low nibble first; sc: n x cols / 16.
 * ---------------------------------------------------------------------------------------------------------- */
static uint32_t fp4_scale_code(float v) /* mm_fp4.hip:26-43 */
{
  const float a = fminf(v, 448.0f);
  if (!(a > 0.0f))
    return 0;
  int e;
  const float m = frexpf(a, &e);
  int E = e - 1 + 7;
  if (E >= 1)
  {
    float q = rintf((m * 2.0f - 1.0f) * 8.0f);
    if (q >= 8.0f)
      q = 0.0f, E++;
    if (E > 15 || (E == 15 && q > 6.0f))
      return 0x7E;
    return (uint32_t)(E << 3) | (uint32_t)q;
  }
  const float q = rintf(a / 0.001953125f);
  return q >= 8.0f ? 0x08u : (uint32_t)q;
}
static float fp4_scale_value(uint32_t c) /* kernels/round.h:87-93, codes up to 0x7E */
{
  return c >> 3 ? ldexpf(1.0f + (float)(c & 7) / 8.0f, (int)(c >> 3) - 7) : (float)c * 0.001953125f;
}
static const float fp4_grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
static uint32_t fp4_code_nearest(float x) /* mm_fp4.hip:46-59 */
{
  const float a = fabsf(x);
  uint32_t i;
  if (a <= 0.25f) i = 0;
  else if (a < 0.75f) i = 1;
  else if (a <= 1.25f) i = 2;
  else if (a < 1.75f) i = 3;
  else if (a <= 2.5f) i = 4;
  else if (a < 3.5f) i = 5;
  else if (a <= 5.0f) i = 6;
  else i = 7;
  return i ? (x < 0.0f ? 8u : 0u) | i : 0u;
}
static float fp4_uniform(uint32_t seed, uint64_t i) /* mm_fp4.hip:64-69 */
{
  uint32_t h = (uint32_t)i * 0x9E3779B1u ^ (uint32_t)(i >> 32) * 0x85EBCA77u ^ seed;
  h ^= h >> 16, h *= 0x85EBCA6Bu, h ^= h >> 13, h *= 0xC2B2AE35u, h ^= h >> 16;
  return (float)(h >> 8) * (1.0f / 16777216.0f);
}
static uint32_t fp4_code_stochastic(float x, float u) /* mm_fp4.hip:73-81 */
{
  const float a = fabsf(x);
  uint32_t i = 0;
  while (i < 7 && a >= fp4_grid[i + 1])
    i++;
  if (i < 7 && u < (a - fp4_grid[i]) / (fp4_grid[i + 1] - fp4_grid[i]))
    i++;
  return i ? (x < 0.0f ? 8u : 0u) | i : 0u;
}
ORC_API void orc_fp4_act(const void *x, int bf16, uint32_t xs, uint32_t n, uint32_t cols, float gs, uint32_t seed,
                         uint8_t *q, uint8_t *sc) /* mm_fp4.hip:84-112 */
{
  for (uint32_t t = 0; t < n; t++)
    for (uint32_t b = 0; b < cols / 16; b++)
    {
      float v[16], amax = 0.0f;
      for (int j = 0; j < 16; j++)
      {
        const uint64_t at = (uint64_t)t * xs + b * 16 + j;
        if (bf16)
        {
          const uint32_t bits = (uint32_t)((const uint16_t *)x)[at] << 16;
          memcpy(&v[j], &bits, 4);
        }
        else
          v[j] = ((const float *)x)[at];
        amax = fmaxf(amax, fabsf(v[j]));
      }
      const uint32_t s = fp4_scale_code(amax / 6.0f / gs);
      const float sf = fp4_scale_value(s) * gs;
      sc[(uint64_t)t * (cols / 16) + b] = (uint8_t)s;
      uint8_t *o = q + (uint64_t)t * (cols / 2) + b * 8;
      for (int j = 0; j < 16; j++)
      {
        const float c = sf > 0.0f ? fminf(fmaxf(v[j] / sf, -6.0f), 6.0f) : 0.0f;
        const uint64_t k = (uint64_t)t * cols + b * 16 + j;
        const uint32_t code = seed ? fp4_code_stochastic(c, fp4_uniform(seed, k)) : fp4_code_nearest(c);
        if (j % 2 == 0)
          o[j / 2] = (uint8_t)code;
        else
          o[j / 2] |= (uint8_t)(code << 4);
      }
    }
}

/* mm_fp4's sums the way the reference's test takes them (tests/gpu/test_mm_fp4_gpu.hip:129-153): double sums over the
 * quantized values - weight (E2M1 value) (UE4M3 scale, its sign bit not read), activation (E2M1 value) (E4M3 scale) -
 * times scale; also the sums of the products' magnitudes (for an error bound). y, mag: n x rows doubles. */
ORC_API void orc_fp4_mm(const uint8_t *w, uint32_t rows, uint32_t cols, const uint8_t *q, const uint8_t *sc, uint32_t n,
                        double scale, double *y, double *mag)
{
  const uint32_t nb = cols / 64;
  for (uint32_t t = 0; t < n; t++)
    for (uint32_t r = 0; r < rows; r++)
    {
      double s = 0.0, m = 0.0;
      for (uint32_t b = 0; b < nb; b++)
      {
        const uint8_t *blk = w + ((uint64_t)r * nb + b) * 36;
        for (int sb = 0; sb < 4; sb++)
          for (int j = 0; j < 16; j++)
          {
            const uint8_t byte = blk[4 + 8 * sb + (j & 7)];
            const uint32_t cw = (j < 8 ? byte : byte >> 4) & 15;
            const double wv = (cw & 8 ? -1.0 : 1.0) * fp4_grid[cw & 7] * (double)ue4m3_value(blk[sb]);
            const uint64_t c = (uint64_t)b * 64 + sb * 16 + j;
            const uint32_t ca = (q[((uint64_t)t * cols + c) / 2] >> (4 * (c & 1))) & 15;
            const double av = (ca & 8 ? -1.0 : 1.0) * fp4_grid[ca & 7] * (double)fp4_scale_value(sc[(uint64_t)t * (cols / 16) + c / 16] & 0x7F);
            s += wv * av, m += fabs(wv * av);
          }
      }
      y[(uint64_t)t * rows + r] = s * scale;
      if (mag)
        mag[(uint64_t)t * rows + r] = m * fabs(scale);
    }
}

/* ------------------------------------------------------------------------------------------------------------
 * mm_x16_attn (kernels/mm.hip:105-135): each head's last rope_dim values rotated back - pair (2i, 2i + 1) at angle
 * pos[t] freqs[i]: with cs = cos, sn = -sin, (a cs - b sn, a sn + b cs) - then every 32 values to E4M3 under their
 * power-of-two scale (orc_fp8_round's rule), then f16 in the tiled layout; rows up to the next multiple of 16 zero.
 * Returns the overflow flag.
 * ---------------------------------------------------------------------------------------------------------- */
ORC_API int orc_x16_attn(const float *x, uint32_t xs, uint32_t n, uint32_t cols, uint32_t head_dim, uint32_t rope_dim,
                         const float *freqs, const int32_t *pos, uint16_t *x16)
{
  int over = 0;
  const uint32_t padded = (n + 15) / 16 * 16, r0 = head_dim - rope_dim;
  for (uint32_t t = 0; t < padded; t++)
    for (uint32_t c0 = 0; c0 < cols; c0 += 32)
    {
      float v[32];
      for (uint32_t j = 0; j < 32; j++)
        v[j] = t < n ? x[(uint64_t)t * xs + c0 + j] : 0.0f;
      if (t < n)
      {
        if (c0 % head_dim >= r0)
          for (uint32_t j = 0; j < 32; j += 2)
          {
            const float ang = (float)pos[t] * freqs[((c0 + j) % head_dim - r0) / 2];
            const float cs = cosf(ang), sn = -sinf(ang), a = v[j], b = v[j + 1];
            const float lo = a * cs, lo2 = b * sn, hi = a * sn, hi2 = b * cs;
            v[j] = lo - lo2, v[j + 1] = hi + hi2;
          }
        if (!orc_fp8_round(v, 32, NULL, 0))
          return -1;
      }
      for (uint32_t j = 0; j < 32; j++)
      {
        const uint32_t c = c0 + j;
        if (!(fabsf(v[j]) <= 65504.0f))
          over = 1;
        x16[(uint64_t)(t / 16) * 16 * cols + (uint64_t)(c / 16) * 256 + (t % 16) * 16 + c % 16] = half_bits(v[j]);
      }
    }
  return over;
}
