// GGUF block decoders for the device: a block's values as F32 (8 at a time), and a 32-value sub-block as packed
// int8 codes for the int8 lane. Every value is the bits gguf-py's dequantize gives (the same products, each rounded
// once); the block layouts are the GGUF's own, read where they lie.
//
// Replaces the reference's kernels/quant.h:65-362 (decode<T>) and kernels/q8.h:28-162 (codes<T>, block_sum<T>).
#pragma once
#include "common.cuh"

namespace osmos {

constexpr int kChunk = 8;  // values decoded at a time: the unit the F32 matvec deals to its lanes

// the codebook tables a kernel reads: pointers into shared memory when the kernel staged them there, else the
// global copies
struct Grids {
  const uint64_t* g64;  // the type's 8-value grid (IQ2_XXS, IQ2_XS, IQ2_S, IQ1_S / IQ1_M)
  const uint32_t* g32;  // IQ3_XXS's 4-value grid
  const uint8_t* sign;  // the 7-bit sign index -> 8 sign bits (even parity)
};

template <uint32_t T> struct Fmt;
#define OSMOS_FMT(name, id, nvalues, nbytes, paths)                              \
  template <> struct Fmt<id> {                                                   \
    static constexpr int values = nvalues, bytes = nbytes;                       \
    static constexpr int chunks = nvalues / kChunk, subs = nvalues / 32;         \
  };
OSMOS_FMT(Q4_0, 2, 32, 18, 0) OSMOS_FMT(Q8_0, 8, 32, 34, 0) OSMOS_FMT(Q2_K, 10, 256, 84, 0)
OSMOS_FMT(Q4_K, 12, 256, 144, 0) OSMOS_FMT(IQ2_XXS, 16, 256, 66, 0) OSMOS_FMT(IQ2_XS, 17, 256, 74, 0)
OSMOS_FMT(IQ3_XXS, 18, 256, 98, 0) OSMOS_FMT(IQ1_S, 19, 256, 50, 0) OSMOS_FMT(IQ2_S, 22, 256, 82, 0)
OSMOS_FMT(IQ1_M, 29, 256, 56, 0) OSMOS_FMT(MXFP4, 39, 32, 17, 0) OSMOS_FMT(NVFP4, 40, 64, 36, 0)
#undef OSMOS_FMT

// which grid table a type's kernels stage (0: none)
template <uint32_t T> struct GridOf { static constexpr int words64 = 0, words32 = 0; static constexpr bool signs = false; };
template <> struct GridOf<QTYPE_IQ2_XXS> { static constexpr int words64 = 256, words32 = 0; static constexpr bool signs = true; };
template <> struct GridOf<QTYPE_IQ2_XS> { static constexpr int words64 = 512, words32 = 0; static constexpr bool signs = true; };
template <> struct GridOf<QTYPE_IQ2_S> { static constexpr int words64 = 1024, words32 = 0; static constexpr bool signs = false; };
template <> struct GridOf<QTYPE_IQ1_S> { static constexpr int words64 = 2048, words32 = 0; static constexpr bool signs = false; };
template <> struct GridOf<QTYPE_IQ1_M> { static constexpr int words64 = 2048, words32 = 0; static constexpr bool signs = false; };
template <> struct GridOf<QTYPE_IQ3_XXS> { static constexpr int words64 = 0, words32 = 256; static constexpr bool signs = true; };

template <uint32_t T> __device__ __forceinline__ const uint64_t* global_grid64() {
  if constexpr (T == QTYPE_IQ2_XXS) return osmos_grid_iq2xxs;
  else if constexpr (T == QTYPE_IQ2_XS) return osmos_grid_iq2xs;
  else if constexpr (T == QTYPE_IQ2_S) return osmos_grid_iq2s;
  else if constexpr (T == QTYPE_IQ1_S || T == QTYPE_IQ1_M) return osmos_grid_iq1s;
  else return nullptr;
}

// the calling block copies its type's tables into `smem` (at least grid_smem_bytes<T>() of it, 8-byte aligned) and
// returns pointers to the copies; every thread of the block must call it (it ends with a barrier)
template <uint32_t T> __host__ __device__ constexpr int grid_smem_bytes() {
  return GridOf<T>::words64 * 8 + GridOf<T>::words32 * 4 + (GridOf<T>::signs ? 128 : 0);
}
template <uint32_t T> __device__ inline Grids stage_grids(uint8_t* smem) {
  Grids g{nullptr, nullptr, nullptr};
  if constexpr (GridOf<T>::words64 > 0) {
    uint64_t* d = (uint64_t*) smem;
    const uint64_t* s = global_grid64<T>();
    for (int i = threadIdx.x; i < GridOf<T>::words64; i += blockDim.x) d[i] = s[i];
    g.g64 = d, smem += GridOf<T>::words64 * 8;
  }
  if constexpr (GridOf<T>::words32 > 0) {
    uint32_t* d = (uint32_t*) smem;
    for (int i = threadIdx.x; i < GridOf<T>::words32; i += blockDim.x) d[i] = osmos_grid_iq3xxs[i];
    g.g32 = d, smem += GridOf<T>::words32 * 4;
  }
  if constexpr (GridOf<T>::signs) {
    for (int i = threadIdx.x; i < 128; i += blockDim.x) smem[i] = osmos_ksigns[i];
    g.sign = smem;
  }
  if constexpr (grid_smem_bytes<T>() > 0) __syncthreads();
  return g;
}

__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, int g, int& sc, int& mn) {
  if (g < 4) {
    sc = s[g] & 0x3F, mn = s[g + 4] & 0x3F;
  } else {
    sc = (s[g + 4] & 0x0F) | ((s[g - 4] >> 6) << 4), mn = (s[g + 4] >> 4) | ((s[g] >> 6) << 4);
  }
}

__device__ __forceinline__ float iq1m_scale(const uint8_t* b) {
  const uint32_t s0 = ld16(b + 48), s1 = ld16(b + 50), s2 = ld16(b + 52), s3 = ld16(b + 54);
  return half_value((s0 >> 12) | ((s1 >> 8) & 0x00F0) | ((s2 >> 4) & 0x0F00) | (s3 & 0xF000));
}

// an NVFP4 sub-block scale as ggml reads it: the byte 0x7F is zero, any other byte is read without its sign bit
__device__ __forceinline__ float ue4m3_value(uint32_t c) {
  const uint32_t mag = c & 0x7F;
  if (c == 0x7F) return 0.0f;
  if (mag >> 3) return __uint_as_float((mag << 20) + (120u << 23));
  return (float) mag * 0.001953125f;
}

__device__ __forceinline__ void grid_values8(uint64_t grid, uint32_t signs, float scale, float* v) {
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float x = mul_rn(scale, (float) (uint32_t) ((grid >> (8 * j)) & 0xFF));
    v[j] = (signs >> j) & 1 ? -x : x;
  }
}

// values 8k .. 8k + 7 of the block at b
template <uint32_t T> __device__ __forceinline__ void decode8(const uint8_t* b, int k, float* v, const Grids& g) {
  if constexpr (T == QTYPE_Q4_0) {
    const float d = half_value(ld16(b));
    const uint8_t* qs = b + 2 + (k % 2) * 8;
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = mul_rn(d, (float) ((int) ((qs[j] >> (4 * (k / 2))) & 0x0F) - 8));
  } else if constexpr (T == QTYPE_Q8_0) {
    const float d = half_value(ld16(b));
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = mul_rn((float) (int8_t) b[2 + k * 8 + j], d);
  } else if constexpr (T == QTYPE_Q4_K) {
    const int grp = k / 4, l0 = (k % 4) * 8;
    int sc, mn;
    q4k_scale_min(b + 4, grp, sc, mn);
    const float ds = mul_rn(half_value(ld16(b)), (float) sc), dm = mul_rn(half_value(ld16(b + 2)), (float) mn);
    const uint8_t* qs = b + 16 + (grp / 2) * 32 + l0;
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = __fsub_rn(mul_rn(ds, (float) ((qs[j] >> (4 * (grp % 2))) & 0x0F)), dm);
  } else if constexpr (T == QTYPE_Q2_K) {
    const int grp = k / 2, l0 = (k % 4) * 8, shift = 2 * ((k % 16) / 4);
    const uint8_t* qs = b + 16 + 32 * (k / 16) + l0;
    const float dl = mul_rn(half_value(ld16(b + 80)), (float) (b[grp] & 0x0F));
    const float ml = mul_rn(half_value(ld16(b + 82)), (float) (b[grp] >> 4));
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = __fsub_rn(mul_rn(dl, (float) ((qs[j] >> shift) & 0x03)), ml);
  } else if constexpr (T == QTYPE_IQ2_XXS) {
    const uint8_t* q = b + 2 + (k / 4) * 8;
    const uint32_t aux = ld32(q + 4);
    const float db = mul_rn(mul_rn(half_value(ld16(b)), 0.5f + (float) (aux >> 28)), 0.25f);
    grid_values8(g.g64[q[k % 4]], g.sign[(aux >> (7 * (k % 4))) & 0x7F], db, v);
  } else if constexpr (T == QTYPE_IQ2_XS) {
    const uint32_t q = ld16(b + 2 + 2 * k);
    const int s = (b[66 + k / 4] >> (4 * ((k / 2) % 2))) & 0x0F;
    const float db = mul_rn(mul_rn(half_value(ld16(b)), 0.5f + (float) s), 0.25f);
    grid_values8(g.g64[q & 511], g.sign[q >> 9], db, v);
  } else if constexpr (T == QTYPE_IQ2_S) {
    const int s = (b[74 + k / 4] >> (4 * ((k / 2) % 2))) & 0x0F;
    const float db = mul_rn(mul_rn(half_value(ld16(b)), 0.5f + (float) s), 0.25f);
    const uint32_t idx = b[2 + k] | ((b[66 + k / 4] >> (2 * (k % 4))) & 0x03) << 8;
    grid_values8(g.g64[idx], b[34 + k], db, v);
  } else if constexpr (T == QTYPE_IQ3_XXS) {
    const uint8_t* q = b + 2 + (k / 4) * 8 + (k % 4) * 2;
    const uint32_t aux = ld32(b + 66 + (k / 4) * 4);
    const float db = mul_rn(mul_rn(half_value(ld16(b)), 0.5f + (float) (aux >> 28)), 0.5f);
    const uint64_t grid = (uint64_t) g.g32[q[0]] | (uint64_t) g.g32[q[1]] << 32;
    grid_values8(grid, g.sign[(aux >> (7 * (k % 4))) & 0x7F], db, v);
  } else if constexpr (T == QTYPE_IQ1_S) {
    const uint32_t h = ld16(b + 34 + 2 * (k / 4));
    const float dl = mul_rn(half_value(ld16(b)), (float) (2 * (int) ((h >> 12) & 0x07) + 1));
    const float delta = h & 0x8000 ? -0.125f : 0.125f;
    const uint64_t grid = g.g64[b[2 + k] | ((h >> (3 * (k % 4))) & 0x07) << 8];
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = mul_rn(dl, __fadd_rn((float) (int8_t) (grid >> (8 * j)), delta));
  } else if constexpr (T == QTYPE_IQ1_M) {
    const uint64_t sc = ld64(b + 48);
    const int s = (int) ((sc >> (16 * (k / 8) + 3 * ((k / 2) % 4))) & 0x07);
    const float dl = mul_rn(iq1m_scale(b), (float) (2 * s + 1));
    const uint32_t h = (b[32 + k / 2] >> (4 * (k % 2))) & 0x0F;
    const float delta = h & 0x08 ? -0.125f : 0.125f;
    const uint64_t grid = g.g64[b[k] | (h & 0x07) << 8];
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = mul_rn(dl, __fadd_rn((float) (int8_t) (grid >> (8 * j)), delta));
  } else if constexpr (T == QTYPE_MXFP4) {
    // 2^(e - 128): F32's exponent field e - 1, the two lowest (e = 0, 1) its subnormals 2^-128, 2^-127
    const uint32_t e = b[0];
    const float dd = __uint_as_float(e >= 2 ? (e - 1) << 23 : 0x00200000u << e);
    const uint8_t* qs = b + 1 + (k % 2) * 8;
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = mul_rn(dd, (float) osmos_e2m1_doubled[(qs[j] >> (4 * (k / 2))) & 0x0F]);
  } else if constexpr (T == QTYPE_NVFP4) {
    const float d = mul_rn(ue4m3_value(b[k / 2]), 0.5f);
    const uint8_t* qs = b + 4 + (k / 2) * 8;
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = mul_rn(d, (float) osmos_e2m1_doubled[(qs[j] >> (4 * (k % 2))) & 0x0F]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// the int8 lane's view of a 32-value sub-block (the arithmetic contract: kernels/lane.h:43-66 in the reference)
// ---------------------------------------------------------------------------------------------------------------
struct LaneCodes {
  int w[8];      // 32 int8 codes, 4 a word, value order
  int delta[4];  // IQ1: +-1 a chunk of 8 (the weight is 8 * grid + delta, in eighths); else 0
  int s21[2];    // a half's integer scale factor in eighths: 2s + 1 (IQ3_XXS: 2 (2s + 1); Q2_K: 8 sc)
  float d;       // the block's f16 scale
  int m8[2];     // Q2_K: a half's 8 m
  float dmin;    // Q2_K
};

// 4 sign bits -> 4 byte masks (0xFF where the bit is set)
__device__ __forceinline__ uint32_t byte_mask4(uint32_t bits) {
  return (((bits & 0xFu) * 0x00204081u) & 0x01010101u) * 0xFFu;
}
template <uint32_t T> constexpr bool kLaneIq1 = (T == QTYPE_IQ1_S || T == QTYPE_IQ1_M);
template <uint32_t T> constexpr bool kLanePlain = (T == QTYPE_Q4_0 || T == QTYPE_Q8_0);

// How a block's bytes are read: through a pointer (global or shared memory, 2-byte aligned at best) ...
struct PtrReader {
  const uint8_t* b;
  __device__ __forceinline__ uint32_t u8(int o) const { return b[o]; }
  __device__ __forceinline__ uint32_t u16(int o) const { return ld16(b + o); }
  __device__ __forceinline__ uint32_t u32(int o) const { return ld32(b + o); }
  __device__ __forceinline__ uint64_t u64(int o) const { return ld64(b + o); }
};
// ... or out of registers: the block's bytes were loaded as NW aligned 32-bit words, the block starting A bytes
// (0 or 2) into the first one. Every offset a decoder asks for is a compile-time constant once its loops are
// unrolled, so each read is one shift / byte-permute of a named register.
template <int NW, int A>
struct WordWindow {
  uint32_t w[NW];
  __device__ __forceinline__ uint32_t u8(int o) const { const int p = o + A; return __byte_perm(w[p >> 2], 0, 0x4440 + (p & 3)); }
  __device__ __forceinline__ uint32_t u16(int o) const { const int p = o + A; return __byte_perm(w[p >> 2], 0, (p & 2) ? 0x4432 : 0x4410); }
  __device__ __forceinline__ uint32_t u32(int o) const {
    const int p = o + A;
    return (p & 2) ? __funnelshift_r(w[p >> 2], w[(p >> 2) + 1], 16) : w[p >> 2];
  }
  __device__ __forceinline__ uint64_t u64(int o) const { return (uint64_t) u32(o) | (uint64_t) u32(o + 4) << 32; }
};

// How the codebooks are looked up: plain tables (one copy) ...
struct PlainLuts {
  Grids g;
  __device__ __forceinline__ uint64_t grid64(uint32_t i) const { return g.g64[i]; }
  __device__ __forceinline__ uint32_t grid32(uint32_t i) const { return g.g32[i]; }
  __device__ __forceinline__ void sign_masks(uint32_t s7, uint32_t& m0, uint32_t& m1) const {
    const uint32_t s = g.sign[s7];
    m0 = byte_mask4(s), m1 = byte_mask4(s >> 4);
  }
  __device__ __forceinline__ uint4 sign_masks4(uint32_t s7) const {
    uint32_t m0, m1;
    sign_masks(s7, m0, m1);
    return make_uint4(m0, m1, m0 & 0x01010101u, m1 & 0x01010101u);
  }
};

// 8 unsigned grid bytes negated where the mask bytes are 0xFF, as two words of int8: (v ^ m) + (m & 1) a byte - no
// byte of an IQ2 / IQ3 grid is 0, so no carry crosses a byte
__device__ __forceinline__ void apply_masks(uint64_t grid, uint32_t m0, uint32_t m1, int& lo, int& hi) {
  lo = (int) (((uint32_t) grid ^ m0) + (m0 & 0x01010101u));
  hi = (int) (((uint32_t) (grid >> 32) ^ m1) + (m1 & 0x01010101u));
}

// the same with the masks' "+ 1" words (m & 0x01010101) already at hand
__device__ __forceinline__ void apply_masks_carry(uint32_t g0, uint32_t g1, uint4 m, int& lo, int& hi) {
  lo = (int) ((g0 ^ m.x) + m.z), hi = (int) ((g1 ^ m.y) + m.w);
}

// IQ1_M's f16 scale out of its four scale words
template <class R> __device__ __forceinline__ float iq1m_scale_rd(const R& rd) {
  const uint32_t s0 = rd.u16(48), s1 = rd.u16(50), s2 = rd.u16(52), s3 = rd.u16(54);
  return half_value((s0 >> 12) | ((s1 >> 8) & 0x00F0) | ((s2 >> 4) & 0x0F00) | (s3 & 0xF000));
}

// sub-block j (32 values) of the block read through rd, its codebooks through lut
template <uint32_t T, class R, class L>
__device__ __forceinline__ void lane_codes_rd(const R& rd, int j, LaneCodes& c, const L& lut) {
  if constexpr (T == QTYPE_IQ2_XXS) {
    const uint32_t aux = rd.u32(2 + 8 * j + 4);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint64_t grid = lut.grid64(rd.u8(2 + 8 * j + k));
      apply_masks_carry((uint32_t) grid, (uint32_t) (grid >> 32), lut.sign_masks4((aux >> (7 * k)) & 0x7F), c.w[2 * k], c.w[2 * k + 1]);
    }
    c.s21[0] = c.s21[1] = 2 * (int) (aux >> 28) + 1;
    c.d = half_value(rd.u16(0));
  } else if constexpr (T == QTYPE_IQ2_XS) {
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint32_t q = rd.u16(2 + 2 * (4 * j + k));
      const uint64_t grid = lut.grid64(q & 511);
      apply_masks_carry((uint32_t) grid, (uint32_t) (grid >> 32), lut.sign_masks4(q >> 9), c.w[2 * k], c.w[2 * k + 1]);
    }
    const uint32_t s = rd.u8(66 + j);
    c.s21[0] = 2 * (int) (s & 0x0F) + 1, c.s21[1] = 2 * (int) (s >> 4) + 1;
    c.d = half_value(rd.u16(0));
  } else if constexpr (T == QTYPE_IQ2_S) {
    const uint32_t qh = rd.u8(66 + j);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int kk = 4 * j + k;
      const uint32_t sg = rd.u8(34 + kk);
      apply_masks(lut.grid64(rd.u8(2 + kk) | ((qh >> (2 * k)) & 0x03) << 8), byte_mask4(sg), byte_mask4(sg >> 4),
                  c.w[2 * k], c.w[2 * k + 1]);
    }
    const uint32_t s = rd.u8(74 + j);
    c.s21[0] = 2 * (int) (s & 0x0F) + 1, c.s21[1] = 2 * (int) (s >> 4) + 1;
    c.d = half_value(rd.u16(0));
  } else if constexpr (T == QTYPE_IQ3_XXS) {
    const uint32_t aux = rd.u32(66 + 4 * j);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      apply_masks_carry(lut.grid32(rd.u8(2 + 8 * j + 2 * k)), lut.grid32(rd.u8(2 + 8 * j + 2 * k + 1)),
                        lut.sign_masks4((aux >> (7 * k)) & 0x7F), c.w[2 * k], c.w[2 * k + 1]);
    }
    c.s21[0] = c.s21[1] = 2 * (2 * (int) (aux >> 28) + 1);
    c.d = half_value(rd.u16(0));
  } else if constexpr (T == QTYPE_IQ1_S) {
    const uint32_t h = rd.u16(34 + 2 * j);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint64_t grid = lut.grid64(rd.u8(2 + 4 * j + k) | ((h >> (3 * k)) & 0x07) << 8);
      c.w[2 * k] = (int) (uint32_t) grid, c.w[2 * k + 1] = (int) (uint32_t) (grid >> 32);
      c.delta[k] = h & 0x8000 ? -1 : 1;
    }
    c.s21[0] = c.s21[1] = 2 * (int) ((h >> 12) & 0x07) + 1;
    c.d = half_value(rd.u16(0));
  } else if constexpr (T == QTYPE_IQ1_M) {
    const uint64_t sc = rd.u64(48);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int kk = 4 * j + k;
      const uint32_t h = (rd.u8(32 + kk / 2) >> (4 * (kk % 2))) & 0x0F;
      const uint64_t grid = lut.grid64(rd.u8(kk) | (h & 0x07) << 8);
      c.w[2 * k] = (int) (uint32_t) grid, c.w[2 * k + 1] = (int) (uint32_t) (grid >> 32);
      c.delta[k] = h & 0x08 ? -1 : 1;
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int kk = 4 * j + 2 * h;
      c.s21[h] = 2 * (int) ((sc >> (16 * (kk / 8) + 3 * ((kk / 2) % 4))) & 0x07) + 1;
    }
    c.d = iq1m_scale_rd(rd);
  } else if constexpr (T == QTYPE_Q2_K) {
    const int base = 16 + 32 * (j / 4), shift = 2 * (j % 4);
#pragma unroll
    for (int t = 0; t < 8; t++) c.w[t] = (int) ((rd.u32(base + 4 * t) >> shift) & 0x03030303u);
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t sm = rd.u8(2 * j + h);
      c.s21[h] = 8 * (int) (sm & 0x0F), c.m8[h] = 8 * (int) (sm >> 4);
    }
    c.d = half_value(rd.u16(80)), c.dmin = half_value(rd.u16(82));
  } else if constexpr (T == QTYPE_Q4_0) {
    // value i < 16 is byte i's low nibble, 16 + i its high nibble, each less 8: as signed bytes without a borrow
    // between them ((n | 0x80) - 8) ^ 0x80. (j: the 18-byte block's index in the bytes rd holds)
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const uint32_t raw = rd.u32(18 * j + 2 + 4 * t);
      c.w[t] = (int) ((((raw & 0x0F0F0F0Fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
      c.w[4 + t] = (int) (((((raw >> 4) & 0x0F0F0F0Fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
    }
    c.d = half_value(rd.u16(18 * j));
  } else if constexpr (T == QTYPE_Q8_0) {
#pragma unroll
    for (int t = 0; t < 8; t++) c.w[t] = (int) rd.u32(34 * j + 2 + 4 * t);
    c.d = half_value(rd.u16(34 * j));
  }
}

// sub-block j (32 values) of the block at b (for the 32-value types j is 0: b is the block itself)
template <uint32_t T> __device__ __forceinline__ void lane_codes(const uint8_t* b, int j, LaneCodes& c, const Grids& g) {
  lane_codes_rd<T>(PtrReader{b}, j, c, PlainLuts{g});
}

__device__ __forceinline__ float lane_part(float d, int s21, int isum) {
  return mul_rn(mul_rn(mul_rn(d, (float) s21), 0.125f), (float) isum);
}

// a half's exact integer sum against x's words 4h .. 4h + 3 (IQ1: 8 (grid . x) + delta (sum of x) a chunk)
template <uint32_t T> __device__ __forceinline__ void lane_half(const LaneCodes& c, const int* x, int h, int& isum, int& xsum) {
  int s = 0, sx = 0;
#pragma unroll
  for (int k = 2 * h; k < 2 * h + 2; k++) {
    const int gx = __dp4a(c.w[2 * k + 1], x[2 * k + 1], __dp4a(c.w[2 * k], x[2 * k], 0));
    if constexpr (kLaneIq1<T> || T == QTYPE_Q2_K) {
      const int cx = __dp4a(0x01010101, x[2 * k + 1], __dp4a(0x01010101, x[2 * k], 0));
      sx += cx;
      s += kLaneIq1<T> ? 8 * gx + c.delta[k] * cx : gx;
    } else {
      s += gx;
    }
  }
  isum = s, xsum = sx;
}

// the sub-block's value before x's scale: each half's integer dot, then the contract's products, the halves added
template <uint32_t T> __device__ __forceinline__ float lane_block_sum(const LaneCodes& c, const int* x) {
  int i0, i1, x0, x1;
  lane_half<T>(c, x, 0, i0, x0);
  lane_half<T>(c, x, 1, i1, x1);
  if constexpr (kLanePlain<T>) {
    return mul_rn(c.d, (float) (i0 + i1));
  } else if constexpr (T == QTYPE_Q2_K) {
    const float p0 = __fsub_rn(lane_part(c.d, c.s21[0], i0), lane_part(c.dmin, c.m8[0], x0));
    const float p1 = __fsub_rn(lane_part(c.d, c.s21[1], i1), lane_part(c.dmin, c.m8[1], x1));
    return __fadd_rn(p0, p1);
  } else {
    return __fadd_rn(lane_part(c.d, c.s21[0], i0), lane_part(c.d, c.s21[1], i1));
  }
}

// the lane's exp and activation (kernels/lane.h:17-41, 69-75 in the reference), operation for operation
__device__ __forceinline__ float lane_exp(float x) {
  if (x > 88.72283905f) return __int_as_float(0x7F800000);
  const float k = rintf(mul_rn(x, 1.44269504089f));
  float r = __fmaf_rn(-k, 0.693145751953125f, x);
  r = __fmaf_rn(-k, 1.428606765330187e-06f, r);
  float p = 1.0f / 5040.0f;
  p = __fmaf_rn(p, r, 1.0f / 720.0f);
  p = __fmaf_rn(p, r, 1.0f / 120.0f);
  p = __fmaf_rn(p, r, 1.0f / 24.0f);
  p = __fmaf_rn(p, r, 1.0f / 6.0f);
  p = __fmaf_rn(p, r, 0.5f);
  p = __fmaf_rn(p, r, 1.0f);
  p = __fmaf_rn(p, r, 1.0f);
  return ldexpf(p, (int) k);
}

__device__ __forceinline__ float lane_swiglu(float gate, float up, float lim, float scale) {
  const float gv = fminf(gate, lim), uv = fminf(fmaxf(up, -lim), lim);
  return mul_rn(mul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, lane_exp(-gv))), uv), scale);
}

}  // namespace osmos
