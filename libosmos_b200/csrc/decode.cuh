// GGUF block decoders for the device: a block's values as F32 (8 at a time), and a 32-value sub-block as packed
// int8 codes for the int8 lane. Every value is the bits gguf-py's dequantize gives (the same products, each rounded
// once); the block layouts are the GGUF's own, read where they lie.
//
// Replaces the reference's kernels/quant.h:65-362 (decode<T>) and kernels/q8.h:28-162 (codes<T>, block_sum<T>) with one
// field reader a type (sub_of, chunk_of) under both.
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
OSMOS_FMT(Q5_1, 7, 32, 24, 0) OSMOS_FMT(Q3_K, 11, 256, 110, 0) OSMOS_FMT(Q5_K, 13, 256, 176, 0)
OSMOS_FMT(Q6_K, 14, 256, 210, 0) OSMOS_FMT(IQ4_NL, 20, 32, 18, 0) OSMOS_FMT(IQ4_XS, 23, 256, 136, 0)
OSMOS_FMT(Q2_0, 42, 64, 18, 0) OSMOS_FMT(MXFP8, 43, 32, 33, 0)
// (the unquantized types: a "block" here is the 8 values the kernels decode at a time)
OSMOS_FMT(F32, 0, 8, 32, 0) OSMOS_FMT(BF16, 30, 8, 16, 0)
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

// ---------------------------------------------------------------------------------------------------------------
// How a block's bytes are read: through a pointer (global or shared memory, 2-byte aligned at best) ...
// ---------------------------------------------------------------------------------------------------------------
struct PtrReader {
  const uint8_t* b;
  __device__ __forceinline__ uint32_t u8(int o) const { return b[o]; }
  __device__ __forceinline__ uint32_t u16(int o) const { return ld16(b + o); }
  __device__ __forceinline__ uint32_t u32(int o) const { return ld32(b + o); }
  __device__ __forceinline__ uint64_t u64(int o) const { return ld64(b + o); }
  // four bytes at any offset (blocks of an odd size: MXFP4, MXFP8)
  __device__ __forceinline__ uint32_t u32b(int o) const { return b[o] | b[o + 1] << 8 | b[o + 2] << 16 | (uint32_t) b[o + 3] << 24; }
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
  __device__ __forceinline__ uint32_t u32b(int o) const {
    const int p = o + A;
    return (p & 3) ? __funnelshift_r(w[p >> 2], w[(p >> 2) + 1], 8 * (p & 3)) : w[p >> 2];
  }
};

// 4 sign bits -> 4 byte masks (0xFF where the bit is set)
__device__ __forceinline__ uint32_t byte_mask4(uint32_t bits) {
  return (((bits & 0xFu) * 0x00204081u) & 0x01010101u) * 0xFFu;
}

// How the codebooks are looked up: plain tables (one copy) ...
struct PlainLuts {
  Grids g;
  __device__ __forceinline__ uint64_t grid64(uint32_t i) const { return g.g64[i]; }
  __device__ __forceinline__ uint32_t grid32(uint32_t i) const { return g.g32[i]; }
  __device__ __forceinline__ uint4 sign_masks4(uint32_t s7) const {
    const uint32_t s = g.sign[s7], m0 = byte_mask4(s), m1 = byte_mask4(s >> 4);
    return make_uint4(m0, m1, m0 & 0x01010101u, m1 & 0x01010101u);
  }
};
// (... or replicated in shared memory: lane_staged.cuh's RepLuts, the same three calls)

// ---------------------------------------------------------------------------------------------------------------
// A block taken apart. Every consumer here - the F32 values of quant_dequant and the matvecs, the f16 tiles of the
// matrix products, the int8 lane's packed codes - starts from the same two steps, written once a type:
//   sub_of    what a 32-value stretch of a block says once for all its values (scale fields, index words), as read;
//   chunk_of  8 neighbouring values as eight signed bytes in two words (value order), codebook entries looked up and
//             signs applied, with the integer and F16 scale fields that belong to them - nothing multiplied yet.
// The codes are worked on a word (four of them) at a time: masks, shifts and byte permutes, never a byte loop. What
// the fields mean is the GGUF format's; which products make a value, and in which order they round, is said where
// they are made (chunk_values, lane_codes_rd).
// ---------------------------------------------------------------------------------------------------------------
constexpr uint32_t kLow4 = 0x0F0F0F0Fu, kLow2 = 0x03030303u, kOnes = 0x01010101u, kTops = 0x80808080u;

// the low four bits of `bits` as four bytes of 0 / 1
__device__ __forceinline__ uint32_t spread4(uint32_t bits) { return ((bits & 0xFu) * 0x00204081u) & kOnes; }
// four unsigned bytes (each below 128) less the bytes of n4 (each at most 127), as signed bytes: with the top bits
// set first no borrow leaves a byte
__device__ __forceinline__ int less4(uint32_t v, uint32_t n4) { return (int) (((v | kTops) - n4) ^ kTops); }
// four 4-bit codes, a byte each -> their entries of a 16-entry byte table held as four words: a byte permute of
// each half of the table, the code's top bit choosing between them
__device__ __forceinline__ int table16(uint32_t codes, uint32_t t0, uint32_t t1, uint32_t t2, uint32_t t3) {
  const uint32_t low = codes & 0x07070707u, two = low | low >> 4;  // bytes 0 and 2: a pair of selectors each
  const uint32_t sel = __byte_perm(two, 0, 0x4420);
  const uint32_t top = ((codes >> 3) & kOnes) * 0xFFu;
  return (int) ((__byte_perm(t0, t1, sel) & ~top) | (__byte_perm(t2, t3, sel) & top));
}
__device__ __forceinline__ int iq4nl4(uint32_t codes) {
  constexpr uint32_t t[4] = {OSMOS_IQ4NL_WORDS};
  return table16(codes, t[0], t[1], t[2], t[3]);
}
__device__ __forceinline__ int e2m1x2_4(uint32_t codes) {  // E2M1 doubled: 0 1 2 3 4 6 8 12 and their negatives
  constexpr uint32_t t[4] = {OSMOS_E2M1_WORDS};
  return table16(codes, t[0], t[1], t[2], t[3]);
}
// unsigned grid bytes negated where the mask bytes are 0xFF: (v ^ m) + (m & 1) a byte - no byte of an IQ2 / IQ3 grid
// is 0, so no carry leaves a byte
__device__ __forceinline__ int negated4(uint32_t g, uint32_t m, uint32_t m_ones) { return (int) ((g ^ m) + m_ones); }

// an NVFP4 sub-block scale as ggml reads it: the byte 0x7F is zero, any other byte is read without its sign bit
__device__ __forceinline__ float ue4m3_value(uint32_t c) {
  const uint32_t mag = c & 0x7F;
  if (c == 0x7F) return 0.0f;
  if (mag >> 3) return __uint_as_float((mag << 20) + (120u << 23));
  return (float) mag * 0.001953125f;
}
// an E4M3 code (torch's float8_e4m3fn: 0x7F / 0xFF are NaN, no infinities)
__device__ __forceinline__ float e4m3_value(uint32_t c) {
  const uint32_t sign = (c & 0x80u) << 24, mag = c & 0x7Fu;
  if (mag == 0x7Fu) return __uint_as_float(0x7FC00000u | sign);
  if (mag >> 3) return __uint_as_float(sign | ((mag << 20) + (120u << 23)));
  return __uint_as_float(sign | __float_as_uint((float) mag * 0.001953125f));
}
// 2^(e - bias) for an E8M0 byte, every value exact (the lowest are F32 subnormals; bias 127's e = 255 is 2^128: inf)
__device__ __forceinline__ float e8m0_value(uint32_t e, int bias) {
  const int x = (int) e - bias;  // the power
  if (x >= 128) return __uint_as_float(0x7F800000u);
  if (x >= -126) return __uint_as_float((uint32_t) (x + 127) << 23);
  return __uint_as_float(0x00400000u >> (-127 - x));
}

struct Sub {  // a 32-value stretch's shared fields: two words as read (a type's own meaning), the block's two F16s
  uint32_t a, b;
  float d, e;
};
struct Chunk {   // 8 values
  int lo, hi;    // their codes, signed bytes: values 0 .. 3 and 4 .. 7
  float d, e;    // the scale (and the second F16 field: dmin, Q5_1's m) that applies to them
  int s, m;      // the integer scale and minimum fields (IQ1: m the delta's sign, +-1)
};

// sub-block j of the block o bytes into what rd reads
template <uint32_t T, class R>
__device__ __forceinline__ Sub sub_of(const R& rd, int o, int j) {
  Sub s{0u, 0u, 0.0f, 0.0f};
  if constexpr (T == QTYPE_Q4_0 || T == QTYPE_Q8_0 || T == QTYPE_IQ4_NL || T == QTYPE_Q2_0) {
    s.d = half_value(rd.u16(o));
  } else if constexpr (T == QTYPE_Q5_1) {
    s.d = half_value(rd.u16(o)), s.e = half_value(rd.u16(o + 2)), s.a = rd.u32(o + 4);  // a: the 32 fifth bits
  } else if constexpr (T == QTYPE_MXFP4) {
    s.d = e8m0_value(rd.u8(o), 128);
  } else if constexpr (T == QTYPE_MXFP8) {
    s.d = e8m0_value(rd.u8(o), 127);
  } else if constexpr (T == QTYPE_NVFP4) {
    s.a = rd.u16(o + 2 * j);  // the two UE4M3 bytes of its two 16s
  } else if constexpr (T == QTYPE_Q4_K || T == QTYPE_Q5_K) {
    // twelve bytes hold eight 6-bit (scale, minimum) pairs: the first four whole in bytes 0 .. 7's low bits, the last
    // four split between bytes 8 .. 11's nibbles and the top bits of bytes 0 .. 7
    const uint32_t lo = rd.u8(o + 4 + (j & 3)), hi = rd.u8(o + 8 + (j & 3)), nib = rd.u8(o + 12 + (j & 3));
    s.a = j < 4 ? lo & 0x3Fu : (nib & 0x0Fu) | (lo >> 6) << 4;
    s.b = j < 4 ? hi & 0x3Fu : (nib >> 4) | (hi >> 6) << 4;
    s.d = half_value(rd.u16(o)), s.e = half_value(rd.u16(o + 2));
  } else if constexpr (T == QTYPE_Q2_K) {
    s.a = rd.u16(o + 2 * j);  // its two 16s' (scale, minimum) nibble pairs
    s.d = half_value(rd.u16(o + 80)), s.e = half_value(rd.u16(o + 82));
  } else if constexpr (T == QTYPE_Q3_K) {
    // sixteen 6-bit scales: low nibbles in bytes 0 .. 7 (scale g < 8 the low nibble of byte g, else the high one of
    // byte g - 8), the top two bits in bytes 8 .. 11 (scale g: bits 2 (g / 4) of byte 8 + g % 4); a, b: its two 16s'
    auto scale6 = [&](int g) -> uint32_t {
      const uint32_t low = g < 8 ? rd.u8(o + 96 + g) & 0x0Fu : rd.u8(o + 96 + g - 8) >> 4;
      return low | ((rd.u8(o + 104 + g % 4) >> (2 * (g / 4))) & 0x03u) << 4;
    };
    s.a = scale6(2 * j), s.b = scale6(2 * j + 1);
    s.d = half_value(rd.u16(o + 108));
  } else if constexpr (T == QTYPE_Q6_K) {
    s.a = rd.u16(o + 192 + 2 * j);  // its two 16s' signed scale bytes
    s.d = half_value(rd.u16(o + 208));
  } else if constexpr (T == QTYPE_IQ4_XS) {
    s.a = ((rd.u8(o + 4 + j / 2) >> (4 * (j & 1))) & 0x0Fu) | ((rd.u16(o + 2) >> (2 * j)) & 0x03u) << 4;  // the 6-bit scale
    s.d = half_value(rd.u16(o));
  } else if constexpr (T == QTYPE_IQ2_XXS) {
    s.a = rd.u32(o + 2 + 8 * j), s.b = rd.u32(o + 6 + 8 * j);  // four grid indices; four 7-bit signs and the scale
    s.d = half_value(rd.u16(o));
  } else if constexpr (T == QTYPE_IQ2_XS) {
    s.a = rd.u8(o + 66 + j);  // its two 16s' scale nibbles
    s.d = half_value(rd.u16(o));
  } else if constexpr (T == QTYPE_IQ2_S) {
    s.a = rd.u8(o + 66 + j), s.b = rd.u8(o + 74 + j);  // the indices' top two bits; the scale nibbles
    s.d = half_value(rd.u16(o));
  } else if constexpr (T == QTYPE_IQ3_XXS) {
    s.b = rd.u32(o + 66 + 4 * j);  // four 7-bit signs and the scale
    s.d = half_value(rd.u16(o));
  } else if constexpr (T == QTYPE_IQ1_S) {
    s.a = rd.u16(o + 34 + 2 * j);  // four 3-bit index tops, the scale, the delta's sign
    s.d = half_value(rd.u16(o));
  } else if constexpr (T == QTYPE_IQ1_M) {
    s.a = rd.u32(o + 48), s.b = rd.u32(o + 52);  // the block's four scale words; their top nibbles make its F16
    s.d = half_value(((s.a >> 12) & 0x000Fu) | ((s.a >> 24) & 0x00F0u) | ((s.b >> 4) & 0x0F00u) | ((s.b >> 16) & 0xF000u));
  }
  return s;
}

// chunk kk (0 .. 3) of that sub-block
template <uint32_t T, class R, class L>
__device__ __forceinline__ Chunk chunk_of(const R& rd, int o, int j, int kk, const Sub& sb, const L& lut) {
  Chunk c{0, 0, sb.d, sb.e, 0, 0};
  const int k = 4 * j + kk;  // the chunk's place in the block
  if constexpr (T == QTYPE_Q4_0 || T == QTYPE_IQ4_NL || T == QTYPE_Q5_1 || T == QTYPE_MXFP4) {
    // 16 bytes: value i < 16 a byte's low nibble, value 16 + i its high one
    const int at = o + (T == QTYPE_Q5_1 ? 8 : T == QTYPE_MXFP4 ? 1 : 2) + 8 * (kk & 1), sh = 4 * (kk >> 1);
    const uint32_t n0 = ((T == QTYPE_MXFP4 ? rd.u32b(at) : rd.u32(at)) >> sh) & kLow4;
    const uint32_t n1 = ((T == QTYPE_MXFP4 ? rd.u32b(at + 4) : rd.u32(at + 4)) >> sh) & kLow4;
    if constexpr (T == QTYPE_Q4_0) c.lo = less4(n0, 0x08080808u), c.hi = less4(n1, 0x08080808u);
    else if constexpr (T == QTYPE_IQ4_NL) c.lo = iq4nl4(n0), c.hi = iq4nl4(n1);
    else if constexpr (T == QTYPE_MXFP4) c.lo = e2m1x2_4(n0), c.hi = e2m1x2_4(n1);
    else {
      const uint32_t fifth = sb.a >> (8 * kk);
      c.lo = (int) (n0 | spread4(fifth) << 4), c.hi = (int) (n1 | spread4(fifth >> 4) << 4);
    }
  } else if constexpr (T == QTYPE_Q8_0) {
    c.lo = (int) rd.u32(o + 2 + 8 * kk), c.hi = (int) rd.u32(o + 6 + 8 * kk);
  } else if constexpr (T == QTYPE_MXFP8) {
    c.lo = (int) rd.u32b(o + 1 + 8 * kk), c.hi = (int) rd.u32b(o + 5 + 8 * kk);  // E4M3 codes, as they are
  } else if constexpr (T == QTYPE_NVFP4) {
    // a 16's 8 bytes: values 0 .. 7 the low nibbles, 8 .. 15 the high ones; half its UE4M3 scale
    const int at = o + 4 + 8 * (k >> 1), sh = 4 * (k & 1);
    c.lo = e2m1x2_4((rd.u32(at) >> sh) & kLow4), c.hi = e2m1x2_4((rd.u32(at + 4) >> sh) & kLow4);
    c.d = mul_rn(ue4m3_value((sb.a >> (8 * (kk >> 1))) & 0xFFu), 0.5f);
  } else if constexpr (T == QTYPE_Q2_0) {
    // two bytes: eight 2-bit codes, each less 1 (a byte's four codes 6 bits apart land a byte apart)
    const uint32_t w = rd.u16(o + 2 + 2 * k), x = w & 0xFFu, y = w >> 8;
    c.lo = less4((x | x << 6 | x << 12 | x << 18) & kLow2, kOnes), c.hi = less4((y | y << 6 | y << 12 | y << 18) & kLow2, kOnes);
  } else if constexpr (T == QTYPE_Q4_K || T == QTYPE_Q5_K) {
    // a pair of sub-blocks shares 32 bytes: the even one their low nibbles, the odd one the high
    const int at = o + (T == QTYPE_Q5_K ? 48 : 16) + 32 * (j >> 1) + 8 * kk, sh = 4 * (j & 1);
    uint32_t n0 = (rd.u32(at) >> sh) & kLow4, n1 = (rd.u32(at + 4) >> sh) & kLow4;
    if constexpr (T == QTYPE_Q5_K)  // the fifth bits: bit j of the 32 bytes at 16, a byte a position in the sub-block
      n0 |= ((rd.u32(o + 16 + 8 * kk) >> j) & kOnes) << 4, n1 |= ((rd.u32(o + 20 + 8 * kk) >> j) & kOnes) << 4;
    c.lo = (int) n0, c.hi = (int) n1, c.s = (int) sb.a, c.m = (int) sb.b;
  } else if constexpr (T == QTYPE_Q2_K) {
    // four sub-blocks share 32 bytes, two bits each
    const int at = o + 16 + 32 * (j >> 2) + 8 * kk, sh = 2 * (j & 3);
    c.lo = (int) ((rd.u32(at) >> sh) & kLow2), c.hi = (int) ((rd.u32(at + 4) >> sh) & kLow2);
    const uint32_t sm = sb.a >> (8 * (kk >> 1));
    c.s = (int) (sm & 0x0Fu), c.m = (int) ((sm >> 4) & 0x0Fu);
  } else if constexpr (T == QTYPE_Q3_K) {
    // two low bits as Q2_K's; the third from the 32 mask bytes at 0 (bit j of a position's byte), and without it 4 less
    const int at = o + 32 + 32 * (j >> 2) + 8 * kk, sh = 2 * (j & 3);
    const uint32_t h0 = (rd.u32(o + 8 * kk) >> j) & kOnes, h1 = (rd.u32(o + 4 + 8 * kk) >> j) & kOnes;
    c.lo = less4(((rd.u32(at) >> sh) & kLow2) | h0 << 2, 0x04040404u);
    c.hi = less4(((rd.u32(at + 4) >> sh) & kLow2) | h1 << 2, 0x04040404u);
    c.s = (int) (kk < 2 ? sb.a : sb.b) - 32;
  } else if constexpr (T == QTYPE_Q6_K) {
    // a half of the block (128 values): 64 bytes of low nibbles (sub-blocks 0, 1 the low ones, 2, 3 the high), 32 bytes
    // of top bit pairs (sub-block r at bits 2 r); the code less 32
    const int h = j >> 2, r = j & 3, at = o + 64 * h + 32 * (r & 1) + 8 * kk, top = o + 128 + 32 * h + 8 * kk;
    const uint32_t n0 = (rd.u32(at) >> (4 * (r >> 1))) & kLow4, n1 = (rd.u32(at + 4) >> (4 * (r >> 1))) & kLow4;
    const uint32_t t0 = (rd.u32(top) >> (2 * r)) & kLow2, t1 = (rd.u32(top + 4) >> (2 * r)) & kLow2;
    c.lo = less4(n0 | t0 << 4, 0x20202020u), c.hi = less4(n1 | t1 << 4, 0x20202020u);
    c.s = (int) (int8_t) (sb.a >> (8 * (kk >> 1)));
  } else if constexpr (T == QTYPE_IQ4_XS) {
    const int at = o + 8 + 16 * j + 8 * (kk & 1), sh = 4 * (kk >> 1);
    c.lo = iq4nl4((rd.u32(at) >> sh) & kLow4), c.hi = iq4nl4((rd.u32(at + 4) >> sh) & kLow4);
    c.s = (int) sb.a - 32;
  } else if constexpr (T == QTYPE_IQ2_XXS || T == QTYPE_IQ2_XS || T == QTYPE_IQ2_S || T == QTYPE_IQ3_XXS) {
    // eight codebook bytes and eight signs
    uint32_t g0, g1;
    uint4 m;
    if constexpr (T == QTYPE_IQ2_XXS) {
      const uint64_t g = lut.grid64((sb.a >> (8 * kk)) & 0xFFu);
      g0 = (uint32_t) g, g1 = (uint32_t) (g >> 32), m = lut.sign_masks4((sb.b >> (7 * kk)) & 0x7Fu), c.s = (int) (sb.b >> 28);
    } else if constexpr (T == QTYPE_IQ2_XS) {
      const uint32_t q = rd.u16(o + 2 + 2 * k);  // 9 bits of index, 7 of signs
      const uint64_t g = lut.grid64(q & 511u);
      g0 = (uint32_t) g, g1 = (uint32_t) (g >> 32), m = lut.sign_masks4(q >> 9), c.s = (int) ((sb.a >> (4 * (kk >> 1))) & 0x0Fu);
    } else if constexpr (T == QTYPE_IQ2_S) {
      const uint64_t g = lut.grid64(rd.u8(o + 2 + k) | ((sb.a >> (2 * kk)) & 0x03u) << 8);
      const uint32_t sg = rd.u8(o + 34 + k), m0 = byte_mask4(sg), m1 = byte_mask4(sg >> 4);  // the signs stored whole
      g0 = (uint32_t) g, g1 = (uint32_t) (g >> 32), m = make_uint4(m0, m1, m0 & kOnes, m1 & kOnes);
      c.s = (int) ((sb.b >> (4 * (kk >> 1))) & 0x0Fu);
    } else {
      g0 = lut.grid32(rd.u8(o + 2 + 8 * j + 2 * kk)), g1 = lut.grid32(rd.u8(o + 3 + 8 * j + 2 * kk));
      m = lut.sign_masks4((sb.b >> (7 * kk)) & 0x7Fu), c.s = (int) (sb.b >> 28);
    }
    c.lo = negated4(g0, m.x, m.z), c.hi = negated4(g1, m.y, m.w);
  } else if constexpr (T == QTYPE_IQ1_S) {
    const uint64_t g = lut.grid64(rd.u8(o + 2 + k) | ((sb.a >> (3 * kk)) & 0x07u) << 8);
    c.lo = (int) (uint32_t) g, c.hi = (int) (uint32_t) (g >> 32);
    c.s = (int) ((sb.a >> 12) & 0x07u), c.m = sb.a & 0x8000u ? -1 : 1;
  } else if constexpr (T == QTYPE_IQ1_M) {
    const uint32_t h = (rd.u8(o + 32 + (k >> 1)) >> (4 * (k & 1))) & 0x0Fu;  // the index's top three bits, the delta's sign
    const uint64_t g = lut.grid64(rd.u8(o + k) | (h & 0x07u) << 8);
    c.lo = (int) (uint32_t) g, c.hi = (int) (uint32_t) (g >> 32);
    // a 3-bit scale each 16 values: scale word k / 8, bits 3 ((k / 2) % 4)
    c.s = (int) (((k & 16 ? sb.b : sb.a) >> (16 * ((k >> 3) & 1) + 3 * ((k >> 1) & 3))) & 0x07u), c.m = h & 0x08u ? -1 : 1;
  }
  return c;
}

// the chunk's values as F32: the bits of gguf-py's dequantize - each product below rounded once, in this order
template <uint32_t T>
__device__ __forceinline__ void chunk_values(const Chunk& c, float* v) {
  auto code = [&](int i) -> float { return (float) (int) (int8_t) ((uint32_t) (i < 4 ? c.lo : c.hi) >> (8 * (i & 3))); };
  if constexpr (T == QTYPE_MXFP8) {
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = mul_rn(c.d, e4m3_value(((uint32_t) (i < 4 ? c.lo : c.hi) >> (8 * (i & 3))) & 0xFFu));
  } else if constexpr (T == QTYPE_Q5_1) {  // d q + m
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fadd_rn(mul_rn(c.d, code(i)), c.e);
  } else if constexpr (T == QTYPE_Q4_K || T == QTYPE_Q5_K || T == QTYPE_Q2_K) {  // (d s) q - (dmin m)
    const float ds = mul_rn(c.d, (float) c.s), dm = mul_rn(c.e, (float) c.m);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fsub_rn(mul_rn(ds, code(i)), dm);
  } else if constexpr (T == QTYPE_IQ1_S || T == QTYPE_IQ1_M) {  // (d (2 s + 1)) (grid +- 1/8)
    const float dl = mul_rn(c.d, (float) (2 * c.s + 1)), delta = c.m < 0 ? -0.125f : 0.125f;
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = mul_rn(dl, __fadd_rn(code(i), delta));
  } else {
    float scale = c.d;  // the plain blocks, MXFP4, NVFP4 (its half scale made with the chunk): d q
    if constexpr (T == QTYPE_Q3_K || T == QTYPE_Q6_K || T == QTYPE_IQ4_XS) scale = mul_rn(c.d, (float) c.s);  // (d s) q
    else if constexpr (T == QTYPE_IQ3_XXS) scale = mul_rn(mul_rn(c.d, 0.5f + (float) c.s), 0.5f);  // (d (s + 1/2) / 2) (+-grid)
    else if constexpr (T == QTYPE_IQ2_XXS || T == QTYPE_IQ2_XS || T == QTYPE_IQ2_S) scale = mul_rn(mul_rn(c.d, 0.5f + (float) c.s), 0.25f);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = mul_rn(scale, code(i));  // (a sign on the code is the sign on the product, bit for bit)
  }
}

// values 8k .. 8k + 7 of the block at b (for the unquantized types a "block" is 8 values)
template <uint32_t T> __device__ __forceinline__ void decode8(const uint8_t* b, int k, float* v, const Grids& g) {
  if constexpr (T == QTYPE_F32) {
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(ld32(b + 4 * i));
  } else if constexpr (T == QTYPE_BF16) {
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(ld16(b + 2 * i) << 16);
  } else {
    const PtrReader rd{b};
    const PlainLuts lut{g};
    const Sub sb = sub_of<T>(rd, 0, k >> 2);
    chunk_values<T>(chunk_of<T>(rd, 0, k >> 2, k & 3, sb, lut), v);
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
template <uint32_t T> constexpr bool kLaneIq1 = (T == QTYPE_IQ1_S || T == QTYPE_IQ1_M);
template <uint32_t T> constexpr bool kLanePlain = (T == QTYPE_Q4_0 || T == QTYPE_Q8_0);

// sub-block j (32 values) of the block read through rd, its codebooks through lut: the four chunks' codes as they
// are, the scale fields as the contract's integer factors. (The plain 32-value blocks: j is the block's index in the
// bytes rd holds.)
template <uint32_t T, class R, class L>
__device__ __forceinline__ void lane_codes_rd(const R& rd, int j, LaneCodes& c, const L& lut) {
  const int o = kLanePlain<T> ? Fmt<T>::bytes * j : 0, sj = kLanePlain<T> ? 0 : j;
  const Sub sb = sub_of<T>(rd, o, sj);
  c.d = sb.d, c.dmin = sb.e;
#pragma unroll
  for (int kk = 0; kk < 4; kk++) {
    const Chunk ch = chunk_of<T>(rd, o, sj, kk, sb, lut);
    c.w[2 * kk] = ch.lo, c.w[2 * kk + 1] = ch.hi;
    c.delta[kk] = kLaneIq1<T> ? ch.m : 0;
    if ((kk & 1) == 0) {  // a half's fields are its first chunk's
      if constexpr (T == QTYPE_Q2_K) c.s21[kk >> 1] = 8 * ch.s, c.m8[kk >> 1] = 8 * ch.m;
      else if constexpr (T == QTYPE_IQ3_XXS) c.s21[kk >> 1] = 2 * (2 * ch.s + 1);
      else c.s21[kk >> 1] = 2 * ch.s + 1;
    }
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
