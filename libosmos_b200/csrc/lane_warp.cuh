// What a lane kernel whose warps read a row with L lanes needs (lane_ring.cu): a lane's view of its
// sub-block of a superblock in shared memory, and IQ3_XXS's sums without negated codes.
#pragma once
#include "lane_staged.cuh"

namespace osmos {
namespace lanes {

using namespace tma;
using staged::RepLuts2;

// a superblock's bytes through shared-memory loads at run-time offsets (2-byte aligned at best)
struct SmemReader {
  uint32_t b;
  __device__ __forceinline__ uint32_t u8(int o) const { return lds8(b + o); }
  __device__ __forceinline__ uint32_t u16(int o) const { return lds16(b + o); }
  __device__ __forceinline__ uint32_t u32(int o) const { return lds16(b + o) | lds16(b + o + 2) << 16; }
  __device__ __forceinline__ uint64_t u64(int o) const { return (uint64_t) u32(o) | (uint64_t) u32(o + 4) << 32; }
};

// What of a superblock a lane reads, worked out once: the lane's sub-block index j is the same for all its blocks,
// and so is its superblocks' alignment (a row is a multiple of 4 bytes, the lane's superblocks an even count apart)
struct LaneAt {
  uint32_t j;     // the sub-block
  uint32_t qoff;  // IQ3_XXS: the aligned word holding the sub-block's first grid index, from the superblock's start
  uint32_t sh;    // IQ3_XXS: 16 when that index lies mid-word (an aligned superblock), else 0
};

// sub-block at.j of the superblock at shared address sb
template <uint32_t T>
__device__ __forceinline__ void sub_codes(uint32_t sb, const LaneAt& at, LaneCodes& c, const RepLuts2<T>& lut) {
  if constexpr (T == QTYPE_IQ3_XXS) {
    // the 8 grid indices and the sign / scale word, each out of the aligned words around it: both lie 2 mod 4 bytes
    // into the superblock, so they start mid-word when the superblock is aligned and on a word when it is not
    const uint32_t sh = at.sh, al = sb + at.qoff;
    const uint32_t q0 = lds32(al), q1 = lds32(al + 4), q2 = lds32(al + 8);
    const uint32_t ala = al + 64u - 4u * at.j;
    const uint32_t aux = __funnelshift_r(lds32(ala), lds32(ala + 4), sh);
    const uint32_t w[2] = {__funnelshift_r(q0, q1, sh), __funnelshift_r(q1, q2, sh)};
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint32_t i0 = __byte_perm(w[k >> 1], 0, 0x4440 + 2 * (k & 1)), i1 = __byte_perm(w[k >> 1], 0, 0x4441 + 2 * (k & 1));
      const uint2 mm = lut.sign_masks2((aux >> (7 * k)) & 0x7F);
      c.w[2 * k] = negated4(lut.grid32(i0), mm.x, mm.x & kOnes), c.w[2 * k + 1] = negated4(lut.grid32(i1), mm.y, mm.y & kOnes);
    }
    c.s21[0] = c.s21[1] = 2 * (2 * (int) (aux >> 28) + 1);
    c.d = half_value(lds16(sb));
  } else {
    lane_codes_rd<T>(SmemReader{sb}, (int) at.j, c, lut);
  }
}

// IQ3_XXS's block sums without negating a code: the signed dot sum s_i g_i x_i is dp4a(g, x) - 2 dp4a(g & m, x) (m the
// byte mask of the negative values), so the mask costs one AND a word and a second dp4a a token instead of an XOR,
// an addition and a carry word - the integer pipe is the busier one here. Exact integers, the contract's products:
// the same bits as lane_block_sum.
template <int NTL, int NT, int NB>
__device__ __forceinline__ void iq3_block_sums(uint32_t sb, const LaneAt& at, const RepLuts2<QTYPE_IQ3_XXS>& lut,
                                               const int (&xq)[NT][NB][8], int k, float* out) {
  const uint32_t sh = at.sh, al = sb + at.qoff;
  const uint32_t q0 = lds32(al), q1 = lds32(al + 4), q2 = lds32(al + 8);
  const uint32_t ala = al + 64u - 4u * at.j;
  const uint32_t aux = __funnelshift_r(lds32(ala), lds32(ala + 4), sh);
  const uint32_t w[2] = {__funnelshift_r(q0, q1, sh), __funnelshift_r(q1, q2, sh)};
  int pos[NTL][2], neg[NTL][2];  // a half's dots: all values, and the negative ones
#pragma unroll
  for (int t = 0; t < NTL; t++) pos[t][0] = pos[t][1] = neg[t][0] = neg[t][1] = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const uint32_t i0 = __byte_perm(w[c >> 1], 0, 0x4440 + 2 * (c & 1)), i1 = __byte_perm(w[c >> 1], 0, 0x4441 + 2 * (c & 1));
    const uint2 mm = lut.sign_masks2((aux >> (7 * c)) & 0x7F);
    const int g0 = (int) lut.grid32(i0), g1 = (int) lut.grid32(i1);
    const int n0 = g0 & (int) mm.x, n1 = g1 & (int) mm.y;
#pragma unroll
    for (int t = 0; t < NTL; t++) {
      pos[t][c >> 1] = __dp4a(g1, xq[t][k][2 * c + 1], __dp4a(g0, xq[t][k][2 * c], pos[t][c >> 1]));
      neg[t][c >> 1] = __dp4a(n1, xq[t][k][2 * c + 1], __dp4a(n0, xq[t][k][2 * c], neg[t][c >> 1]));
    }
  }
  const int s21 = 2 * (2 * (int) (aux >> 28) + 1);
  const float d = half_value(lds16(sb));
#pragma unroll
  for (int t = 0; t < NTL; t++)
    out[t] = __fadd_rn(lane_part(d, s21, pos[t][0] - 2 * neg[t][0]), lane_part(d, s21, pos[t][1] - 2 * neg[t][1]));
}

// IQ1_M's block sums from aligned reads: a 56-byte superblock starts on 8 bytes wherever its row starts on 16, so the
// sub-block's four index bytes are one word, its four (index top, delta sign) nibbles one half-word and the
// superblock's scale words one 8-byte read - where the field reader goes a byte or a half-word at a time. A chunk's
// integer sum is the contract's 8 (grid . x) + delta (sum of x) with delta +-1; exact integers, the same products and
// order as lane_block_sum: the same bits.
template <int NTL, int NT, int NB>
__device__ __forceinline__ void iq1m_block_sums(uint32_t sb, const LaneAt& at, const RepLuts2<QTYPE_IQ1_M>& lut,
                                                const int (&xq)[NT][NB][8], int k, float* out) {
  const uint32_t j = at.j;
  const uint32_t qs = lds32(sb + 4u * j), qh = lds16(sb + 32u + 2u * j);
  const uint2 sc = lds64(sb + 48u);
  // the superblock's F16 scale lies in the four scale words' top nibbles; this sub-block's two 3-bit scales in word j / 2
  const float d = half_value(((sc.x >> 12) & 0x000Fu) | ((sc.x >> 24) & 0x00F0u) | ((sc.y >> 4) & 0x0F00u) | ((sc.y >> 16) & 0xF000u));
  const uint32_t fields = ((j & 4u ? sc.y : sc.x) >> (16u * ((j >> 1) & 1u))) >> (6u * (j & 1u));
  const int s21[2] = {2 * (int) (fields & 7u) + 1, 2 * (int) ((fields >> 3) & 7u) + 1};
  int sum[NTL][2];
#pragma unroll
  for (int t = 0; t < NTL; t++) sum[t][0] = sum[t][1] = 0;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    const uint64_t g = lut.grid64(((qs >> (8 * c)) & 0xFFu) | ((qh >> (4 * c)) & 7u) << 8);
    const int g0 = (int) (uint32_t) g, g1 = (int) (uint32_t) (g >> 32);
    const int delta = (qh >> (4 * c + 3)) & 1u ? -1 : 1;
#pragma unroll
    for (int t = 0; t < NTL; t++) {
      const int gx = __dp4a(g1, xq[t][k][2 * c + 1], __dp4a(g0, xq[t][k][2 * c], 0));
      const int cx = __dp4a(0x01010101, xq[t][k][2 * c + 1], __dp4a(0x01010101, xq[t][k][2 * c], 0));
      sum[t][c >> 1] += 8 * gx + delta * cx;
    }
  }
#pragma unroll
  for (int t = 0; t < NTL; t++) out[t] = __fadd_rn(lane_part(d, s21[0], sum[t][0]), lane_part(d, s21[1], sum[t][1]));
}

}  // namespace lanes
}  // namespace osmos
