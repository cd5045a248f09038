// The dense F32-activation matvec (mv_run / mv_strided, 1 .. 8 tokens) with the weights staged through shared memory
// by bulk copies. Same sums as mv.cu's kernel: of a row, lane l runs one fmaf chain over chunks l, l + 32, ... (8
// values a chunk, in value order), then the xor tree 16, 8, 4, 2, 1.
//
// A block takes a contiguous run of rows and keeps the tokens' x in shared memory. Its 16 warps do not meet again
// after that: each warp owns a ring of slots (a slot: RW whole rows, one bulk copy, one mbarrier), issues its own
// copies, and refills a slot as soon as it has summed it - so there is no block-wide barrier in the loop, and a
// block holds 16 x (slots - 1) copies in flight. Plain 32-value blocks are decoded with one byte-permute and one fmaf a
// value (see scaled4); the other types go through the same decode8 as the generic kernel.
//
// Two kernels. One token and rows of at most 2048 values (the decode step's usual shape): every lane keeps its 64
// values of x in registers for the whole launch, so shared memory serves only the weights (mv_regx_kernel). Else x
// lies in shared memory and is read a chunk at a time (mv_staged_kernel; up to eight tokens, each its own chain of
// the same order, so a token's bits do not depend on how many ride along).
#include "mv_staged_api.h"

#include "decode.cuh"
#include "dispatch.cuh"
#include "tma.cuh"

namespace osmos {
namespace mvs {
namespace {

using namespace tma;

constexpr int kWarps = 16, kThreads = kWarps * kWarp;
constexpr int kMaxSlots = 4;
// dynamic shared memory a block may ask for: 227 KB less the type's static tables and the barriers
template <uint32_t T> constexpr uint32_t kSmemLimit = 226u * 1024u - (uint32_t) ((grid_smem_bytes<T>() + 1023) / 1024 * 1024);

__device__ uint32_t g_status;

struct Args {
  const uint8_t* w;
  const float* x;
  float* y;
  uint32_t rows, cols, xs, ys, n_tok;
  uint32_t slots, slot_bytes, ring_off, units;
  uint32_t* status;
  // grouped forms: blockIdx.y is the entry
  const uint8_t* const* wt;
  const int32_t *cnt, *xrow;
  uint32_t x_mat, x_div, cnt_lo, cnt_hi;  // an entry of this launch has cnt_lo .. cnt_hi tokens (the others belong to another
                                          // launch); of more than NT, the first NT are served
};

// A grouped launch's block finds its entry: false when the entry is not this launch's (nothing read or written).
// Called after pdl_wait: the tables may be the output of the kernel ahead.
template <int NT>
__device__ __forceinline__ bool entry_of_block(const Args& a, const uint8_t*& w, const float*& x, float*& y, uint32_t& n_tok) {
  const uint32_t m = blockIdx.y;
  if (a.cnt) {
    const int32_t c = a.cnt[m];
    if (c < (int32_t) a.cnt_lo || c > (int32_t) a.cnt_hi) return false;
    const uint64_t r0 = (uint64_t) a.xrow[m];
    x = a.x + r0 * a.xs, y = a.y + r0 * a.ys, n_tok = (uint32_t) c < (uint32_t) NT ? (uint32_t) c : (uint32_t) NT;
  } else {
    x = a.x + (uint64_t) (m / a.x_div) * a.x_mat, y = a.y + (uint64_t) m * a.rows, n_tok = 1;
  }
  w = a.wt[m];
  if ((uintptr_t) w & 15u) {  // such a matrix cannot be copied in bulk: reported, its rows left alone
    if (threadIdx.x == 0) atomicOr(a.status, 2u);
    return false;
  }
  return true;
}

// Small integers reach F32 without a conversion instruction: byte j of `bytes` (a value n < 256) placed in bits 8 .. 15
// of 0x47000000 is the F32 32768 + n, one byte-permute.
template <int J> __device__ __forceinline__ float biased(uint32_t bytes) {
  return __uint_as_float(__byte_perm(bytes, 0x47000000u, 0x7404 | (J << 4)));
}

// d (n - bias) for the four bytes n of `bytes`, each one fmaf: d (32768 + n) - d (32768 + bias), where the second
// product `c` is exact (d has 11 significant bits, 32768 + bias at most 13) and so is the difference - the same bits
// as mul_rn(d, (float) (n - bias)), whose product is exact too.
__device__ __forceinline__ void scaled4(uint32_t bytes, float d, float c, float* v) {
  v[0] = __fmaf_rn(d, biased<0>(bytes), c), v[1] = __fmaf_rn(d, biased<1>(bytes), c);
  v[2] = __fmaf_rn(d, biased<2>(bytes), c), v[3] = __fmaf_rn(d, biased<3>(bytes), c);
}

// Two F32 fused multiply-adds in one instruction (sm_100's packed F32 pipe): element by element the same IEEE
// operation as fmaf, so the same bits - one issue slot for two rows' chains instead of two.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
template <uint32_t T> constexpr bool kPlainPair = (T == QTYPE_Q4_0 || T == QTYPE_Q8_0);

// ---- what of a row a lane reads, worked out once: the lane's chunk of each 256-value stretch is at a fixed place ----
template <uint32_t T> struct LanePlan {  // any type: decode8 through a pointer
  static constexpr uint32_t kStretch = Fmt<T>::bytes * (256 / Fmt<T>::values);
  uint32_t lane;
  __device__ __forceinline__ explicit LanePlan(uint32_t l) : lane(l) {}
  __device__ __forceinline__ void values(uint32_t, const uint8_t* row_ptr, uint32_t it, float* v, const Grids& g) const {
    const uint32_t c = lane + 32u * it;
    decode8<T>(row_ptr + (c / Fmt<T>::chunks) * Fmt<T>::bytes, (int) (c % Fmt<T>::chunks), v, g);
  }
};
template <> struct LanePlan<QTYPE_Q4_0> {
  static constexpr uint32_t kStretch = 144;
  uint32_t al, sh, doff, s4;
  __device__ __forceinline__ explicit LanePlan(uint32_t l) {
    const uint32_t b = l >> 2, k = l & 3u, a0 = b * 18u + 2u + 8u * (k & 1u);
    al = a0 & ~3u, sh = (a0 & 2u) * 8u, doff = b * 18u, s4 = 4u * (k >> 1);
  }
  __device__ __forceinline__ void values(uint32_t row, const uint8_t*, uint32_t it, float* v, const Grids&) const {
    const uint32_t base = row + it * kStretch;
    const uint32_t r0 = lds32(base + al), r1 = lds32(base + al + 4), r2 = lds32(base + al + 8);
    const float d = half_value(lds16(base + doff)), neg = mul_rn(d, -32776.0f);
    scaled4((__funnelshift_r(r0, r1, sh) >> s4) & 0x0F0F0F0Fu, d, neg, v);
    scaled4((__funnelshift_r(r1, r2, sh) >> s4) & 0x0F0F0F0Fu, d, neg, v + 4);
  }
  // the same chunk undecoded: its eight codes as bytes of m[0], m[1]; value j is fmaf(d, 32768 + byte j, neg)
  __device__ __forceinline__ void codes(uint32_t row, uint32_t it, uint32_t* m, float& d, float& neg) const {
    const uint32_t base = row + it * kStretch;
    const uint32_t r0 = lds32(base + al), r1 = lds32(base + al + 4), r2 = lds32(base + al + 8);
    d = half_value(lds16(base + doff)), neg = mul_rn(d, -32776.0f);
    m[0] = (__funnelshift_r(r0, r1, sh) >> s4) & 0x0F0F0F0Fu, m[1] = (__funnelshift_r(r1, r2, sh) >> s4) & 0x0F0F0F0Fu;
  }
};
template <> struct LanePlan<QTYPE_Q8_0> {
  static constexpr uint32_t kStretch = 272;
  uint32_t al, sh, doff;
  __device__ __forceinline__ explicit LanePlan(uint32_t l) {
    const uint32_t b = l >> 2, k = l & 3u, a0 = b * 34u + 2u + 8u * k;
    al = a0 & ~3u, sh = (a0 & 2u) * 8u, doff = b * 34u;
  }
  __device__ __forceinline__ void values(uint32_t row, const uint8_t*, uint32_t it, float* v, const Grids&) const {
    const uint32_t base = row + it * kStretch;
    const uint32_t r0 = lds32(base + al), r1 = lds32(base + al + 4), r2 = lds32(base + al + 8);
    const float d = half_value(lds16(base + doff)), neg = mul_rn(d, -32896.0f);
    scaled4(__funnelshift_r(r0, r1, sh) ^ 0x80808080u, d, neg, v);
    scaled4(__funnelshift_r(r1, r2, sh) ^ 0x80808080u, d, neg, v + 4);
  }
  __device__ __forceinline__ void codes(uint32_t row, uint32_t it, uint32_t* m, float& d, float& neg) const {
    const uint32_t base = row + it * kStretch;
    const uint32_t r0 = lds32(base + al), r1 = lds32(base + al + 4), r2 = lds32(base + al + 8);
    d = half_value(lds16(base + doff)), neg = mul_rn(d, -32896.0f);
    m[0] = __funnelshift_r(r0, r1, sh) ^ 0x80808080u, m[1] = __funnelshift_r(r1, r2, sh) ^ 0x80808080u;
  }
};

template <> struct LanePlan<QTYPE_Q4_K> {
  // lane l's chunk of a 144-byte block: group l / 4 (its 6-bit scale and min among the 12 packed bytes), values
  // 8 (l % 4) .. of the group - the low (even group) or high nibbles of 8 bytes; everything but the bytes themselves
  // is worked out once. A row starts on 16 bytes and a block is 144 long, so every read is aligned.
  static constexpr uint32_t kStretch = 144;
  uint32_t qoff, s4, b8, upper;
  __device__ __forceinline__ explicit LanePlan(uint32_t l) {
    const uint32_t grp = l >> 2;
    qoff = 16u + (grp >> 1) * 32u + (l & 3u) * 8u, s4 = 4u * (grp & 1u), b8 = 8u * (grp & 3u), upper = grp >> 2;
  }
  __device__ __forceinline__ void values(uint32_t row, const uint8_t*, uint32_t it, float* v, const Grids&) const {
    const uint32_t base = row + it * kStretch;
    const uint32_t hd = lds32(base);
    const uint32_t a0 = (lds32(base + 4) >> b8) & 0xFFu, a1 = (lds32(base + 8) >> b8) & 0xFFu, a2 = (lds32(base + 12) >> b8) & 0xFFu;
    const uint32_t sc = upper ? (a2 & 0x0Fu) | ((a0 >> 6) << 4) : a0 & 63u;
    const uint32_t mn = upper ? (a2 >> 4) | ((a1 >> 6) << 4) : a1 & 63u;
    // d sc has at most 17 significant bits and a code 4: the product is exact, so one fmaf against the biased code
    // gives the bits of mul_rn(d sc, n); then the min is taken off, rounded once - decode8's value
    const float ds = mul_rn(half_value(hd & 0xFFFFu), (float) sc), dm = mul_rn(half_value(hd >> 16), (float) mn);
    const float c = mul_rn(ds, -32768.0f);
    const uint2 q = lds64(base + qoff);
    const uint32_t m0 = (q.x >> s4) & 0x0F0F0F0Fu, m1 = (q.y >> s4) & 0x0F0F0F0Fu;
    v[0] = __fsub_rn(__fmaf_rn(ds, biased<0>(m0), c), dm), v[1] = __fsub_rn(__fmaf_rn(ds, biased<1>(m0), c), dm);
    v[2] = __fsub_rn(__fmaf_rn(ds, biased<2>(m0), c), dm), v[3] = __fsub_rn(__fmaf_rn(ds, biased<3>(m0), c), dm);
    v[4] = __fsub_rn(__fmaf_rn(ds, biased<0>(m1), c), dm), v[5] = __fsub_rn(__fmaf_rn(ds, biased<1>(m1), c), dm);
    v[6] = __fsub_rn(__fmaf_rn(ds, biased<2>(m1), c), dm), v[7] = __fsub_rn(__fmaf_rn(ds, biased<3>(m1), c), dm);
  }
};

template <> struct LanePlan<QTYPE_MXFP4> {
  // lane l's chunk of a 136-byte stretch: block l / 4 (17 bytes: the scale's exponent, then 16 bytes of codes), its
  // bytes 8 (l % 2) .., the low (l % 4 < 2) or high nibbles. The codes' values (doubled) come from a 16-entry F32 table
  // in shared memory (`tbl`, set by the kernel): sixteen different banks, where the constant bank would serve a warp's
  // different codes one after another.
  static constexpr uint32_t kStretch = 136;
  uint32_t al, sh, eoff, s4, tbl;
  __device__ __forceinline__ explicit LanePlan(uint32_t l) : tbl(0) {
    const uint32_t b = l >> 2, k = l & 3u, a0 = b * 17u + 1u + 8u * (k & 1u);
    al = a0 & ~3u, sh = (a0 & 3u) * 8u, eoff = b * 17u, s4 = 4u * (k >> 1);
  }
  __device__ __forceinline__ void values(uint32_t row, const uint8_t*, uint32_t it, float* v, const Grids&) const {
    const uint32_t base = row + it * kStretch;
    const uint32_t r0 = lds32(base + al), r1 = lds32(base + al + 4), r2 = lds32(base + al + 8);
    const uint32_t e = lds8(base + eoff);
    const float dd = __uint_as_float(e >= 2 ? (e - 1) << 23 : 0x00200000u << e);
    // a code's table offset (4 code) in each byte
    const uint32_t w[2] = {((__funnelshift_r(r0, r1, sh) >> s4) & 0x0F0F0F0Fu) << 2, ((__funnelshift_r(r1, r2, sh) >> s4) & 0x0F0F0F0Fu) << 2};
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = mul_rn(dd, ldsf(tbl + ((w[j >> 2] >> (8 * (j & 3))) & 0xFFu)));
  }
};

template <uint32_t T, int NT, int RW, bool GROUP>
__global__ void __launch_bounds__(kThreads, 1) mv_staged_kernel(const Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(16) uint8_t tables[grid_smem_bytes<T>() > 0 ? grid_smem_bytes<T>() : 16];
  __shared__ float e2m1_values[16];  // MXFP4: a code's value, doubled
  if constexpr (T == QTYPE_MXFP4) {
    if (threadIdx.x < 16) e2m1_values[threadIdx.x] = (float) osmos_e2m1_doubled[threadIdx.x];
  }
  __shared__ __align__(8) uint64_t full[kWarps][kMaxSlots];
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t row_bytes = a.cols / Fmt<T>::values * Fmt<T>::bytes;
  const uint32_t S = a.slots;
  uint8_t* ring = smem + a.ring_off + warp * S * a.slot_bytes;
  const uint8_t* mat = a.w;
  const float* xin = a.x;
  float* yout = a.y;
  uint32_t n_tok = a.n_tok;
  if constexpr (GROUP) {
    pdl_wait();  // (a dependent launch: the tables and x may be the output of the kernel ahead)
    pdl_launch_next();
    if (!entry_of_block<NT>(a, mat, xin, yout, n_tok)) return;  // (the whole block)
  }

  // this block's units (RW rows each), dealt to its warps round-robin
  const uint32_t u_lo = (uint32_t) ((uint64_t) blockIdx.x * a.units / gridDim.x);
  const uint32_t u_hi = (uint32_t) ((uint64_t) (blockIdx.x + 1) * a.units / gridDim.x);
  auto issue = [&](uint32_t i) {  // one lane: the warp's i-th unit into slot i % S
    const uint32_t u = u_lo + warp + i * kWarps;
    if (u >= u_hi) return;
    const uint32_t r0 = u * RW, nrows = a.rows - r0 < (uint32_t) RW ? a.rows - r0 : (uint32_t) RW;
    const uint32_t slot = i % S, bytes = nrows * row_bytes;
    bar_expect(&full[warp][slot], bytes);
    bulk_load(ring + slot * a.slot_bytes, mat + (uint64_t) r0 * row_bytes, bytes, &full[warp][slot]);
  };
  if (lane == 0) {
    for (uint32_t s = 0; s < S; s++) bar_init(&full[warp][s], 1);
    bar_init_fence();
    for (uint32_t i = 0; i < S; i++) issue(i);
  }

  if constexpr (!GROUP) {
    pdl_wait();  // (a dependent launch: x may be the output of the kernel ahead; the weight copies above are not)
    pdl_launch_next();
  }
  // the tokens' x (the live ones) and the codebooks, while the first copies fly
  const uint32_t live = n_tok < (uint32_t) NT ? n_tok : (uint32_t) NT;
  {
    const uint32_t per = a.cols / 4;
    // a token's chunks as two planes - every chunk's first four values, then every chunk's last four - so that a
    // warp's 16-byte reads of one plane are contiguous (chunk after chunk 32 bytes apart, they would pair up on banks)
    for (uint32_t i = tid; i < live * per; i += kThreads) {
      const uint32_t t = i / per, j = i - t * per;
      ((float4*) smem)[t * per + (j & 1u) * (per / 2) + (j >> 1)] = __ldg((const float4*) (xin + (uint64_t) t * a.xs) + j);
    }
  }
  const Grids g = stage_grids<T>(tables);
  __syncthreads();

  uint32_t xa[NT];  // a token slot past the live ones repeats the last live token: summed, never stored
#pragma unroll
  for (int t = 0; t < NT; t++) xa[t] = smem_addr(smem) + ((uint32_t) t < live ? (uint32_t) t : live - 1) * a.cols * 4u;
  const uint32_t ni = a.cols / 256;
  LanePlan<T> plan(lane);
  if constexpr (T == QTYPE_MXFP4) plan.tbl = smem_addr(e2m1_values);

  for (uint32_t i = 0;; i++) {
    const uint32_t u = u_lo + warp + i * kWarps;
    if (u >= u_hi) break;
    const uint32_t slot = i % S;
    if (!bar_wait(&full[warp][slot], (i / S) & 1u)) {  // a copy never landed: report it and leave
      if (lane == 0) atomicOr(a.status, 1u);
      break;
    }
    const uint8_t* sp = ring + slot * a.slot_bytes;
    const uint32_t sa = smem_addr(sp);
    float acc[RW][NT];
#pragma unroll
    for (int q = 0; q < RW; q++)
#pragma unroll
      for (int t = 0; t < NT; t++) acc[q][t] = 0.0f;
    for (uint32_t it = 0; it < ni; it++) {
      float v[RW][kChunk];
#pragma unroll
      for (int q = 0; q < RW; q++) plan.values(sa + q * row_bytes, sp + q * row_bytes, it, v[q], g);
#pragma unroll
      for (int t = 0; t < NT; t++) {
        const uint32_t xc = xa[t] + (lane + 32u * it) * 16u;
        const float4 lo = lds128f(xc), hi = lds128f(xc + a.cols * 2u);
#pragma unroll
        for (int q = 0; q < RW; q++) {
          float s = acc[q][t];
          s = __fmaf_rn(v[q][0], lo.x, s), s = __fmaf_rn(v[q][1], lo.y, s);
          s = __fmaf_rn(v[q][2], lo.z, s), s = __fmaf_rn(v[q][3], lo.w, s);
          s = __fmaf_rn(v[q][4], hi.x, s), s = __fmaf_rn(v[q][5], hi.y, s);
          s = __fmaf_rn(v[q][6], hi.z, s), s = __fmaf_rn(v[q][7], hi.w, s);
          acc[q][t] = s;
        }
      }
    }
    // every lane is done reading the slot: refill it
    __syncwarp();
    if (lane == 0) {
      fence_async_smem();
      issue(i + S);
    }
    const uint32_t r0 = u * RW;
#pragma unroll
    for (int q = 0; q < RW; q++)
#pragma unroll
      for (int t = 0; t < NT; t++) {
        const float s = xor_tree<kWarp>(acc[q][t]);
        if (lane == 0 && r0 + q < a.rows && (uint32_t) t < live) yout[(uint64_t) t * a.ys + r0 + q] = s;
      }
  }
}

constexpr int kRegIters = 8;  // 256-value stretches of a row whose x a lane can keep in registers (cols <= 2048)

template <uint32_t T, int RW, bool GROUP>
__global__ void __launch_bounds__(kThreads, 1) mv_regx_kernel(const Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(16) uint8_t tables[grid_smem_bytes<T>() > 0 ? grid_smem_bytes<T>() : 16];
  __shared__ float e2m1_values[16];  // MXFP4: a code's value, doubled
  if constexpr (T == QTYPE_MXFP4) {
    if (threadIdx.x < 16) e2m1_values[threadIdx.x] = (float) osmos_e2m1_doubled[threadIdx.x];
  }
  __shared__ __align__(8) uint64_t full[kWarps][kMaxSlots];
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t row_bytes = a.cols / Fmt<T>::values * Fmt<T>::bytes;
  const uint32_t S = a.slots, ni = a.cols / 256;
  uint8_t* ring = smem + warp * S * a.slot_bytes;
  const uint8_t* mat = a.w;
  const float* xin = a.x;
  float* yout = a.y;
  if constexpr (GROUP) {
    pdl_wait();  // (a dependent launch: the tables and x may be the output of the kernel ahead)
    pdl_launch_next();
    uint32_t n_tok;
    if (!entry_of_block<1>(a, mat, xin, yout, n_tok)) return;  // (the whole block)
  }

  const uint32_t u_lo = (uint32_t) ((uint64_t) blockIdx.x * a.units / gridDim.x);
  const uint32_t u_hi = (uint32_t) ((uint64_t) (blockIdx.x + 1) * a.units / gridDim.x);
  auto issue = [&](uint32_t i) {  // one lane: the warp's i-th unit into slot i % S
    const uint32_t u = u_lo + warp + i * kWarps;
    if (u >= u_hi) return;
    const uint32_t r0 = u * RW, nrows = a.rows - r0 < (uint32_t) RW ? a.rows - r0 : (uint32_t) RW;
    const uint32_t slot = i % S, bytes = nrows * row_bytes;
    bar_expect(&full[warp][slot], bytes);
    bulk_load(ring + slot * a.slot_bytes, mat + (uint64_t) r0 * row_bytes, bytes, &full[warp][slot]);
  };
  if (lane == 0) {
    for (uint32_t s = 0; s < S; s++) bar_init(&full[warp][s], 1);
    bar_init_fence();
    for (uint32_t i = 0; i < S; i++) issue(i);
  }
  if constexpr (!GROUP) {
    pdl_wait();  // (a dependent launch: x may be the output of the kernel ahead; the weight copies above are not)
    pdl_launch_next();
  }
  // the lane's x: chunk lane + 32 it of every stretch
  float xr[kRegIters][kChunk];
#pragma unroll
  for (int it = 0; it < kRegIters; it++) {
    float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
    if ((uint32_t) it < ni) {
      const float4* xp = (const float4*) (xin + (lane + 32u * it) * kChunk);
      lo = __ldg(xp), hi = __ldg(xp + 1);
    }
    xr[it][0] = lo.x, xr[it][1] = lo.y, xr[it][2] = lo.z, xr[it][3] = lo.w;
    xr[it][4] = hi.x, xr[it][5] = hi.y, xr[it][6] = hi.z, xr[it][7] = hi.w;
  }
  const Grids g = stage_grids<T>(tables);
  __syncthreads();  // the barriers' initialisation, seen by every lane that will wait on them
  LanePlan<T> plan(lane);
  if constexpr (T == QTYPE_MXFP4) plan.tbl = smem_addr(e2m1_values);

  for (uint32_t i = 0;; i++) {
    const uint32_t u = u_lo + warp + i * kWarps;
    if (u >= u_hi) break;
    const uint32_t slot = i % S;
    if (!bar_wait(&full[warp][slot], (i / S) & 1u)) {  // a copy never landed: report it and leave
      if (lane == 0) atomicOr(a.status, 1u);
      break;
    }
    const uint8_t* sp = ring + slot * a.slot_bytes;
    const uint32_t sa = smem_addr(sp);
    float acc[RW];
#pragma unroll
    for (int q = 0; q < RW; q++) acc[q] = 0.0f;
    if constexpr (kPlainPair<T> && RW == 2) {
      // the two rows' chains side by side in the packed F32 instructions: every element the same fmaf as below
      uint64_t acc2 = pack2(0.0f, 0.0f);
#pragma unroll
      for (int it = 0; it < kRegIters; it++) {
        if ((uint32_t) it < ni) {
          uint32_t m0[2], m1[2];
          float d0, n0, d1, n1;
          plan.codes(sa, (uint32_t) it, m0, d0, n0);
          plan.codes(sa + row_bytes, (uint32_t) it, m1, d1, n1);
          const uint64_t dd = pack2(d0, d1), nn = pack2(n0, n1);
#pragma unroll
          for (int j = 0; j < kChunk; j++) {
            const uint32_t sel = 0x7404u | ((uint32_t) (j & 3) << 4);
            const uint64_t b = pack2(__uint_as_float(__byte_perm(m0[j >> 2], 0x47000000u, sel)),
                                     __uint_as_float(__byte_perm(m1[j >> 2], 0x47000000u, sel)));
            acc2 = fma2(fma2(dd, b, nn), pack2(xr[it][j], xr[it][j]), acc2);
          }
        }
      }
      unpack2(acc2, acc[0], acc[1]);
    } else {
#pragma unroll
      for (int it = 0; it < kRegIters; it++) {
        if ((uint32_t) it < ni) {
#pragma unroll
          for (int q = 0; q < RW; q++) {
            float v[kChunk];
            plan.values(sa + q * row_bytes, sp + q * row_bytes, (uint32_t) it, v, g);
            float s = acc[q];
#pragma unroll
            for (int j = 0; j < kChunk; j++) s = __fmaf_rn(v[j], xr[it][j], s);
            acc[q] = s;
          }
        }
      }
    }
    __syncwarp();  // every lane is done reading the slot: refill it
    if (lane == 0) {
      fence_async_smem();
      issue(i + S);
    }
    const uint32_t r0 = u * RW;
#pragma unroll
    for (int q = 0; q < RW; q++) {
      const float s = xor_tree<kWarp>(acc[q]);
      if (lane == 0 && r0 + q < a.rows) yout[r0 + q] = s;
    }
  }
}

struct Device {
  int sms = 0;
  uint32_t* status = nullptr;
};

const Device* device_info() {
  static Device devs[64];
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
  if (!devs[d].status) {
    void* at = nullptr;
    int sms = 0;
    if (cudaGetSymbolAddress(&at, g_status) != cudaSuccess || !at) return nullptr;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || sms <= 0) return nullptr;
    devs[d].sms = sms, devs[d].status = (uint32_t*) at;
  }
  return &devs[d];
}

template <uint32_t T, int NT, int RW, bool REGX, bool GROUP>
int launch(const Request& r, const Device* dev, uint32_t slots, uint32_t cnt_lo, cudaStream_t s, uint32_t cnt_hi = (uint32_t) NT) {
  const uint32_t row_bytes = r.cols / Fmt<T>::values * Fmt<T>::bytes;
  Args a{};
  a.w = (const uint8_t*) r.w, a.x = r.x, a.y = r.y, a.rows = r.rows, a.cols = r.cols, a.xs = r.xs, a.ys = r.ys;
  a.n_tok = GROUP ? (uint32_t) NT : r.n_tok, a.slots = slots, a.slot_bytes = RW * row_bytes;
  a.ring_off = REGX ? 0u : (a.n_tok * r.cols * 4u + 127u) & ~127u;
  a.units = (r.rows + RW - 1) / RW;
  a.status = dev->status;
  a.wt = (const uint8_t* const*) r.wt, a.cnt = r.cnt, a.xrow = r.xrow, a.x_mat = r.x_mat, a.x_div = r.x_div, a.cnt_lo = cnt_lo, a.cnt_hi = cnt_hi;
  const uint32_t total = a.ring_off + kWarps * slots * a.slot_bytes + 16u;  // + the window's read past a last block
  static bool sized[64] = {};  // (one record a template instance, one flag a device)
  void (*kernel)(const Args);
  if constexpr (REGX) kernel = mv_regx_kernel<T, RW, GROUP>;
  else kernel = mv_staged_kernel<T, NT, RW, GROUP>;
  if (!allow_dynamic_smem(kernel, (int) kSmemLimit<T>, sized)) return 0;
  dim3 grid((uint32_t) dev->sms);
  if (a.units < grid.x) grid.x = a.units;
  if constexpr (GROUP) {  // an entry's rows over a few blocks: about four units a warp each, at most eight blocks
    const uint32_t per = a.units / (4u * kWarps);
    grid.x = per < 1u ? 1u : per > 8u ? 8u : per, grid.y = r.n_entries;
  }
  return launch_dependent(kernel, grid, dim3(kThreads), total, s, a) == cudaSuccess ? 1 : -1;
}

// as deep a ring as fits beside n_tok tokens' x (0 tokens: x in registers)
template <uint32_t T>
uint32_t slots_for(uint32_t rw, uint32_t x_tokens, uint32_t cols) {
  const uint32_t row_bytes = cols / Fmt<T>::values * Fmt<T>::bytes, budget = kSmemLimit<T> - 16u;
  const uint32_t x_bytes = (x_tokens * cols * 4u + 127u) & ~127u;
  if (x_bytes >= budget) return 0;
  const uint32_t n = (budget - x_bytes) / (kWarps * rw * row_bytes);
  return n > (uint32_t) kMaxSlots ? (uint32_t) kMaxSlots : n;
}

template <uint32_t T>
int by_shape(const Request& r, cudaStream_t s) {
  const Device* dev = device_info();
  if (!dev) return 0;
  const uint32_t row_bytes = r.cols / Fmt<T>::values * Fmt<T>::bytes;
  if (r.cols % 256 || row_bytes % 16u) return 0;  // whole 256-value stretches; a row's bytes are a bulk copy's
  if (r.n_tok > 8) return 0;
  const bool regx = r.n_tok == 1 && r.cols <= 256u * kRegIters;
  // two rows a unit (the decode of one overlaps the other's chain; with x in shared memory they share its loads)
  // when the matrix has rows to spare and the ring still has three slots
  const uint32_t xt = regx ? 0u : r.n_tok;
  const bool pair = (uint64_t) r.rows >= 8ull * kWarps * dev->sms && slots_for<T>(2, xt, r.cols) >= 3;
  const uint32_t slots = slots_for<T>(pair ? 2 : 1, xt, r.cols);
  if (slots < 2) return 0;
  if (regx) return pair ? launch<T, 1, 2, true, false>(r, dev, slots, 0, s) : launch<T, 1, 1, true, false>(r, dev, slots, 0, s);
  if (r.n_tok <= 1) return pair ? launch<T, 1, 2, false, false>(r, dev, slots, 0, s) : launch<T, 1, 1, false, false>(r, dev, slots, 0, s);
  if (r.n_tok <= 2) return pair ? launch<T, 2, 2, false, false>(r, dev, slots, 0, s) : launch<T, 2, 1, false, false>(r, dev, slots, 0, s);
  // 3 .. 8 tokens: a chunk is decoded once and meets every token's values (four or eight chains a row)
  if (r.n_tok <= 4) return pair ? launch<T, 4, 2, false, false>(r, dev, slots, 0, s) : launch<T, 4, 1, false, false>(r, dev, slots, 0, s);
  return pair ? launch<T, 8, 2, false, false>(r, dev, slots, 0, s) : launch<T, 8, 1, false, false>(r, dev, slots, 0, s);
}

// The grouped forms: a block an (entry, part of its rows). By token, the entries are served in classes of their token
// count - 1, 2, 3 .. 4, 5 .. 8 - a launch a class up to the call's max_cnt, each over all entries: a block whose entry
// belongs to another class leaves at once, so an entry of one token never pays for eight chains.
template <uint32_t T>
int grouped(const Request& r, cudaStream_t s) {
  const Device* dev = device_info();
  if (!dev) return 0;
  const uint32_t row_bytes = r.cols / Fmt<T>::values * Fmt<T>::bytes;
  if (r.cols % 256 || row_bytes % 16u || !r.n_entries || r.n_entries > 65535u) return 0;
  const uint32_t most = r.cnt ? r.n_tok : 1u;
  // every class this call needs must fit, or none is taken (the generic kernel then serves the whole call)
  const bool regx = r.cols <= 256u * kRegIters;
  const uint32_t top = most <= 1 ? 1u : most <= 2 ? 2u : most <= 4 ? 4u : 8u;
  if (slots_for<T>(1, top == 1 && regx ? 0u : top, r.cols) < 2) return 0;
  // (the last class also takes the entries whose count is past the call's max_cnt: their first max_cnt tokens)
  constexpr uint32_t kAny = 0x7FFFFFFFu;
  int st = regx ? launch<T, 1, 1, true, true>(r, dev, slots_for<T>(1, 0, r.cols), 1, s, top == 1 ? kAny : 1u)
                : launch<T, 1, 1, false, true>(r, dev, slots_for<T>(1, 1, r.cols), 1, s, top == 1 ? kAny : 1u);
  if (st > 0 && top >= 2) st = launch<T, 2, 1, false, true>(r, dev, slots_for<T>(1, 2, r.cols), 2, s, top == 2 ? kAny : 2u);
  if (st > 0 && top >= 4) st = launch<T, 4, 1, false, true>(r, dev, slots_for<T>(1, 4, r.cols), 3, s, top == 4 ? kAny : 4u);
  if (st > 0 && top >= 8) st = launch<T, 8, 1, false, true>(r, dev, slots_for<T>(1, 8, r.cols), 5, s, kAny);
  return st;
}

}  // namespace

int try_launch(uint32_t type, const Request& r, void* stream) {
  if (!r.rows || !r.n_tok || r.n_tok > 8 || r.cols % 8) return 0;
  if (r.wt) {  // grouped: every entry's x row starts on 16 bytes when the first does and the strides are whole words of 16
    if (((uintptr_t) r.x & 15u) || r.xs % 4 || r.x_mat % 4) return 0;
#define CASE(T) return grouped<T>(r, (cudaStream_t) stream);
    OSMOS_SWITCH_QUANT(type, CASE, return 0)
#undef CASE
  }
  if (((uintptr_t) r.w | (uintptr_t) r.x) & 15u) return 0;
  if (r.n_tok > 1 && r.xs % 4) return 0;
#define CASE(T) return by_shape<T>(r, (cudaStream_t) stream);
  OSMOS_SWITCH_QUANT(type, CASE, return 0)
#undef CASE
}

uint32_t max_tokens(uint32_t type, uint32_t cols) {
  if (!cols || cols % 256) return 0;
#define CASE(T)                                                                          \
  {                                                                                      \
    if ((cols / Fmt<T>::values * Fmt<T>::bytes) % 16u) return 0;                          \
    uint32_t n = 8;                                                                      \
    while (n && slots_for<T>(1, n, cols) < 2) n--;                                       \
    return n;                                                                            \
  }
  OSMOS_SWITCH_QUANT(type, CASE, return 0)
#undef CASE
}

uint32_t read_status() {
  const Device* dev = device_info();
  if (!dev) return 0x80000000u;
  uint32_t v = 0, zero = 0;
  if (cudaMemcpy(&v, dev->status, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return 0x80000000u;
  cudaMemcpy(dev->status, &zero, sizeof zero, cudaMemcpyHostToDevice);
  return v;
}

}  // namespace mvs
}  // namespace osmos
