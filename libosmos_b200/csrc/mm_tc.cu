// The prefill matrix products over f16 activations (include/osmos_b200/mm.h: mm_run, mm_run2, mm_group, mm_tokens)
// on the 5th-generation tensor cores: tcgen05.mma kind::f16, F32 accumulators in tensor memory.
//
// The weights' exact values are rounded to f16 (nearest) as they are decoded, the activations are the caller's x16
// (mm_x16's tiled f16), and every product is accumulated in F32 along K in one pass - the reference's arithmetic
// (kernels/mm.h: f16 operands, F32 accumulation) with the tensor core's own order of additions instead of its waves'
// partitions; a token's column is computed from that column alone, so its bits do not depend on the tokens beside
// it or on where in the batch it stands.
//
// A block computes 128 weight rows x 128, 256 or 512 tokens of one matrix (the most that still leaves every SM a
// block), a weight decoded once a block.
// Twenty-five warps, four roles:
//   loader (4 warps)     cp.async of the tokens' 16-byte pieces of x16 into the B operand's layout, its arrivals on the
//                        stage's second "full" mbarrier made by the hardware when the copies land
//   producers (16 warps, two teams of 8 on alternate steps) per 64-value step of K: decode the rows' 8-value chunks to f16 and store them as the A
//                        operand (four K = 16 sub-tiles of 128 rows, K-major core matrices of 8 rows x 16 bytes), and
//                        cp.async the tokens' 16-byte pieces of x16 into the same layout (B, four sub-tiles a
//                        128-token accumulator); a proxy fence and an arrive on the stage's "full" mbarrier. Two stages; the rows'
//                        bytes reach the decoders through shared memory, 256 values of K at a time (128 of Q8_0).
//   issuer (1 warp)      per step and accumulator four tcgen05.mma M128 N128 K16 (the first of the whole K loop
//                        overwrites, the rest accumulate), then tcgen05.commit onto the stage's "empty" mbarrier; after
//                        the last step a commit onto "done".
//   epilogue (4 warps)   thread = one weight row (its TMEM lane): tcgen05.ld the sums, scale, store y[t][row] - or, for
//                        mm_run_silu, silu(scale sum) to y and as f16 into the next product's tiled activations; for
//                        mm_run_gated_mean the block's rows are hc streams' rows of the same dim values (row map
//                        below), each thread gates its sum, and the streams are added in order through shared memory
//                        (the operand ring, idle by then).
// Every mbarrier wait is bounded (%globaltimer); a wait that runs out raises the status word, every role falls through
// to the common exit and tensor memory is released.
#include <cuda.h>

#include <cstring>

#include "act.cuh"
#include "decode.cuh"
#include "dispatch.cuh"
#include "fp4_tc_api.h"
#include "mm_tc_api.h"
#include "osmos_b200/mm.h"
#include "tma.cuh"

namespace osmos {
namespace mm_tc {
namespace {

using namespace tma;

constexpr int kM = 128, kN = 128;  // rows a block; tokens an accumulator
constexpr int kMaxAcc = 4;         // accumulators a block: 512 tokens
constexpr int kEpiWarps = 4, kProdWarps = 16;
constexpr int kLoaderWarps = 4;
// Roles go by the warp scheduler a warp lives on (its index mod 4): scheduler 0 has the issuer - whose chain of tcgen05
// instructions a step is the critical path, and must not queue for issue slots behind the decoders - the four loaders
// and one producer; the other fifteen producers share schedulers 1 to 3 with the epilogue warps.
constexpr int kIssuerWarp = 4;
__host__ __device__ constexpr int loader_of(int warp) { return (warp >= 8 && warp <= 20 && warp % 4 == 0) ? (warp - 8) / 4 : -1; }
__host__ __device__ constexpr int producer_of(int warp) {
  return warp == 24 ? 15 : (warp >= 5 && warp <= 23 && warp % 4 != 0) ? ((warp - 5) / 4) * 3 + warp % 4 - 1 : -1;
}
static_assert(producer_of(5) == 0 && producer_of(7) == 2 && producer_of(9) == 3 && producer_of(23) == 14 && producer_of(24) == 15 &&
                  producer_of(8) == -1 && producer_of(4) == -1 && loader_of(8) == 0 && loader_of(20) == 3 && loader_of(24) == -1,
              "sixteen producers, four loaders");
constexpr int kProdThreads = kProdWarps * kWarp, kLoaderThreads = kLoaderWarps * kWarp;
// The producers work as kGroups teams, team g on the K steps g, g + kGroups, ...: a step's chain (raw bytes out of
// shared memory, decode, store, proxy fence, arrival) is latency, and two steps' chains run side by side.
// (A team comes back to a stage after at most as many steps as the ring is deep, so its parity waits never skip a phase.)
constexpr int kGroups = 2, kTeamThreads = kProdThreads / kGroups;
constexpr int kThreads = (kEpiWarps + 1 + kLoaderWarps + kProdWarps) * kWarp;
constexpr int kStep = 64;                        // values of K a stage
constexpr int kSubTile = kM * 32;                // one K = 16 operand sub-tile: 128 rows x 32 bytes
constexpr int kSubs = kStep / 16;                // sub-tiles a stage an operand: 4
constexpr int kStageA = kSubs * kSubTile;        // 16 KB
constexpr int kMaxStages = 4;

__device__ uint32_t g_status;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// shared-memory matrix descriptor of one sub-tile: K-major, no swizzle, core matrices of 8 rows x 16 bytes; the next
// 16 bytes of K are 128 bytes on (leading offset), the next 8 rows 256 bytes on (stride offset)
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr) {
  return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) (128u >> 4) << 16 | (uint64_t) (256u >> 4) << 32 | (uint64_t) 1 << 46;
}
// the same for a sub-tile a tensor-map copy wrote with the 32-byte swizzle: rows of 32 bytes (one MMA's K), the two
// 16-byte halves of a row exchanged in every second group of four rows; 8 rows are 256 bytes
__device__ __forceinline__ uint64_t tile_desc_sw32(uint32_t addr) {
  return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) 1 << 16 | (uint64_t) (256u >> 4) << 32 | (uint64_t) 1 << 46 | (uint64_t) 6 << 61;
}
// instruction descriptor: D F32, A and B f16, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t) (kN >> 3) << 17) | ((uint32_t) (kM >> 4) << 24);

// ---- the common types' chunks straight to f16 -----------------------------------------------------------------
// Eight values of a block whose bytes lie in shared memory at `blk` (4-byte aligned here), as eight f16 in a uint4:
// the same F32 value decode8 gives (each product rounded once), then rounded to f16. Small integers reach F32 by a
// byte permute (byte n into bits 8 .. 15 of 0x47000000 = 32768 + n), and a product d n as fmaf(d, 32768 + n,
// -32768 d): the subtrahend is a power of two times d, so the one rounding is the product's own.
template <int J> __device__ __forceinline__ float biased(uint32_t bytes) {
  return __uint_as_float(__byte_perm(bytes, 0x47000000u, 0x7404 | (J << 4)));
}
__device__ __forceinline__ uint32_t half2_bits(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *(const uint32_t*) &h;
}
// the rows' bytes come through shared memory this many values of K at a time (a whole number of blocks; fewer for the
// widest type, whose two raw buffers would otherwise cost the ring a stage), in slots of an odd number of 16-byte
// pieces a row
template <uint32_t T> constexpr uint32_t kRawK = (T == QTYPE_Q8_0) ? 128u : 256u;
template <uint32_t T> constexpr uint32_t kRawBytes = kRawK<T> / Fmt<T>::values * Fmt<T>::bytes;
template <uint32_t T> constexpr uint32_t kRawSlot = ((kRawBytes<T> + 30u + 15u) & ~15u) | 16u;
template <uint32_t T> constexpr bool kFastChunk = (T == QTYPE_Q4_K || T == QTYPE_Q4_0 || T == QTYPE_Q8_0);

template <uint32_t T>
__device__ __forceinline__ uint4 fast_chunk(const uint8_t* blk, uint32_t k) {
  uint4 out;
  if constexpr (T == QTYPE_Q4_K) {
    // chunk k of the 256-value block: group k / 4 (its 6-bit scale and min out of the 12 packed bytes), values
    // 8 (k % 4) .. of the group: the low (even group) or high nibbles of 8 bytes
    const uint32_t* wp = (const uint32_t*) blk;
    const uint32_t grp = k >> 2, b8 = 8u * (grp & 3u);
    const uint32_t hd = wp[0], a0 = (wp[1] >> b8) & 0xFFu, a1 = (wp[2] >> b8) & 0xFFu, a2 = (wp[3] >> b8) & 0xFFu;
    const uint32_t sc = grp < 4 ? a0 & 63u : (a2 & 0x0Fu) | ((a0 >> 6) << 4);
    const uint32_t mn = grp < 4 ? a1 & 63u : (a2 >> 4) | ((a1 >> 6) << 4);
    const float ds = mul_rn(half_value(hd & 0xFFFFu), (float) sc), dm = mul_rn(half_value(hd >> 16), (float) mn);
    const float c = mul_rn(ds, -32768.0f);
    const uint32_t* q = wp + 4 + (grp >> 1) * 8 + (k & 3u) * 2;
    const uint32_t s4 = 4u * (grp & 1u), m0 = (q[0] >> s4) & 0x0F0F0F0Fu, m1 = (q[1] >> s4) & 0x0F0F0F0Fu;
    out.x = half2_bits(__fsub_rn(__fmaf_rn(ds, biased<0>(m0), c), dm), __fsub_rn(__fmaf_rn(ds, biased<1>(m0), c), dm));
    out.y = half2_bits(__fsub_rn(__fmaf_rn(ds, biased<2>(m0), c), dm), __fsub_rn(__fmaf_rn(ds, biased<3>(m0), c), dm));
    out.z = half2_bits(__fsub_rn(__fmaf_rn(ds, biased<0>(m1), c), dm), __fsub_rn(__fmaf_rn(ds, biased<1>(m1), c), dm));
    out.w = half2_bits(__fsub_rn(__fmaf_rn(ds, biased<2>(m1), c), dm), __fsub_rn(__fmaf_rn(ds, biased<3>(m1), c), dm));
  } else {
    // a 32-value block with one f16 scale (2-byte aligned: read by halves): chunk k's 8 codes
    const uint16_t* hp = (const uint16_t*) blk;
    const float d = half_value(hp[0]);
    uint32_t m0, m1;
    float c;
    if constexpr (T == QTYPE_Q4_0) {  // d (n - 8): bytes 8 (k % 2) .., low (k < 2) or high nibbles
      const uint16_t* q = hp + 1 + 4 * (k & 1u);
      const uint32_t s4 = 4u * (k >> 1);
      m0 = (((uint32_t) q[0] | (uint32_t) q[1] << 16) >> s4) & 0x0F0F0F0Fu;
      m1 = (((uint32_t) q[2] | (uint32_t) q[3] << 16) >> s4) & 0x0F0F0F0Fu;
      c = mul_rn(d, -32776.0f);
    } else {  // Q8_0: d q, the signed byte as q + 128
      const uint16_t* q = hp + 1 + 4 * k;
      m0 = ((uint32_t) q[0] | (uint32_t) q[1] << 16) ^ 0x80808080u;
      m1 = ((uint32_t) q[2] | (uint32_t) q[3] << 16) ^ 0x80808080u;
      c = mul_rn(d, -32896.0f);
    }
    out.x = half2_bits(__fmaf_rn(d, biased<0>(m0), c), __fmaf_rn(d, biased<1>(m0), c));
    out.y = half2_bits(__fmaf_rn(d, biased<2>(m0), c), __fmaf_rn(d, biased<3>(m0), c));
    out.z = half2_bits(__fmaf_rn(d, biased<0>(m1), c), __fmaf_rn(d, biased<1>(m1), c));
    out.w = half2_bits(__fmaf_rn(d, biased<2>(m1), c), __fmaf_rn(d, biased<3>(m1), c));
  }
  return out;
}

struct Args {
  const uint8_t* w;          // one matrix (wt NULL)
  const uint8_t* const* wt;  // grouped: the matrices
  const int32_t* cnt;        // grouped: tokens a matrix
  const uint32_t *xoff, *yoff;  // grouped: where a matrix's tokens start in x16 (halves) and y (floats)
  const __half* x16;
  float* y;
  uint32_t rows, cols, n, xts, ys;
  uint32_t accs;  // accumulators (128 tokens each) a block: 1, 2 or 4
  uint32_t use_tma;  // the activations come by tensor-map copies (mm_run), else by 16-byte cp.async (mm_group)
  uint32_t stages, stage_bytes, raw_off;  // the operand ring's depth, a stage's bytes; where the raw weight buffers start
  float scale;
  uint32_t* status;
  // the epilogue (the kernel's EPI): kStore y = scale sum; kSilu y = silu(scale sum), and its f16 into x16_out (rows wide, tiled);
  // kGatedMean: the matrix is hc streams of dim rows, out[t][d] = (sum over s in order of xn[t][s][d]
  // sigmoid(sum_t[s dim + d])) / hc, and its f16 into x16_out (dim wide, token t at row out_row0 + t; NULL: none)
  __half* x16_out;
  int32_t* overflow;
  const float* xn;
  float* out;
  uint32_t hc, dim, per, out_row0;  // per: the dim values a block takes (hc per <= 128 rows of its tile are used)
};
enum : uint32_t { kStore = 0, kSilu = 1, kGatedMean = 2 };

struct Shared {
  uint64_t full_a[kMaxStages], full_b[kMaxStages], empty[kMaxStages], done;
  uint32_t tmem_base;
  int fail;
};

// EPI: the epilogue (kStore / kSilu / kGatedMean), a compile-time choice so that the plain product carries none of
// the others' code
template <uint32_t T, uint32_t EPI>
__global__ void __launch_bounds__(kThreads, 1) mm_tc_kernel(const Args a, const __grid_constant__ CUtensorMap tmap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ Shared sh;
  __shared__ __align__(16) uint8_t tables[grid_smem_bytes<T>() > 0 ? grid_smem_bytes<T>() : 16];
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t m = blockIdx.y, row0 = blockIdx.x * kM, span = a.accs * kN, c0 = blockIdx.z * span;
  const uint32_t n_tok = a.wt ? (uint32_t) (a.cnt[m] > 0 ? a.cnt[m] : 0) : a.n;
  if (c0 >= n_tok) return;  // the whole block, before anything is allocated
  const uint32_t n_valid = n_tok - c0 < span ? n_tok - c0 : span;
  const uint32_t n_valid16 = (n_valid + 15u) & ~15u;  // x16 holds whole tiles of 16 tokens
  const uint32_t n_acc = (n_valid + kN - 1) / kN;
  const uint32_t steps = a.cols / kStep;
  const uint64_t row_bytes = (uint64_t) (a.cols / Fmt<T>::values) * Fmt<T>::bytes;
  const uint8_t* w = a.wt ? a.wt[m] : a.w;
  // the weight row behind row r of the block's tile: the matrix's next 128 rows - or, for the gated mean, stream
  // r / per's row of value d0 + r % per, so the hc sums of one output value lie in one block (a row past the matrix,
  // or past the streams, repeats a valid one and is never stored)
  const uint32_t d0 = blockIdx.x * a.per;
  auto wrow = [&](uint32_t r) -> uint32_t {
    if constexpr (EPI != kGatedMean) return row0 + r < a.rows ? row0 + r : a.rows - 1;
    const uint32_t st = r / a.per, d = d0 + (r - st * a.per);
    return (st < a.hc ? st : a.hc - 1) * a.dim + (d < a.dim ? d : a.dim - 1);
  };
  const __half* x16 = a.x16 + (a.wt ? a.xoff[m] : 0u);
  float* y = a.y + (a.wt ? a.yoff[m] : 0u);

  if (tid == 0) {
    for (int i = 0; i < kMaxStages; i++) bar_init(&sh.full_a[i], kProdWarps / kGroups), bar_init(&sh.full_b[i], a.use_tma ? 1u : (uint32_t) kLoaderThreads), bar_init(&sh.empty[i], 1);
    bar_init(&sh.done, 1);
    sh.fail = 0;
    bar_init_fence();
  }
  if (warp == (uint32_t) kIssuerWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sh.tmem_base)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  const Grids g = stage_grids<T>(tables);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sh.tmem_base;
  const uint32_t S = a.stages;

  if (producer_of((int) warp) >= 0) {
    // ================= producers =================
    // The rows' bytes come through shared memory kRawK values of K at a time: 16-byte cp.async pieces of the aligned
    // span around each row's bytes (a block may start anywhere in a 16-byte piece), two buffers, the next block's values
    // on their way while these are decoded - so the decoders' many narrow reads are shared-memory reads.
    const uint32_t pt = (uint32_t) producer_of((int) warp) * kWarp + lane;
    constexpr uint32_t kKb = kRawK<T>, kKbBytes = kRawBytes<T>, kSlot = kRawSlot<T>;
    constexpr uint32_t kPieces = (kKbBytes + 30u + 15u) / 16u;  // (the slot may be one piece longer: an odd count)
    uint8_t* raw = smem + a.raw_off;
    const uint8_t* w_end = w + (uint64_t) a.rows * row_bytes;
    const uint32_t kblocks = (a.cols + kKb - 1) / kKb;
    auto fetch_raw = [&](uint32_t kb) {  // the rows' bytes of K block kb into buffer kb % 2
      uint8_t* buf = raw + (kb & 1u) * (kM * kSlot);
      for (uint32_t i = pt; i < (uint32_t) kM * kPieces; i += kProdThreads) {
        const uint32_t r = i / kPieces, piece = i - r * kPieces;
        const uint32_t row = wrow(r);
        const uint8_t* src = (const uint8_t*) ((uintptr_t) (w + row * row_bytes + (uint64_t) kb * kKbBytes) & ~(uintptr_t) 15) + piece * 16u;
        const uint32_t have = src >= w_end ? 0u : (w_end - src < 16 ? (uint32_t) (w_end - src) : 16u);  // (zero fill past the tensor)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(buf + r * kSlot + piece * 16u)), "l"(src), "r"(have)
                     : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // this thread's chunks of a step: chunk kc of rows 64 apart (eight neighbouring threads take one K piece of eight
    // neighbouring rows - eight different 16-byte bank columns of the operand tile, and of the raw buffer, whose row
    // slots are an odd number of 16-byte pieces); what does not change from step to step is worked out here
    constexpr int kMine = kM * (kStep / 8) / kTeamThreads;
    static_assert(kMine * kTeamThreads == kM * (kStep / 8) && kTeamThreads % 64 == 0, "every producer thread the same number of chunks");
    const uint32_t team = pt / kTeamThreads, tt = pt % kTeamThreads;  // the thread's team and its place in it
    const uint32_t kc = (tt >> 3) & 7u;
    uint32_t slot_at[kMine], dst_at[kMine], base15[kMine];
#pragma unroll
    for (int u = 0; u < kMine; u++) {
      const uint32_t task = tt + (uint32_t) u * kTeamThreads, r = (task >> 6) * 8u + (task & 7u);
      const uint32_t row = wrow(r);  // (a row past the matrix repeats the last one)
      slot_at[u] = r * kSlot, dst_at[u] = (kc >> 1) * kSubTile + (r >> 3) * 256 + (kc & 1u) * 128 + (r & 7u) * 16;
      base15[u] = (uint32_t) ((uintptr_t) (w + row * row_bytes) & 15u);
    }
    bool dead = false;  // a wait ran out: no more work, but the producers' own barrier is still kept
    fetch_raw(0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    static_assert((kKb / kStep) % kGroups == 0, "every team has steps in every K block");
    for (uint32_t it = team; it < steps; it += kGroups) {
      const uint32_t stage = it % S, use = it / S, kb = it / (kKb / kStep), sub = it % (kKb / kStep);
      const bool first = sub == team;  // the team's first step of K block kb
      if (first) {  // this thread's pieces of block kb have landed; after the barrier everyone's have, and block
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // kb - 1's buffer is free for kb + 1
        asm volatile("bar.sync 1, %0;" ::"n"(kProdThreads) : "memory");
      }
      if (!dead && use > 0 && !bar_wait(&sh.empty[stage], (use - 1) & 1u)) sh.fail = 1, dead = true;
      if (dead) continue;
      if (first && kb + 1 < kblocks) fetch_raw(kb + 1);
      // A: the chunk decoded to 8 halves, 16 bytes, to sub-tile kc / 2 of the stage
      uint8_t* sa = smem + stage * a.stage_bytes;
      const uint8_t* buf = raw + (kb & 1u) * (kM * kSlot);
      const uint32_t cl = sub * (kStep / kChunk) + kc;  // the chunk's index in its K block
      const uint32_t in_blk = (cl / Fmt<T>::chunks) * Fmt<T>::bytes, k_in = cl % Fmt<T>::chunks;
      const uint32_t kb15 = (kb * kKbBytes) & 15u;
#pragma unroll
      for (int u = 0; u < kMine; u++) {
        const uint8_t* blk = buf + slot_at[u] + ((base15[u] + kb15) & 15u) + in_blk;
        uint4 out;
        bool done = false;
        if constexpr (kFastChunk<T>) {
          if (T != QTYPE_Q4_K || ((uintptr_t) blk & 3u) == 0) out = fast_chunk<T>(blk, k_in), done = true;
        }
        if (!done) {
          float v[kChunk];
          decode8<T>(blk, (int) k_in, v, g);
          out.x = half2_bits(v[0], v[1]), out.y = half2_bits(v[2], v[3]);
          out.z = half2_bits(v[4], v[5]), out.w = half2_bits(v[6], v[7]);
        }
        *(uint4*) (sa + dst_at[u]) = out;
      }
      fence_async_smem();  // these writes before the tensor core's reads
      __syncwarp();
      if (lane == 0) bar_arrive(&sh.full_a[stage]);  // (one arrival a warp: 512 would queue on the one word)
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (loader_of((int) warp) >= 0) {
    // ================= the activations' loader =================
    // token n's 8-value piece kc of step `it`, 16 bytes, to sub-tile (n / 128, kc / 2) of the step's stage; the warp
    // never waits for its own copies: each thread's arrival on the stage's barrier is made by the hardware when that
    // thread's copies have landed, so the loads run as far ahead of the tensor core as the ring is deep
    const uint32_t lt = (uint32_t) loader_of((int) warp) * kWarp + lane;
    if (a.use_tma) {
      // One warp, a tensor-map copy a (128 tokens, 16 values of K) sub-tile: the tiled x16 seen as [token tile][K
      // fragment][token in tile][value in fragment], a box of 8 tiles x 1 fragment written with the 32-byte swizzle the
      // MMA reads (tiles past the last are filled with zeros); the stage's barrier counts the bytes.
      if (lt < (uint32_t) kWarp) {
        const uint32_t ops = n_acc * kSubs;
        for (uint32_t it = 0; it < steps; it++) {
          const uint32_t stage = it % S, use = it / S;
          if (use > 0 && !bar_wait(&sh.empty[stage], (use - 1) & 1u)) {
            sh.fail = 1;
            break;
          }
          if (lt == 0) bar_expect(&sh.full_b[stage], ops * kSubTile);
          __syncwarp();
          if (lt < ops) {
            const uint32_t acc = lt / kSubs, q = lt % kSubs;
            const uint32_t dst = smem_addr(smem + stage * a.stage_bytes + kStageA) + (acc * kSubs + q) * kSubTile;
            asm volatile(
                "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
                "l"(&tmap), "r"(0), "r"(0), "r"(it * kSubs + q), "r"(c0 / MM_TILE + acc * (kN / MM_TILE)), "r"(smem_addr(&sh.full_b[stage]))
                : "memory");
          }
        }
      }
    } else
    for (uint32_t it = 0; it < steps; it++) {
      const uint32_t stage = it % S, use = it / S;
      if (use > 0 && !bar_wait(&sh.empty[stage], (use - 1) & 1u)) {
        sh.fail = 1;
        break;
      }
      const uint32_t sb = smem_addr(smem + stage * a.stage_bytes + kStageA);
      const uint32_t pieces = n_valid16 * (kStep / 8);
      for (uint32_t i = lt; i < pieces; i += kLoaderThreads) {
        // (eight neighbouring threads: one K piece of eight neighbouring tokens - eight different 16-byte bank
        // columns of the operand tile, so a store takes no more passes than its bytes need)
        const uint32_t kc = (i >> 3) & 7u, n = (i >> 6) * 8u + (i & 7u), acc = n / kN, nn = n % kN;
        cp_async16(sb + (acc * kSubs + (kc >> 1)) * kSubTile + (nn >> 3) * 256 + (kc & 1u) * 128 + (nn & 7u) * 16,
                   x16 + mm_x16_at(c0 + n, it * kStep + kc * 8, a.xts));
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&sh.full_b[stage])) : "memory");
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == (uint32_t) kIssuerWarp) {
    // ================= issuer =================
    bool ok = true;
    for (uint32_t it = 0; it < steps && !sh.fail; it++) {
      const uint32_t stage = it % S, use = it / S;
      if (!bar_wait(&sh.full_a[stage], use & 1u) || !bar_wait(&sh.full_b[stage], use & 1u)) {
        sh.fail = 1, ok = false;
        break;
      }
      fence_async_smem();  // the loader's copies (seen through the barrier) before the tensor core's reads
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint32_t sa = smem_addr(smem + stage * a.stage_bytes), sb = sa + kStageA;
        for (uint32_t acc = 0; acc < n_acc; acc++)
          for (uint32_t q = 0; q < (uint32_t) kSubs; q++) {
            const uint64_t da = tile_desc(sa + q * kSubTile);
            const uint64_t db = a.use_tma ? tile_desc_sw32(sb + (acc * kSubs + q) * kSubTile) : tile_desc(sb + (acc * kSubs + q) * kSubTile);
            const uint32_t accumulate = (it | q) != 0 ? 1u : 0u;
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(
                    tmem + acc * kN),
                "l"(da), "l"(db), "r"(kIdesc), "r"(accumulate)
                : "memory");
          }
        // the stage's operands are free once these have run
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&sh.empty[stage]))
                     : "memory");
      }
      __syncwarp();
    }
    if (ok && !sh.fail && lane == 0)
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&sh.done)) : "memory");
    __syncwarp();
  }
  // ================= epilogue =================
  // Every warp, once its own role is done: a warp reads the tensor-memory lanes of its quarter (its index mod 4: the
  // hardware's rule), so the six or seven warps of a quarter share its rows' 32-token chunks - twenty-five warps
  // storing instead of four. (The gated mean's exchange through shared memory stays with the first four warps.)
  if (EPI != kGatedMean || warp < (uint32_t) kEpiWarps) {
    const uint32_t quarter = warp % 4u, part = EPI == kGatedMean ? 0u : warp / 4u;
    const uint32_t parts = EPI == kGatedMean ? 1u : ((uint32_t) (kThreads / kWarp) - quarter + 3u) / 4u;  // the quarter's warps
    const uint32_t row = 32u * quarter + lane;  // this thread's weight row of the tile = its TMEM lane
    const uint32_t lane_base = tmem + ((32u * quarter) << 16);
    if (!bar_wait(&sh.done, 0)) {
      // (the K loop's own waits are 0.2 s each and can queue up: look again while nobody has given up)
      bool landed = false;
      for (uint32_t tries = 0; tries < 25u && !sh.fail && !landed; tries++) landed = bar_wait(&sh.done, 0);
      if (!landed) sh.fail = 1;
    }
    // (nobody else writes the word once the last product has landed or been given up: after this barrier every
    // epilogue thread reads the same value, so all of them or none take the barriers below)
    if constexpr (EPI == kGatedMean) asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * kWarp) : "memory");
    if (!sh.fail) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (uint32_t acc = 0; acc < n_acc; acc++) {
#pragma unroll 1
        for (uint32_t c32 = 0; c32 < (uint32_t) kN; c32 += 32) {
          if (acc * kN + c32 >= n_valid) break;
          if ((acc * (uint32_t) (kN / 32) + c32 / 32u) % parts != part) continue;  // (a chunk of another warp of the quarter)
          uint32_t r[32];
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
              "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
              : "r"(lane_base + acc * kN + c32)
              : "memory");
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if constexpr (EPI == kGatedMean) {
            // each thread gates its row's sums into the idle operand ring ([token of the 32][tile row]); then thread e
            // adds value e % per's streams in order for the tokens e / per, e / per + 128 / per, ...
            float* ex = (float*) smem;
            const uint32_t st = row / a.per, d = d0 + (row - st * a.per);
            const bool mine = st < a.hc && d < a.dim;
#pragma unroll
            for (int i = 0; i < 32; i++) {
              const uint32_t t = acc * kN + c32 + i;
              float p = 0.0f;
              if (mine && t < n_valid)
                p = mul_rn(a.xn[((uint64_t) (c0 + t) * a.hc + st) * a.dim + d], sigmoidf(__uint_as_float(r[i])));
              ex[i * kM + row] = p;
            }
            asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * kWarp) : "memory");
            const uint32_t j = row % a.per, tg = row / a.per, groups = (uint32_t) kM / a.per;
            if (tg < groups && d0 + j < a.dim) {
              for (uint32_t i = tg; i < 32u; i += groups) {
                const uint32_t t = acc * kN + c32 + i;
                if (t >= n_valid) break;
                float sum = 0.0f;
                for (uint32_t q = 0; q < a.hc; q++) sum = __fadd_rn(sum, ex[i * kM + q * a.per + j]);
                const float v = __fdiv_rn(sum, (float) a.hc);
                a.out[(uint64_t) (c0 + t) * a.dim + d0 + j] = v;
                if (a.x16_out) x16_store(a.x16_out, a.overflow, a.out_row0 + c0 + t, d0 + j, a.dim, v);
              }
            }
            asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * kWarp) : "memory");  // (the next 32 tokens reuse ex)
          } else if (row0 + row < a.rows) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
              const uint32_t t = acc * kN + c32 + i;
              if (t < n_valid) {
                float v = __uint_as_float(r[i]);
                if (a.scale != 1.0f) v = mul_rn(v, a.scale);
                if constexpr (EPI == kSilu) {
                  v = siluf(v);
                  x16_store(a.x16_out, a.overflow, c0 + t, row0 + row, a.rows, v);
                }
                y[(uint64_t) (c0 + t) * a.ys + row0 + row] = v;
              }
            }
          }
        }
      }
    }
  }
  // ================= common exit =================
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == (uint32_t) kIssuerWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
  if (tid == 0 && sh.fail) atomicOr(a.status, 1u);
}

uint32_t* status_word() {
  static uint32_t* at[64];
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
  if (!at[d]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
    at[d] = (uint32_t*) p;
  }
  return at[d];
}

// the driver's tensor-map encoder, looked up once (no link against the driver library)
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled) p;
  }
  return fn;
}

// the tiled x16 of n tokens (rows xts values long) as [token tile][K fragment][token in tile][value in fragment]
bool x16_map(const void* x16, uint32_t n, uint32_t xts, CUtensorMap* tm) {
  const EncodeTiled enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[4] = {MM_TILE, MM_TILE, xts / MM_TILE, (n + MM_TILE - 1) / MM_TILE};
  const cuuint64_t strides[3] = {MM_TILE * 2, MM_TILE * MM_TILE * 2, (cuuint64_t) MM_TILE * xts * 2};
  const cuuint32_t box[4] = {MM_TILE, MM_TILE, 1, kN / MM_TILE}, unit[4] = {1, 1, 1, 1};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(x16), dims, strides, box, unit, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <uint32_t T, uint32_t EPI = kStore>
bool launch(Args a, uint32_t n_mat, uint32_t max_cnt, cudaStream_t s) {
  alignas(64) CUtensorMap tmap;
  memset(&tmap, 0, sizeof tmap);
  a.use_tma = 0;
  if (!a.wt && x16_map(a.x16, a.n, a.xts, &tmap)) a.use_tma = 1;
  a.status = status_word();
  if (!a.status) return false;
  int sms = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return false;
  constexpr uint32_t kSlot = kRawSlot<T>, kLimit = 224u * 1024u - (uint32_t) ((grid_smem_bytes<T>() + 1023) / 1024 * 1024);
  const uint32_t row_tiles = EPI == kGatedMean ? (a.dim + a.per - 1) / a.per : (a.rows + kM - 1) / kM;
  auto stages_for = [&](uint32_t k) { return k >= 4 ? 2u : k == 2 ? 3u : 4u; };  // a deeper ring where a stage is small
  auto smem_for = [&](uint32_t k) { return stages_for(k) * (kStageA + k * kSubs * kSubTile) + 2u * kM * kSlot; };
  // tokens a block: the accumulator count (1, 2 or 4 of 128 tokens; a weight is decoded once a block) with the least
  // estimated time - waves of blocks over the SMs times a block's time, which measured ~0.85 + 0.45 k a step with the
  // activations copied 16 bytes at a time and ~0.95 + 0.12 k with tensor-map copies
  a.accs = 1;
  float best = 0.0f;
  for (uint32_t k = 1; k <= (uint32_t) kMaxAcc; k <<= 1) {
    if (smem_for(k) > kLimit) break;
    const uint64_t blocks = (uint64_t) row_tiles * n_mat * ((max_cnt + k * kN - 1) / (k * kN));
    const float cost = (float) ((blocks + sms - 1) / sms) * (a.use_tma ? 0.95f + 0.12f * (float) k : 0.85f + 0.45f * (float) k);
    if (k == 1 || cost < best) best = cost, a.accs = k;
  }
  a.stages = stages_for(a.accs), a.stage_bytes = kStageA + a.accs * kSubs * kSubTile, a.raw_off = a.stages * a.stage_bytes;
  const int smem_bytes = (int) smem_for(a.accs);
  static bool sized[64] = {};  // (one record a template instance, one flag a device)
  if (!allow_dynamic_smem(mm_tc_kernel<T, EPI>, (int) kLimit, sized)) return false;
  const dim3 grid(row_tiles, n_mat, (max_cnt + a.accs * kN - 1) / (a.accs * kN));
  mm_tc_kernel<T, EPI><<<grid, kThreads, smem_bytes, s>>>(a, tmap);
  return launched();
}

}  // namespace

bool shape_ok(uint32_t type, uint32_t rows, uint32_t cols) {
  const OsmosQTypeInfo* t = qtype_row(type);
  return t && rows && rows % MM_TILE == 0 && cols && cols % 128 == 0 && cols % t->values == 0;
}

namespace {
template <uint32_t EPI>
bool run_with(uint32_t type, const Args& a, void* stream) {
#define CASE(T) return launch<T, EPI>(a, 1, a.n, stream_of(stream));
  OSMOS_SWITCH_QUANT(type, CASE, return false)
#undef CASE
}
}  // namespace

bool run(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const void* x16, uint32_t n, float* y, uint32_t ys,
         float scale, void* stream) {
  if (!w || !x16 || !y || !n || n > MM_MAX_TOKENS || !shape_ok(type, rows, cols) || (n > 1 && ys < rows)) return false;
  if ((uintptr_t) x16 & 15u) return false;
  Args a{};
  a.w = (const uint8_t*) w, a.x16 = (const __half*) x16, a.y = y, a.rows = rows, a.cols = cols, a.n = n, a.xts = cols;
  a.ys = ys, a.scale = scale;
  return run_with<kStore>(type, a, stream);
}

bool run_silu(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const void* x16, uint32_t n, float* y, uint32_t ys,
              float scale, void* x16_out, int32_t* overflow, void* stream) {
  if (!w || !x16 || !y || !x16_out || x16_out == x16 || !overflow || !n || n > MM_SILU_MAX_TOKENS ||
      !shape_ok(type, rows, cols) || (n > 1 && ys < rows) || (((uintptr_t) x16 | (uintptr_t) x16_out) & 15u))
    return false;
  Args a{};
  a.w = (const uint8_t*) w, a.x16 = (const __half*) x16, a.y = y, a.rows = rows, a.cols = cols, a.n = n, a.xts = cols;
  a.ys = ys, a.scale = scale, a.x16_out = (__half*) x16_out, a.overflow = overflow;
  return run_with<kSilu>(type, a, stream);
}

bool run_gated_mean(uint32_t type, const void* w, uint32_t hc, uint32_t dim, uint32_t cols, const void* x16, uint32_t n,
                    const float* xn, float* out, void* out16, uint32_t row0, int32_t* overflow, void* stream) {
  if (!w || !x16 || !xn || !out || out16 == x16 || (out16 && !overflow) || !n || n > MM_MAX_TOKENS || !hc ||
      hc > MM_GATED_MEAN_MAX_HC || !dim || dim % MM_TILE || (uint64_t) hc * dim > 0xFFFFFFFFull ||
      !shape_ok(type, hc * dim, cols) || ((uintptr_t) x16 & 15u))
    return false;
  Args a{};
  a.w = (const uint8_t*) w, a.x16 = (const __half*) x16, a.rows = hc * dim, a.cols = cols, a.n = n, a.xts = cols;
  a.scale = 1.0f, a.x16_out = (__half*) out16, a.overflow = overflow, a.xn = xn, a.out = out;
  a.hc = hc, a.dim = dim, a.out_row0 = row0;
  a.per = ((uint32_t) kM / hc) & ~(uint32_t) (MM_TILE - 1);  // whole tiles of 16 values: 128, 64, 32, 32, 16, ... for 1 - 8 streams
  return run_with<kGatedMean>(type, a, stream);
}

}  // namespace mm_tc
}  // namespace osmos

using namespace osmos;

extern "C" bool mm_known(uint32_t type) { return qtype_row(type) != nullptr; }
extern "C" bool mm_fits(uint32_t type, uint32_t rows, uint32_t cols) { return mm_tc::shape_ok(type, rows, cols); }
extern "C" uint32_t mm_col_tiles(uint32_t type, uint32_t n) {
  if (!qtype_row(type)) return 0;
  return n <= (uint32_t) mm_tc::kN ? 1u : n <= 2u * mm_tc::kN ? 2u : (uint32_t) mm_tc::kMaxAcc;
}
extern "C" uint32_t mm_status(void) {
  uint32_t* at = mm_tc::status_word();
  if (!at) return 0x80000000u;
  uint32_t v = 0, zero = 0;
  if (cudaMemcpy(&v, at, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return 0x80000000u;
  cudaMemcpy(at, &zero, sizeof zero, cudaMemcpyHostToDevice);
  return v | fp4_tc::read_status();  // (the block-scaled FP4 product's record beside the f16 product's)
}

extern "C" bool mm_run(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const void* x16, uint32_t n, float* y,
                       uint32_t ys, void* stream) {
  return mm_tc::run(type, w, rows, cols, x16, n, y, ys, 1.0f, stream);
}

extern "C" bool mm_run_silu(uint32_t type, const void* w, uint32_t rows, uint32_t cols, const void* x16, uint32_t n,
                            float* y, uint32_t ys, float scale, void* x16_out, int32_t* overflow, void* stream) {
  return mm_tc::run_silu(type, w, rows, cols, x16, n, y, ys, scale, x16_out, overflow, stream);
}

extern "C" bool mm_run_gated_mean(uint32_t type, const void* w, uint32_t hc, uint32_t dim, uint32_t cols, const void* x16,
                                  uint32_t n, const float* xn, float* out, void* out16, uint32_t row0, int32_t* overflow,
                                  void* stream) {
  return mm_tc::run_gated_mean(type, w, hc, dim, cols, x16, n, xn, out, out16, row0, overflow, stream);
}

extern "C" bool mm_run2(uint32_t type, const void* w0, uint32_t rows0, float* y0, uint32_t ys0, const void* w1,
                        uint32_t rows1, float* y1, uint32_t ys1, uint32_t cols, const void* x16, uint32_t n, void* stream) {
  if (!w0 || !w1 || !y0 || !y1 || !x16 || !n || n > MM_MAX_TOKENS || !mm_tc::shape_ok(type, rows0, cols) ||
      !mm_tc::shape_ok(type, rows1, cols) || (n > 1 && (ys0 < rows0 || ys1 < rows1)) || ((uintptr_t) x16 & 15u))
    return false;  // (decided for both before either is queued)
  return mm_tc::run(type, w0, rows0, cols, x16, n, y0, ys0, 1.0f, stream) &&
         mm_tc::run(type, w1, rows1, cols, x16, n, y1, ys1, 1.0f, stream);
}

extern "C" bool mm_tokens_scaled(uint32_t type, const void* w0, uint32_t rows0, float* y0, uint32_t ys0, float s0,
                                 const void* w1, uint32_t rows1, float* y1, uint32_t ys1, float s1, uint32_t cols,
                                 const float* x, uint32_t xs, uint32_t n, void* x16, int32_t* overflow, bool ready,
                                 void* stream) {
  if (!w0 || !y0 || !x || !x16 || !overflow || !n || !mm_tc::shape_ok(type, rows0, cols) || (n > 1 && (xs < cols || ys0 < rows0)))
    return false;
  if (w1 && (!y1 || !mm_tc::shape_ok(type, rows1, cols) || (n > 1 && ys1 < rows1))) return false;
  if ((uintptr_t) x16 & 15u) return false;
  for (uint32_t t0 = 0; t0 < n; t0 += MM_MAX_TOKENS) {  // MM_MAX_TOKENS a time through the one x16
    const uint32_t c = n - t0 < MM_MAX_TOKENS ? n - t0 : MM_MAX_TOKENS;
    if (!(ready && n <= MM_MAX_TOKENS) && !mm_x16(x + (uint64_t) t0 * xs, xs, c, cols, x16, overflow, stream)) return false;
    if (!mm_tc::run(type, w0, rows0, cols, x16, c, y0 + (uint64_t) t0 * ys0, ys0, s0, stream)) return false;
    if (w1 && !mm_tc::run(type, w1, rows1, cols, x16, c, y1 + (uint64_t) t0 * ys1, ys1, s1, stream)) return false;
  }
  return true;
}

extern "C" bool mm_tokens(uint32_t type, const void* w0, uint32_t rows0, float* y0, uint32_t ys0, const void* w1,
                          uint32_t rows1, float* y1, uint32_t ys1, uint32_t cols, const float* x, uint32_t xs, uint32_t n,
                          void* x16, int32_t* overflow, bool ready, void* stream) {
  return mm_tokens_scaled(type, w0, rows0, y0, ys0, 1.0f, w1, rows1, y1, ys1, 1.0f, cols, x, xs, n, x16, overflow, ready, stream);
}

extern "C" bool mm_group(uint32_t type, const void* const* w, const int32_t* cnt, uint32_t n_mat, uint32_t max_cnt,
                         uint32_t rows, uint32_t cols, const void* x16, const uint32_t* xoff, uint32_t xts, float* y,
                         const uint32_t* yoff, uint32_t ys, void* stream) {
  if (!w || !cnt || !x16 || !xoff || !y || !yoff || !n_mat || n_mat > 65535 || !max_cnt || max_cnt > MM_MAX_TOKENS ||
      !mm_tc::shape_ok(type, rows, cols) || xts < cols || xts % MM_TILE || ys < rows || ((uintptr_t) x16 & 15u))
    return false;
  mm_tc::Args a{};
  a.wt = (const uint8_t* const*) w, a.cnt = cnt, a.xoff = xoff, a.yoff = yoff, a.x16 = (const __half*) x16, a.y = y;
  a.rows = rows, a.cols = cols, a.xts = xts, a.ys = ys, a.scale = 1.0f;
#define CASE(T) return mm_tc::launch<T>(a, n_mat, max_cnt, stream_of(stream));
  OSMOS_SWITCH_QUANT(type, CASE, return false)
#undef CASE
}
