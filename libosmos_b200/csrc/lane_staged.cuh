// The int8 lane's staged kernel: persistent blocks, weight tiles brought into shared memory by the bulk-copy (TMA)
// engine through a two-stage mbarrier ring, every block of a tile decoded out of registers, codebooks replicated
// per lane so their lookups never collide in a bank.
//
// Work item = (entry, row tile, pair of tokens). A block walks its items in a fixed stride; a seventeenth warp issues
// the items' copies (the tile of gate rows, of up rows when fused, each live token's int8 row as 256-byte pieces, its
// scales) as many stages ahead as shared memory holds, and leaves each item's small facts (live tokens, output rows,
// routed weights) beside its stage, so the sixteen compute warps never wait on a global load.
//
// Per item, two phases:
//   A  a thread takes whole 256-value superblocks of the tile's flat byte stream (thread g: superblock g, two
//      neighbours in a warp two superblocks apart, so every window load is bank-conflict free and its 2-byte
//      alignment is the warp's, a template constant; of a fused pair a warp takes the gate's or the up's). It reads
//      the superblock as aligned 32-bit words into registers, decodes its eight 32-value sub-blocks and writes each
//      sub-block's value before x's scale (two exact integer half dots, then the contract's products) to shared
//      memory.
//   B  a thread is a lane of the contract: it runs the fmaf chain acc = fmaf(d_x, block, acc) over its blocks
//      l, l + L, ... in order, the L lanes of a row are combined by the xor tree, lane 0 stores the sum or the
//      activation of the gate and up sums.
// The split leaves phase A free to order its work for the memory system while phase B fixes the order of every
// floating-point operation, so the bits are those of the generic kernel (q8.cu) and of the CPU oracle.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets bit 0 of the status word (q8_status) and the block
// leaves without touching its outputs again.
#pragma once
#include <type_traits>

#include "decode.cuh"
#include "tma.cuh"

namespace osmos {
namespace staged {

using namespace tma;

constexpr int kComputeWarps = 16, kComputeThreads = kComputeWarps * kWarp;
constexpr int kThreads = kComputeThreads + kWarp, kWarps = kThreads / kWarp;  // + the warp that issues the copies
constexpr int kNT = 2;             // tokens an item carries
constexpr int kMaxStages = 6;
constexpr int kXPiece = 256 + 16;  // a token's 256 int8 of one superblock, padded so neighbours fall in other banks
constexpr uint32_t kListMax = 1024;  // entries whose live (entry, token pair) list a block builds at a time

// ---- the type's superblock: 256 values ---------------------------------------------------------------------------
template <uint32_t T> struct Super {
  static constexpr int bytes = Fmt<T>::bytes * (256 / Fmt<T>::values);
  static constexpr bool parity = bytes % 4 != 0;             // its start alternates between 0 and 2 mod 4
  static constexpr int words = parity ? (bytes + 2 + 3) / 4 : bytes / 4;
  static constexpr int subs = Fmt<T>::subs;                  // 8 for the 256-value types, 1 for the 32-value ones
};

// ---- replicated codebooks ----------------------------------------------------------------------------------------
template <uint32_t T> struct Rep {  // copies of the 64-bit grid / whether the 32-bit grid and the sign masks are used
  static constexpr int g64 = GridOf<T>::words64 == 256 ? 16 : GridOf<T>::words64 == 512 ? 8
                           : GridOf<T>::words64 == 1024 ? 4 : GridOf<T>::words64 == 2048 ? 2 : 0;
  static constexpr int g32 = GridOf<T>::words32 ? 32 : 0;
  static constexpr int mask = GridOf<T>::signs ? 8 : 0;  // copies of the (masks, +1 words) table, 16 bytes an entry
  static constexpr int bytes = GridOf<T>::words64 * g64 * 8 + GridOf<T>::words32 * g32 * 4 + 128 * mask * 16;
};

// the tables' addresses with this thread's copy already chosen (lane l reads copy l, l mod 16, ...: its own banks)
template <uint32_t T> struct RepLuts {
  uint32_t g64, g32, mask;
  __device__ __forceinline__ uint64_t grid64(uint32_t i) const {
    if constexpr (Rep<T>::g64 > 0) {
      const uint2 v = lds64(g64 + i * (Rep<T>::g64 * 8));
      return (uint64_t) v.x | (uint64_t) v.y << 32;
    } else {
      return 0;
    }
  }
  __device__ __forceinline__ uint32_t grid32(uint32_t i) const {
    if constexpr (Rep<T>::g32 > 0) return lds32(g32 + i * 128);
    else return 0;
  }
  __device__ __forceinline__ uint4 sign_masks4(uint32_t s7) const {
    if constexpr (Rep<T>::mask > 0) {
      const int4 m = lds128(mask + s7 * 128);
      return make_uint4((uint32_t) m.x, (uint32_t) m.y, (uint32_t) m.z, (uint32_t) m.w);
    } else {
      return make_uint4(0, 0, 0, 0);
    }
  }
};

// every word of a codebook read once, a thread's loads issued together (a first touch of the table costs a trip to
// L2: one trip, not one a copy), each written COPIES times side by side
template <int COPIES, class W>
__device__ __forceinline__ void replicate(W* dst, const W* src, int words, int threads) {
  constexpr int U = 4;
  for (int i0 = threadIdx.x; i0 < words; i0 += threads * U) {
    W v[U];
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = i0 + u * threads < words ? src[i0 + u * threads] : W(0);
#pragma unroll
    for (int u = 0; u < U; u++)
      if (i0 + u * threads < words) {
#pragma unroll
        for (int c = 0; c < COPIES; c++) dst[(i0 + u * threads) * COPIES + c] = v[u];
      }
  }
}

// the grids; returns where the sign masks' table starts
template <uint32_t T> __device__ inline uint8_t* build_grids(uint8_t* smem, int threads, RepLuts<T>& l) {
  const uint32_t lane = threadIdx.x % kWarp;
  l.g64 = l.g32 = l.mask = 0;
  if constexpr (Rep<T>::g64 > 0) {
    replicate<Rep<T>::g64>((uint64_t*) smem, global_grid64<T>(), GridOf<T>::words64, threads);
    l.g64 = smem_addr(smem) + (lane & (Rep<T>::g64 - 1)) * 8, smem += GridOf<T>::words64 * Rep<T>::g64 * 8;
  }
  if constexpr (Rep<T>::g32 > 0) {
    replicate<32>((uint32_t*) smem, osmos_grid_iq3xxs, GridOf<T>::words32, threads);
    l.g32 = smem_addr(smem) + lane * 4, smem += GridOf<T>::words32 * 32 * 4;
  }
  return smem;
}

template <uint32_t T> __device__ inline RepLuts<T> build_luts(uint8_t* smem, int threads = kThreads) {
  const uint32_t lane = threadIdx.x % kWarp;
  RepLuts<T> l;
  smem = build_grids<T>(smem, threads, l);
  if constexpr (Rep<T>::mask > 0) {
    uint4* d = (uint4*) smem;
    for (int i = threadIdx.x; i < 128 * 8; i += threads) {
      const uint32_t sg = osmos_ksigns[i / 8];
      const uint32_t m0 = byte_mask4(sg), m1 = byte_mask4(sg >> 4);
      d[i] = make_uint4(m0, m1, m0 & 0x01010101u, m1 & 0x01010101u);
    }
    l.mask = smem_addr(d) + (lane & 7) * 16;
  }
  return l;
}

// The same tables with the sign masks as 8-byte (m0, m1) entries in 16 copies (a half-warp's lanes each their own
// banks; an 8-byte read is half the shared-memory passes of the 16-byte one, the two "+ 1" words then cost an AND
// each): for the kernels whose every lane looks masks up at once. In the place of build_luts' 16 KB mask table; every
// thread of the block calls it (it ends on a barrier: the tables are complete when it returns).
template <uint32_t T> struct RepLuts2 : RepLuts<T> {
  uint32_t mask2;
  __device__ __forceinline__ uint2 sign_masks2(uint32_t s7) const { return lds64(mask2 + s7 * 128u); }
  __device__ __forceinline__ uint4 sign_masks4(uint32_t s7) const {
    const uint2 m = sign_masks2(s7);
    return make_uint4(m.x, m.y, m.x & 0x01010101u, m.y & 0x01010101u);
  }
};
template <uint32_t T> __device__ inline RepLuts2<T> build_luts2(uint8_t* smem, int threads) {
  RepLuts2<T> l;
  smem = build_grids<T>(smem, threads, l);
  l.mask2 = 0;
  if constexpr (Rep<T>::mask > 0) {
    const uint32_t lane = threadIdx.x % kWarp, base = smem_addr(smem);
    l.mask = base + (lane & 7u) * 16u;
    // a thread a quarter of an entry's copies: one byte read, four stores
    for (uint32_t i = threadIdx.x; i < 128u * 4u; i += (uint32_t) threads) {
      const uint32_t sg = osmos_ksigns[i / 4u], m0 = byte_mask4(sg), m1 = byte_mask4(sg >> 4);
#pragma unroll
      for (uint32_t c = 0; c < 4u; c++)
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(base + (i * 4u + c) * 8u), "r"(m0), "r"(m1) : "memory");
    }
    l.mask2 = base + (lane & 15u) * 8u;
  }
  __syncthreads();
  return l;
}

// ---- arguments and shared-memory plan ---------------------------------------------------------------------------------
struct Args {
  const uint8_t* w_dense;    // one matrix (tables NULL)
  const uint8_t* const* wg;  // the entries' matrices (gate, or the only one)
  const uint8_t* const* wu;  // fused: the entries' up matrices
  const int32_t *cnt, *xrow, *xin, *win;
  const int8_t* q;
  const float* d;
  const float* scale;
  float lim;
  float* out;
  uint32_t rows, cols, out_stride, n_entries, max_cnt, n_tok;
  uint32_t tile_rows, tiles;  // rows a tile, tiles a matrix
  uint32_t stages;            // the ring's depth
  uint32_t* status;
};

// an item's facts, written by the copy warp beside the item's stage before its copies are issued
struct Meta {
  uint32_t live;        // tokens of this item (1 .. kNT)
  uint32_t out_row;     // its first token's output row
  uint32_t row0, trows; // the tile's first row and its rows
  float scale[kNT];     // fused: each token's routed weight
};

struct Plan {  // byte offsets into dynamic shared memory; the same function on the host and the device
  uint32_t lut, bars, meta, list, stage0, stage_bytes, w_bytes, x_off, x_tok, dx_off, bs, bs_bytes, plane, total;
};

template <uint32_t T>
__host__ __device__ inline Plan make_plan(uint32_t cols, uint32_t tile_rows, int mats, uint32_t stages) {
  Plan p;
  const uint32_t nsb = cols / 256, nblk = cols / 32, row_bytes = nsb * Super<T>::bytes;
  uint32_t at = 0;
  p.lut = at, at += (Rep<T>::bytes + 127u) & ~127u;
  p.bars = at, at += 2 * kMaxStages * 8;  // full[], empty[]
  at = (at + 31u) & ~31u;
  p.meta = at, at += kMaxStages * 32;
  p.list = at, at += kListMax * 4 * 2;  // (entry, token pair) as 16 bits, at most 4 pairs an entry
  at = (at + 127u) & ~127u;
  p.w_bytes = (tile_rows * row_bytes + 15u) & ~15u;
  p.x_off = mats * p.w_bytes;
  p.x_tok = nsb * kXPiece;
  p.dx_off = p.x_off + kNT * p.x_tok;
  p.stage_bytes = (p.dx_off + kNT * nblk * 4 + 127u) & ~127u;
  p.plane = tile_rows * nblk / 32 * 36;  // floats of one (matrix, token) plane: 4 floats of padding every 32
  p.bs_bytes = mats * kNT * p.plane * 4;
  p.bs = at, at += p.bs_bytes;
  p.stage0 = at, at += stages * p.stage_bytes;
  p.total = at;
  return p;
}

// where sub-block value f (a float index into one (matrix, token) plane of the tile) is kept: 4 floats of padding after
// every 32, so that phase A's 32-byte writes (threads 16 floats apart) and phase B's reads (a lane a float) both
// spread over the banks
__device__ __forceinline__ uint32_t bs_at(uint32_t f) { return f + (f >> 5) * 4; }

template <uint32_t T, bool FUSED, bool DENSE>
__global__ void __launch_bounds__(kThreads, 1) lane_staged_kernel(const Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int M = FUSED ? 2 : 1;
  constexpr int SB = Super<T>::bytes;
  static_assert(sizeof(Meta) <= 32, "a stage's facts fit their slot");
  const uint32_t S = a.stages;
  const Plan p = make_plan<T>(a.cols, a.tile_rows, M, S);
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const bool producer = warp == (uint32_t) kComputeWarps;
  const uint32_t nsb = a.cols / 256, nblk = a.cols / 32, row_bytes = nsb * SB;
  const int L = a.cols >= 4096 ? 32 : 16;
  uint64_t* full = (uint64_t*) (smem + p.bars);
  uint64_t* empty = full + kMaxStages;
  Meta* metas = (Meta*) (smem + p.meta);
  uint16_t* list = (uint16_t*) (smem + p.list);
  const uint32_t bs_addr = smem_addr(smem + p.bs);
  __shared__ int s_live_pairs, s_fail;
  __shared__ int s_scan[kWarps];

  if (tid == 0) {
    for (uint32_t st = 0; st < S; st++) bar_init(&full[st], 1), bar_init(&empty[st], kComputeWarps);
    bar_init_fence();
    s_fail = 0;
  }
  const RepLuts<T> luts = build_luts<T>(smem + p.lut);
  __syncthreads();

  // an entry's tokens, never more than the launch's max_cnt
  auto live_count = [&](uint32_t m) -> uint32_t {
    if constexpr (DENSE) return a.n_tok;
    const int32_t c = a.cnt[m];
    return c <= 0 ? 0u : ((uint32_t) c < a.max_cnt ? (uint32_t) c : a.max_cnt);
  };
  // an item's facts and sources -> its stage; every lane of the copy warp. false: a matrix was not 16-byte aligned
  auto issue = [&](uint32_t m, uint32_t grp, uint32_t tile, uint32_t stage) -> bool {
    uint8_t* st = smem + p.stage0 + stage * p.stage_bytes;
    const uint32_t row0 = tile * a.tile_rows;
    const uint32_t trows = a.rows - row0 < a.tile_rows ? a.rows - row0 : a.tile_rows;
    const uint32_t wbytes = trows * row_bytes;
    const uint32_t cnt = live_count(m);
    const uint32_t t0 = grp * kNT, live = cnt - t0 < (uint32_t) kNT ? cnt - t0 : (uint32_t) kNT;
    const uint8_t* wg = (DENSE ? a.w_dense : a.wg[m]) + (uint64_t) row0 * row_bytes;
    const uint8_t* wu_ = wg;
    if constexpr (FUSED) wu_ = a.wu[m] + (uint64_t) row0 * row_bytes;
    if ((((uintptr_t) wg | (uintptr_t) wu_) & 15u) != 0) return false;  // a bulk copy needs 16-byte aligned sources
    const uint32_t r0 = (DENSE ? 0u : (uint32_t) a.xrow[m]) + t0;
    if constexpr (FUSED) {
      if (lane < live) metas[stage].scale[lane] = a.scale[a.win ? a.win[r0 + lane] : r0 + lane];  // token t's routed weight
      __syncwarp();
    }
    if (lane == 0) {
      metas[stage].live = live, metas[stage].out_row = r0, metas[stage].row0 = row0, metas[stage].trows = trows;
      bar_expect(&full[stage], M * wbytes + live * (a.cols + nblk * 4));
    }
    __syncwarp();
    if (lane == 0) bulk_load(st, wg, wbytes, &full[stage]);
    if constexpr (FUSED)
      if (lane == 1) bulk_load(st + p.w_bytes, wu_, wbytes, &full[stage]);
    for (uint32_t t = 0; t < live; t++) {
      const uint32_t r = r0 + t;
      const uint64_t xr = a.xin ? (uint64_t) (uint32_t) a.xin[r] : r;
      for (uint32_t i = lane; i < nsb; i += kWarp)
        bulk_load(st + p.x_off + t * p.x_tok + i * kXPiece, a.q + xr * a.cols + i * 256, 256, &full[stage]);
      if (lane == kWarp - 1) bulk_load(st + p.dx_off + t * nblk * 4, a.d + xr * nblk, nblk * 4, &full[stage]);
    }
    return true;
  };

  // ---- phase A for one superblock alignment (A: its start's byte offset in its first word) and one count of live
  // tokens (NTL): superblock g of matrix `mat`, all eight sub-blocks
  auto phase_a = [&](auto align_tag, auto live_tag, uint32_t st, uint32_t tile_sb, uint32_t mat, uint32_t g_first,
                     uint32_t g_step) {
    constexpr int A = decltype(align_tag)::value, NTL = decltype(live_tag)::value;
    for (uint32_t g = g_first; g < tile_sb; g += g_step) {
      const uint32_t r = g / nsb, i = g - r * nsb;
      const uint32_t xa = st + p.x_off + i * kXPiece;
      const uint32_t out = bs_addr + 4 * (mat * kNT * p.plane + bs_at(r * nblk + i * 8));
      WordWindow<Super<T>::words, A> win;
      const uint32_t src = st + mat * p.w_bytes + g * SB - A;
#pragma unroll
      for (int k = 0; k < Super<T>::words; k++) win.w[k] = lds32(src + 4 * k);
#pragma unroll
      for (int h = 0; h < 2; h++) {
        float v[NTL][4];
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
          LaneCodes c;
          lane_codes_rd<T>(win, 4 * h + jj, c, luts);
#pragma unroll
          for (int t = 0; t < NTL; t++) {
            const int4 lo = lds128(xa + t * p.x_tok + (4 * h + jj) * 32), hi = lds128(xa + t * p.x_tok + (4 * h + jj) * 32 + 16);
            const int x[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            v[t][jj] = lane_block_sum<T>(c, x);
          }
        }
#pragma unroll
        for (int t = 0; t < NTL; t++) sts128(out + 4 * (t * p.plane + 4 * h), v[t][0], v[t][1], v[t][2], v[t][3]);
      }
    }
  };

  // ---- the entries, a list's worth at a time -----------------------------------------------------------------------
  const uint32_t n_entries = DENSE ? 1u : a.n_entries;
  uint32_t it = 0;  // items this block has started, over every list: it names the stage and the barriers' phases
  for (uint32_t e0 = 0; e0 < n_entries; e0 += kListMax) {
    // the live (entry, token pair) list of entries e0 .. e0 + kListMax, in entry order (every warp takes part)
    const uint32_t en = n_entries - e0 < kListMax ? n_entries - e0 : kListMax;
    __syncthreads();
    uint32_t run = 0;  // pairs before this round of threads
    for (uint32_t base = 0; base < en; base += kThreads) {
      const uint32_t m = base + tid;
      uint32_t mine = 0;
      if (m < en) mine = (live_count(e0 + m) + kNT - 1) / kNT;
      uint32_t inc = mine;
#pragma unroll
      for (int o = 1; o < kWarp; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o, kWarp);
        if (lane >= (uint32_t) o) inc += up;
      }
      if (lane == kWarp - 1) s_scan[warp] = (int) inc;
      __syncthreads();
      uint32_t before = run, all = 0;
      for (uint32_t wv = 0; wv < (uint32_t) kWarps; wv++) {
        if (wv < warp) before += (uint32_t) s_scan[wv];
        all += (uint32_t) s_scan[wv];
      }
      const uint32_t pos = before + inc - mine;
      for (uint32_t gq = 0; gq < mine; gq++) list[pos + gq] = (uint16_t) (m | gq << 12);
      run += all;
      __syncthreads();
    }
    if (tid == 0) s_live_pairs = (int) run;
    __syncthreads();
    const uint32_t items = (uint32_t) s_live_pairs * a.tiles;

    auto decode_item = [&](uint32_t q, uint32_t& m, uint32_t& grp, uint32_t& tile) {
      const uint32_t pair = q / a.tiles;
      tile = q - pair * a.tiles;
      const uint32_t v = list[pair];
      m = e0 + (v & 0x0FFFu), grp = v >> 12;
    };

    if (producer) {
      // ---- the copy warp: up to S stages ahead of the compute warps ----
      for (uint32_t q = blockIdx.x; q < items; q += gridDim.x, it++) {
        const uint32_t stage = it % S, use = it / S;
        bool ok = true;
        if (use > 0) ok = bar_wait(&empty[stage], (use - 1u) & 1u);  // the stage's last readers are done with it
        uint32_t m, grp, tile;
        decode_item(q, m, grp, tile);
        const bool aligned = ok && issue(m, grp, tile, stage);
        if (!ok || !aligned) {  // give up: the compute warps' wait runs out and they leave too
          if (lane == 0) atomicOr(a.status, ok ? 2u : 1u), s_fail = 1;
          return;
        }
      }
    } else {
      // ---- the compute warps ----
      // which superblocks of a tile this warp takes: see the header
      uint32_t mat = 0, g_first, g_step;
      const uint32_t par = Super<T>::parity ? (warp & 1u) : 0u;
      {
        const uint32_t w2 = Super<T>::parity ? warp >> 1 : warp;                 // the warp's index among its phase's
        const uint32_t span = Super<T>::parity ? 64u : 32u;                      // superblocks a warp pair / a warp covers
        const uint32_t first = Super<T>::parity ? 2u * lane + par : lane;
        const uint32_t nw = Super<T>::parity ? kComputeWarps / 2 : kComputeWarps;  // such warps
        if constexpr (FUSED) {
          mat = w2 & 1u;
          g_first = first + span * (w2 >> 1), g_step = span * (nw / 2);
        } else {
          g_first = first + span * w2, g_step = span * nw;
        }
      }
      for (uint32_t q = blockIdx.x; q < items; q += gridDim.x, it++) {
        const uint32_t stage = it % S, use = it / S;
        if (!bar_wait(&full[stage], use & 1u)) s_fail = 1;  // a copy never landed
        const uint32_t st = smem_addr(smem + p.stage0 + stage * p.stage_bytes);
        const Meta meta = metas[stage];
        const uint32_t live = meta.live, tile_sb = meta.trows * nsb;
        if (!s_fail) {
          using I0 = std::integral_constant<int, 0>;
          using I1 = std::integral_constant<int, 1>;
          using I2 = std::integral_constant<int, 2>;
          if (par) {
            if constexpr (Super<T>::parity) {
              if (live == 2) phase_a(I2{}, I2{}, st, tile_sb, mat, g_first, g_step);
              else phase_a(I2{}, I1{}, st, tile_sb, mat, g_first, g_step);
            }
          } else {
            if (live == 2) phase_a(I0{}, I2{}, st, tile_sb, mat, g_first, g_step);
            else phase_a(I0{}, I1{}, st, tile_sb, mat, g_first, g_step);
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
        if (s_fail) {  // set before the barrier by whoever gave up: every compute warp sees it here and leaves
          if (tid == 0) atomicOr(a.status, 1u);
          return;
        }

        // ---- phase B: the contract's lanes ----
        const uint32_t lanes_total = meta.trows * (uint32_t) L;
        for (uint32_t vl = tid; vl < lanes_total; vl += kComputeThreads) {
          const uint32_t r = vl / (uint32_t) L, ll = vl % (uint32_t) L;
#pragma unroll
          for (int t = 0; t < kNT; t++) {
            if ((uint32_t) t < live) {
              const uint32_t dxa = st + p.dx_off + (uint32_t) t * nblk * 4;
              const uint32_t pg = bs_addr + 4 * (uint32_t) t * p.plane;
              const uint32_t pu = bs_addr + 4 * (uint32_t) (kNT + t) * p.plane;
              float ag = 0.0f, au = 0.0f;
              for (uint32_t s = ll; s < nblk; s += (uint32_t) L) {
                const float dv = ldsf(dxa + 4 * s);
                const uint32_t at = 4 * bs_at(r * nblk + s);
                ag = __fmaf_rn(dv, ldsf(pg + at), ag);
                if constexpr (FUSED) au = __fmaf_rn(dv, ldsf(pu + at), au);
              }
#pragma unroll
              for (int o = 16; o > 0; o >>= 1)
                if (o < L) {
                  ag = __fadd_rn(ag, __shfl_xor_sync(0xFFFFFFFFu, ag, o, kWarp));
                  if constexpr (FUSED) au = __fadd_rn(au, __shfl_xor_sync(0xFFFFFFFFu, au, o, kWarp));
                }
              if (ll == 0) {
                const uint64_t ro = (uint64_t) meta.out_row + (uint32_t) t;
                if constexpr (FUSED) a.out[ro * a.out_stride + meta.row0 + r] = lane_swiglu(ag, au, a.lim, meta.scale[t]);
                else a.out[ro * a.out_stride + meta.row0 + r] = ag;
              }
            }
          }
        }
        // this warp is done with the stage (its scales were the last thing read) ...
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&empty[stage])) : "memory");
        // ... and every warp with the sub-block values before the next item overwrites them
        asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
      }
    }
  }
}

}  // namespace staged
}  // namespace osmos
