// Q4_K x int8 on the 5th-generation tensor cores (include/osmos_b200/mmq.h): tcgen05.mma kind::i8 with the int32
// group dots in tensor memory, drained group by group into the contract's F32 epilogue.
//
// A block computes 128 weight rows x 128 tokens of one matrix. Twenty warps, four roles:
//   loader (1 warp)       per 256-value step: the rows' raw 144-byte blocks by 16-byte cp.async into a ring of three
//   producers (2 warps)   per 256-value step: unpack the rows' Q4_K nibbles of that superblock into int8 operand
//                         tiles (one 128 x 32 tile a 32-value group, K-major core matrices of 8 rows x 16 bytes),
//                         copy the tokens' int8 codes into the same layout (cp.async), and their dx / sx beside them; then a
//                         proxy fence and an arrive on the stage's "full" mbarrier. Two stages deep.
//   issuer (1 warp)       per group one tcgen05.mma M128 N128 K32 that OVERWRITES one of four 128-column accumulators
//                         in tensor memory, then tcgen05.commit onto that accumulator's "full" mbarrier; after a
//                         step's eight groups a commit onto the stage's "empty" mbarrier (which also counts the sixteen
//                         epilogue warps: they still read the stage's dx / -sx after the tensor core is done).
//   epilogue (16 warps)   thread = one weight row (its TMEM lane) x 32 tokens: tcgen05.ld the group's int32 dots,
//                         acc = fmaf((d sc) dx, (float) I, acc); acc = fmaf(dmin m, -sx, acc) in the contract's order.
//                         The K loop runs partition by partition (256-value blocks p, p + 4, ...), and at the end of
//                         partition p the thread's sums go to y (p = 0) or are added to it (p > 0): the reference's
//                         "partitions added in order", with y as the running sum.
// The integer dots are exact whatever computes them, and every F32 operation is the generic kernel's (mmq.cu), so
// the two give the same bits. The epilogue, not the tensor pipe, sets the pace: every 32-value group's dot leaves
// tensor memory on its own and meets five CUDA-core instructions an element.
//
// Every mbarrier wait is bounded (%globaltimer); a wait that runs out raises the status word, every role falls
// through to the common exit and tensor memory is released.
#include "common.cuh"
#include "mmq_tc_api.h"
#include "osmos_b200/mmq.h"

namespace osmos {
namespace mmq_tc {
namespace {

constexpr int kM = 128, kNMax = 128;           // rows a block, and the most tokens (a block takes 128, 64 or 32: kN)
constexpr int kEpiWarps = 16, kProdWarps = 2;
constexpr int kIssuerWarp = kEpiWarps;         // warp 16
constexpr int kLoaderWarp = kEpiWarps + 1;     // warp 17: the rows' raw blocks, by bulk copies
constexpr int kFirstProdWarp = kEpiWarps + 2;  // warps 18, 19
constexpr int kProdThreads = kProdWarps * kWarp;
constexpr int kThreads = (kEpiWarps + 2 + kProdWarps) * kWarp;
constexpr int kStages = 2, kRawStages = 3, kAccs = 4;
constexpr int kGroups = 8, kBlockBytes = 144, kBlockValues = 256;
constexpr int kTileBytes = kM * MMQ_GROUP;     // one operand tile: 128 rows x 32 int8 = 4 KB
constexpr int kHeadOff = 2 * kGroups * kTileBytes + 2 * kGroups * kNMax * 4;  // after A, B, dx, sx: the rows' 16-byte block heads
constexpr int kStageBytes = kHeadOff + kM * 16;                            // 74 KB
constexpr int kRawBytes = kM * kBlockBytes;    // a step's raw blocks, a row's after another: 18 KB
constexpr uint64_t kWaitLimitNs = 200ull * 1000 * 1000;

__device__ uint32_t g_status;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = smem_addr(bar);
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; spin++) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(a), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin == 0) t0 = global_ns();
    else if (global_ns() - t0 > kWaitLimitNs) return false;
  }
}

// packed F32 pairs: one instruction, two IEEE operations
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// 16 bytes global -> shared, asynchronously (both 16-byte aligned)
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}

// shared-memory matrix descriptor of one operand tile: K-major, no swizzle, core matrices of 8 rows x 16 bytes;
// the next 16 bytes of K are 128 bytes on (leading offset), the next 8 rows 256 bytes on (stride offset)
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) (lbo_bytes >> 4) << 16 | (uint64_t) (sbo_bytes >> 4) << 32 |
         (uint64_t) 1 << 46;
}
// instruction descriptor: D int32, A unsigned 8-bit (the nibbles), B signed 8-bit, both K-major, N = 128, M = 128
__host__ __device__ constexpr uint32_t idesc_for(int n) { return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (kM >> 4) << 24); }

struct Args {
  const uint8_t* const* wt;
  const int32_t* cnt;
  const int8_t* x8;
  const float *dx, *sx;
  const uint32_t *soff, *yoff;
  float* y;
  uint32_t cols, ys;
  uint32_t* status;
};

struct Shared {
  uint64_t full[kStages], empty[kStages], acc_full[kAccs], acc_empty[kAccs], raw_full[kRawStages], raw_empty[kRawStages];
  uint32_t tmem_base;
  int fail;
};

// kN: tokens a block (its accumulators' width): narrower blocks when the launch has few, so the grid still fills the GPU -
// an element's sums do not depend on it
template <int kN>
__global__ void __launch_bounds__(kThreads, 1) q4k_tc_kernel(const Args a) {
  constexpr int kCols = kN / (kEpiWarps / 4);  // tokens an epilogue thread: 32, 16 or 8
  constexpr uint32_t kIdesc = idesc_for(kN);
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ Shared sh;
  const uint32_t tid = threadIdx.x, lane = tid % kWarp, warp = tid / kWarp;
  const uint32_t m = blockIdx.y, n_tok = (uint32_t) a.cnt[m], row0 = blockIdx.x * kM, c0 = blockIdx.z * kN;
  if (c0 >= n_tok) return;  // the whole block, before anything is allocated
  if ((uintptr_t) a.wt[m] & 15u) {  // the rows' blocks come by 16-byte-aligned bulk copies: the block stands down
    if (tid == 0) atomicOr(a.status, 2u);
    return;
  }
  const uint32_t n_valid = n_tok - c0 < (uint32_t) kN ? n_tok - c0 : (uint32_t) kN;
  const uint32_t n_valid16 = (n_valid + 15u) & ~15u;
  const uint32_t nb = a.cols / kBlockValues, groups = a.cols / MMQ_GROUP;
  const uint64_t row_bytes = (uint64_t) nb * kBlockBytes;
  const uint8_t* w = a.wt[m] + (uint64_t) row0 * row_bytes;
  const uint32_t s0 = a.soff[m] + c0;  // the block's first slot: a multiple of 16

  if (tid == 0) {
    for (int i = 0; i < kStages; i++) bar_init(&sh.full[i], 2 * kProdThreads), bar_init(&sh.empty[i], 1 + kEpiWarps);
    for (int i = 0; i < kAccs; i++) bar_init(&sh.acc_full[i], 1), bar_init(&sh.acc_empty[i], kEpiWarps);
    for (int i = 0; i < kRawStages; i++) bar_init(&sh.raw_full[i], kWarp), bar_init(&sh.raw_empty[i], kProdThreads);
    sh.fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == (uint32_t) kIssuerWarp) {  // all of tensor memory: four accumulators of 128 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sh.tmem_base)), "r"(kAccs * kN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sh.tmem_base;

  // the K loop's order: partition p's blocks p, p + 4, ... for p = 0 .. 3; step `it` of it
  auto block_of = [&](uint32_t it, uint32_t& p, bool& last_of_p) -> uint32_t {
    uint32_t left = it;
    for (p = 0; p < 4; p++) {
      const uint32_t in_p = nb > p ? (nb - p + 3) / 4 : 0;
      if (left < in_p) {
        last_of_p = left + 1 == in_p;
        return p + 4 * left;
      }
      left -= in_p;
    }
    last_of_p = true;
    return 0;
  };

  uint8_t* const raw = smem + kStages * kStageBytes;  // the raw ring
  if (warp == (uint32_t) kLoaderWarp) {
    // ================= the rows' raw blocks =================
    // a step's 144-byte block of each of the tile's 128 rows, as far ahead as the raw ring is deep:
    // the trip to memory is over when the producers want the bytes
    for (uint32_t it = 0; it < nb; it++) {
      const uint32_t rs = it % kRawStages, use = it / kRawStages;
      if (use > 0 && !bar_wait(&sh.raw_empty[rs], (use - 1) & 1u)) {
        sh.fail = 1;
        break;
      }
      uint32_t p;
      bool last;
      const uint32_t b = block_of(it, p, last);
      // 16-byte asynchronous copies, nine a row (a bulk copy a row was the slowest thing in the kernel: 128 small requests
      // a step took the copy engine 4.4 us); nobody waits for them: the ring's barrier hears of their landing, an
      // arrival a lane
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      uint8_t* dst = raw + rs * kRawBytes;
      const uint8_t* src = w + (uint64_t) b * kBlockBytes;
      for (uint32_t i = lane; i < (uint32_t) (kM * (kBlockBytes / 16)); i += kWarp) {
        const uint32_t r = i / (kBlockBytes / 16), piece = i % (kBlockBytes / 16);
        cp_async16(dst + r * kBlockBytes + piece * 16, src + r * row_bytes + piece * 16);
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&sh.raw_full[rs])) : "memory");
    }
  } else if (warp >= (uint32_t) kFirstProdWarp) {
    // ================= producers =================
    const uint32_t pt = tid - kFirstProdWarp * kWarp;  // 0 .. kProdThreads - 1
    for (uint32_t it = 0; it < nb; it++) {
      const uint32_t stage = it % kStages, use = it / kStages;
      if (use > 0 && !bar_wait(&sh.empty[stage], (use - 1) & 1u)) {
        sh.fail = 1;
        break;
      }
      uint32_t p;
      bool last;
      const uint32_t b = block_of(it, p, last);
      uint8_t* st = smem + stage * kStageBytes;
      uint8_t* sa = st;                              // A tiles, a group 4 KB
      uint8_t* sb = st + kGroups * kTileBytes;       // B tiles
      float* sdx = (float*) (st + 2 * kGroups * kTileBytes);
      float* ssx = sdx + kGroups * kN;
      // B, dx, sx: asynchronous 16-byte copies straight to their places (no registers, all in flight at once): the
      // tokens' codes in the order they lie in x8 (slot tile, group, slot, half), 16 floats of dx / sx a (tile, group)
      {
        const uint32_t limit = (n_valid16 / 16) * kGroups * 32;
        for (uint32_t i = pt; i < limit; i += kProdThreads) {
          const uint32_t half = i & 1u, sl = (i >> 1) & 15u, g = (i >> 5) & 7u, tile = i >> 8, n = tile * 16 + sl;
          cp_async16(sb + g * kTileBytes + (n >> 3) * 256 + half * 128 + (n & 7u) * 16,
                     a.x8 + mmq_x8_at(s0 + n, (b * kGroups + g) * MMQ_GROUP + half * 16, a.cols));
        }
        const uint32_t limit2 = (n_valid16 / 16) * kGroups * 4 * 2;  // (tile, group, quarter, dx | sx)
        for (uint32_t i = pt; i < limit2; i += kProdThreads) {
          const uint32_t which = i & 1u, qt = (i >> 1) & 3u, g = (i >> 3) & 7u, tile = i >> 6;
          const uint64_t at = mmq_dx_at(s0 + tile * 16 + qt * 4, b * kGroups + g, groups);
          cp_async16((which ? ssx : sdx) + g * kN + tile * 16 + qt * 4, (which ? a.sx : a.dx) + at);
        }
        // nobody waits for these copies: the stage's barrier hears of their landing (an arrival a thread, not counted
        // as one of the expected ones until it happens)
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&sh.full[stage])) : "memory");
      }
      // A: the step's raw blocks have landed; a task = (row, pair of groups): 32 bytes of nibbles -> the low nibbles'
      // group and the high nibbles' group
      const uint32_t rs = it % kRawStages;
      if (!bar_wait(&sh.raw_full[rs], (it / kRawStages) & 1u)) {
        sh.fail = 1;
        break;
      }
      const uint8_t* rawb = raw + rs * kRawBytes;
#pragma unroll 2
      for (uint32_t task = pt; task < 4u * kM; task += kProdThreads) {
        const uint32_t row = task >> 2, gp = task & 3u;
        const uint4* src = (const uint4*) (rawb + row * kBlockBytes + 16 + gp * 32);
        const uint4 r0 = src[0], r1 = src[1];
        const uint32_t at = (row >> 3) * 256 + (row & 7u) * 16;
        uint8_t* lo = sa + (2 * gp) * kTileBytes + at;
        uint8_t* hi = sa + (2 * gp + 1) * kTileBytes + at;
        const uint32_t k = 0x0F0F0F0Fu;
        *(uint4*) lo = make_uint4(r0.x & k, r0.y & k, r0.z & k, r0.w & k);
        *(uint4*) (lo + 128) = make_uint4(r1.x & k, r1.y & k, r1.z & k, r1.w & k);
        *(uint4*) hi = make_uint4((r0.x >> 4) & k, (r0.y >> 4) & k, (r0.z >> 4) & k, (r0.w >> 4) & k);
        *(uint4*) (hi + 128) = make_uint4((r1.x >> 4) & k, (r1.y >> 4) & k, (r1.z >> 4) & k, (r1.w >> 4) & k);
      }
      for (uint32_t r = pt; r < (uint32_t) kM; r += kProdThreads)  // the rows' d, dmin and packed scales, for the epilogue
        *(uint4*) (st + kHeadOff + r * 16) = *(const uint4*) (rawb + r * kBlockBytes);
      bar_arrive(&sh.raw_empty[rs]);  // (this thread has read its part of the raw blocks)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these writes before the tensor core's reads
      bar_arrive(&sh.full[stage]);
    }
  } else if (warp == (uint32_t) kIssuerWarp) {
    // ================= issuer =================
    uint32_t acc_it = 0;
    for (uint32_t it = 0; it < nb && !sh.fail; it++) {
      const uint32_t stage = it % kStages, use = it / kStages;
      if (!bar_wait(&sh.full[stage], use & 1u)) {
        sh.fail = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // (the tokens' codes came by cp.async)
      const uint32_t sa = smem_addr(smem + stage * kStageBytes), sb = sa + kGroups * kTileBytes;
      for (uint32_t g = 0; g < (uint32_t) kGroups; g++, acc_it++) {
        const uint32_t acc = acc_it % kAccs, ause = acc_it / kAccs;
        if (ause > 0 && !bar_wait(&sh.acc_empty[acc], (ause - 1) & 1u)) {
          sh.fail = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) {
          const uint64_t da = tile_desc(sa + g * kTileBytes, 128, 256), db = tile_desc(sb + g * kTileBytes, 128, 256);
          asm volatile(
              "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(
                  tmem + acc * kN),
              "l"(da), "l"(db), "r"(kIdesc), "r"(0)
              : "memory");
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           smem_addr(&sh.acc_full[acc]))
                       : "memory");
        }
        __syncwarp();
      }
      if (sh.fail) break;
      if (lane == 0)  // the stage's operands are free once these eight have run
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                         smem_addr(&sh.empty[stage]))
                     : "memory");
      __syncwarp();
    }
  } else {
    // ================= epilogue =================
    const uint32_t row = 32u * (warp & 3u) + lane;  // this thread's weight row of the tile = its TMEM lane
    const uint32_t col0 = (uint32_t) kCols * (warp >> 2);  // its 32 tokens
    const uint32_t lane_base = tmem + ((32u * (warp & 3u)) << 16);
    float* y = a.y + a.yoff[m] + (uint64_t) c0 * a.ys + row0 + row;
    uint64_t acc[kCols / 2];  // the thread's 32 sums, two neighbouring tokens a register pair
#pragma unroll
    for (int i = 0; i < kCols / 2; i++) acc[i] = 0ull;
    uint32_t acc_it = 0;
    bool dead = false;
    // sixteen tokens' int32 dots of this thread's row out of tensor memory (asynchronous: tcgen05.wait::ld before use;
    // the kernel must build without register spills, a spilled destination would be saved before its value lands)
    auto load16 = [](uint32_t (&r)[16], uint32_t at) {
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
            "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
          : "r"(at)
          : "memory");
    };
    auto load8 = [](uint32_t (&r)[16], uint32_t at) {
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                   : "r"(at)
                   : "memory");
    };
    // NV of them (16 or 8) into the sums, two tokens an instruction (packed F32: each half is the scalar operation, same
    // rounding)
    auto sums = [](auto nv_tag, const uint32_t (&r)[16], uint64_t dsc2, uint64_t ndm2, const float* dx, const float* ns, uint64_t* acc8) {
      constexpr int NV = decltype(nv_tag)::value;
      const ulonglong2* dx4 = (const ulonglong2*) dx;
      const ulonglong2* ns4 = (const ulonglong2*) ns;
      const uint64_t bias2 = pack2(-12582912.0f, -12582912.0f);
#pragma unroll
      for (int q = 0; q < NV / 4; q++) {
        const ulonglong2 dv = dx4[q], nv = ns4[q];
        const uint64_t dxs[2] = {dv.x, dv.y}, nss[2] = {nv.x, nv.y};
#pragma unroll
        for (int e = 0; e < 2; e++) {
          // (float) I without the conversion pipe: |I| <= 32 * 15 * 127 < 2^22, so 1.5 * 2^23 + I is exact
          const uint64_t f = add2(pack2(__int_as_float((int) r[4 * q + 2 * e] + 0x4B400000),
                                        __int_as_float((int) r[4 * q + 2 * e + 1] + 0x4B400000)),
                                  bias2);
          const uint64_t v = mul2(dsc2, dxs[e]);
          acc8[2 * q + e] = fma2(ndm2, nss[e], fma2(v, f, acc8[2 * q + e]));
        }
      }
    };
    for (uint32_t it = 0; it < nb && !dead; it++) {
      const uint32_t stage = it % kStages;
      uint32_t p;
      bool last;
      block_of(it, p, last);
      // the row's scales of this block: d sc and dmin m for its 8 groups, from the head the producers kept in the stage
      // (read once the stage is full: this thread may be a whole step ahead of the producers)
      if (!bar_wait(&sh.full[stage], (it / kStages) & 1u)) {
        sh.fail = 1;
        break;
      }
      const uint4 hd = *(const uint4*) (smem + stage * kStageBytes + kHeadOff + row * 16);
      const float d = half_value(hd.x & 0xFFFFu), dmin = half_value(hd.x >> 16);
      const uint32_t sw[3] = {hd.y, hd.z, hd.w};
      auto sbyte = [&](int i) -> uint32_t { return (sw[i >> 2] >> (8 * (i & 3))) & 0xFFu; };
      const float* sdx = (const float*) (smem + stage * kStageBytes + 2 * kGroups * kTileBytes);
      const float* ssx = sdx + kGroups * kN;
#pragma unroll
      for (uint32_t g = 0; g < (uint32_t) kGroups; g++, acc_it++) {
        uint32_t sc, mn;
        if (g < 4) sc = sbyte(g) & 0x3F, mn = sbyte(g + 4) & 0x3F;
        else sc = (sbyte(g + 4) & 0x0F) | ((sbyte(g - 4) >> 6) << 4), mn = (sbyte(g + 4) >> 4) | ((sbyte(g) >> 6) << 4);
        const float dsc = mul_rn(d, (float) sc), ndm = -mul_rn(dmin, (float) mn);  // (dmin m) (-sx) = (-(dmin m)) sx
        const uint32_t ab = acc_it % kAccs, ause = acc_it / kAccs;
        const uint64_t dsc2 = pack2(dsc, dsc), ndm2 = pack2(ndm, ndm);
        if (!bar_wait(&sh.acc_full[ab], ause & 1u)) {
          sh.fail = 1, dead = true;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t ra[16], rb[16];
        if constexpr (kCols == 8) {
          load8(ra, lane_base + ab * kN + col0);
        } else {
          load16(ra, lane_base + ab * kN + col0);
          if constexpr (kCols == 32) load16(rb, lane_base + ab * kN + col0 + 16);
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // the accumulator is read: hand it back before the arithmetic (the tensor core runs four groups ahead at most,
        // and the slowest of the sixteen warps sets when it may reuse this one)
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) bar_arrive(&sh.acc_empty[ab]);
        sums(std::integral_constant<int, (kCols < 16 ? kCols : 16)>{}, ra, dsc2, ndm2, sdx + g * kN + col0, ssx + g * kN + col0, &acc[0]);
        if constexpr (kCols == 32) sums(std::integral_constant<int, 16>{}, rb, dsc2, ndm2, sdx + g * kN + col0 + 16, ssx + g * kN + col0 + 16, &acc[8]);
      }
      if (dead) break;
      __syncwarp();
      if (lane == 0) bar_arrive(&sh.empty[stage]);  // done with the stage's dx / -sx
      if (last) {  // partition p is complete: y = its sum (p = 0) or y + its sum
#pragma unroll
        for (int i = 0; i < kCols / 2; i++) {
          float pair[2];
          unpack2(acc[i], pair[0], pair[1]);
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const uint32_t t = col0 + 2 * i + h;
            if (t < n_valid) {
              float* at = y + (uint64_t) t * a.ys;
              *at = p == 0 ? pair[h] : __fadd_rn(*at, pair[h]);
            }
          }
          acc[i] = 0ull;
        }
      }
    }
    if (!dead && nb < 4) {  // the partitions without a block still take part in the sum: + 0 (it turns a -0 into +0)
#pragma unroll 1
      for (int i = 0; i < kCols; i++) {
        const uint32_t t = col0 + i;
        if (t < n_valid) {
          float* at = y + (uint64_t) t * a.ys;
          *at = __fadd_rn(*at, 0.0f);
        }
      }
    }
  }
  // ================= common exit =================
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == (uint32_t) kIssuerWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kAccs * kN));
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

}  // namespace

int try_launch(const void* const* w, const int32_t* cnt, uint32_t n_mat, uint32_t max_cnt, uint32_t rows, uint32_t cols,
               const int8_t* x8, const float* dx, const float* sx, const uint32_t* soff, float* y, const uint32_t* yoff,
               uint32_t ys, void* stream) {
  if (rows % kM || cols % kBlockValues || (((uintptr_t) x8 | (uintptr_t) dx | (uintptr_t) sx) & 15u)) return 0;
  uint32_t* status = status_word();
  if (!status) return 0;
  const int smem_bytes = kStages * kStageBytes + kRawStages * kRawBytes;
  Args a{(const uint8_t* const*) w, cnt, x8, dx, sx, soff, yoff, y, cols, ys, status};
  // the widest blocks that still make a grid of about a hundred (148 SMs, a block each): a slice of a matrix's rows, or
  // a few tokens, then takes narrower and therefore more and shorter blocks
  auto blocks = [&](uint32_t n) { return (uint64_t) (rows / kM) * n_mat * ((max_cnt + n - 1) / n); };
  auto go = [&](auto n_tag, bool (&sized)[64]) -> int {
    constexpr int N = decltype(n_tag)::value;
    if (!allow_dynamic_smem(q4k_tc_kernel<N>, smem_bytes, sized)) return 0;
    const dim3 grid(rows / kM, n_mat, (max_cnt + N - 1) / N);
    q4k_tc_kernel<N><<<grid, kThreads, smem_bytes, (cudaStream_t) stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
  };
  static bool sized128[64] = {}, sized64[64] = {}, sized32[64] = {};  // (one flag a device and an instance)
  if (blocks(128) >= 100) return go(std::integral_constant<int, 128>{}, sized128);
  if (blocks(64) >= 100) return go(std::integral_constant<int, 64>{}, sized64);
  return go(std::integral_constant<int, 32>{}, sized32);
}

uint32_t read_status() {
  uint32_t* at = status_word();
  if (!at) return 0x80000000u;
  uint32_t v = 0, zero = 0;
  if (cudaMemcpy(&v, at, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return 0x80000000u;
  cudaMemcpy(at, &zero, sizeof zero, cudaMemcpyHostToDevice);
  return v;
}

}  // namespace mmq_tc
}  // namespace osmos
